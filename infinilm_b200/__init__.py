"""infinilm_b200: a small, whole inference engine for one GPU (B200, sm_100a), built for the
MiniCPM4 architecture out of parts that other architectures can reuse."""
__version__ = "0.1.0"
