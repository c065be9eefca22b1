"""Every (source, macro definitions) pair the package can ask for; `build()` compiles them all."""

# Kernels specialised by head size are compiled for the sizes listed here ahead of time; any
# other multiple of 16 up to 256 is compiled the first time a model asks for it.
PREBUILT_HEAD_DIMS = (16, 32, 48, 64, 128)
PER_HEAD_DIM = ("attn_decode", "attn_prefill", "attn_decode_noalloc")
TC5_HEAD_DIMS = {"attn_prefill_tc5": (64, 128)}      # kernels that exist for these head sizes only


def all_variants():
    from . import build
    jobs = []
    for name in build.all_sources():
        if name in TC5_HEAD_DIMS:
            jobs += [(name, {"HEAD_DIM": hd}) for hd in TC5_HEAD_DIMS[name]]
        elif name in PER_HEAD_DIM:
            jobs += [(name, {"HEAD_DIM": hd}) for hd in PREBUILT_HEAD_DIMS]
        else:
            jobs.append((name, None))
    return jobs
