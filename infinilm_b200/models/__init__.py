from .causal_lm import CausalLM
