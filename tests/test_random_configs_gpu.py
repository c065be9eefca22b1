"""Random configurations of the architecture through the engine: every size drawn anew (heads and groups, head sizes in
steps of 16 up to 256, widths, intermediate sizes and vocabularies that are no power of two and no multiple of 16,
layers, eps, scale factors, biases, plain / partial / long rotary encodings, tied or own head, storage dtype), each
compared with the plain implementation in float32 and bfloat16: the prompt in two portions, then single tokens, eagerly
and replayed as graphs. A size that a kernel cannot take must be refused or take another path, never give a wrong row."""
import random

import pytest
import torch

from replay_util import TOL, build_engine, first_bad_row, plain_logits
from tiny_configs import make_weights, random_ids

pytestmark = pytest.mark.gpu


def random_config(seed: int) -> dict:
    rng = random.Random(1000 + seed)
    hd = rng.choice([16, 32, 48, 64, 80, 96, 112, 128, 256])
    nkv = rng.choice([1, 2, 3])
    group = rng.choice([1, 2, 3, 5, 8, 17]) if hd <= 128 else rng.choice([1, 2])
    nh = nkv * group
    hidden = 8 * rng.randint(5, 40)
    raw = {
        "architectures": ["MiniCPMForCausalLM"], "model_type": "minicpm4",
        "num_hidden_layers": rng.randint(1, 3), "hidden_size": hidden, "num_attention_heads": nh, "num_key_value_heads": nkv,
        "head_dim": hd, "intermediate_size": 8 * rng.randint(9, 60), "vocab_size": rng.randint(97, 700),
        "rope_theta": rng.choice([1e4, 5e4, 1e6]), "max_position_embeddings": 256,
        "scale_emb": round(rng.uniform(1, 12), 2), "dim_model_base": rng.choice([hidden, hidden // 2, 32]),
        "scale_depth": round(rng.uniform(0.8, 2.0), 2), "rms_norm_eps": rng.choice([1e-6, 1e-5, 1e-4]),
        "tie_word_embeddings": rng.random() < 0.5, "torch_dtype": rng.choice(["float32", "bfloat16"]),
    }
    kind = rng.choice(["plain", "partial", "longrope"])
    if kind == "partial":
        raw["partial_rotary_factor"] = rng.choice([0.25, 0.5]) if hd % 64 == 0 else 0.5
        if int(hd * raw["partial_rotary_factor"]) % 16:
            raw.pop("partial_rotary_factor")
    elif kind == "longrope":
        raw["rope_scaling"] = {"rope_type": "longrope", "short_factor": [round(rng.uniform(1, 3), 3) for _ in range(hd // 2)],
                               "long_factor": [round(rng.uniform(2, 6), 3) for _ in range(hd // 2)],
                               "original_max_position_embeddings": rng.choice([64, 256])}
    if rng.random() < 0.4:
        raw.update(attention_bias=True, mlp_bias=rng.random() < 0.5, attention_output_bias=rng.random() < 0.5)
    return raw


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", range(10))
def test_random_configuration(cuda_device, seed, dtype):
    from infinilm_b200.engine import StepEntry
    raw = random_config(seed)
    w = make_weights(raw, seed)
    rng = random.Random(seed)
    n, n_single = rng.randint(40, 120), 24
    ids = random_ids(n + n_single, raw["vocab_size"], 300 + seed)
    ref = plain_logits(raw, w, ids, dtype)
    what = {k: raw[k] for k in ("hidden_size", "num_attention_heads", "num_key_value_heads", "head_dim", "intermediate_size", "vocab_size")}
    for graphs in (False, True):
        eng = build_engine(raw, w, dtype, num_pages=24)
        if graphs:
            eng.enable_graphs()
        seq = eng.open("r")
        cut = rng.randint(2, n - 2)
        got = [eng.step([StepEntry(seq, ids[:cut], list(range(cut)))]).clone(),
               eng.step([StepEntry(seq, ids[cut:n], list(range(n - cut)))]).clone()]
        for t in range(n, n + n_single):
            got.append(eng.step([StepEntry(seq, ids[t:t + 1], [0])]).clone())
        eng.close(seq)
        eng.synchronize()
        got = torch.cat(got, 0)
        bad = first_bad_row(got, ref, TOL[dtype])
        assert bad is None, f"configuration {seed} {what} {dtype} graphs={graphs}: first wrong position {bad} of {got.shape[0]} (prompt cut at {cut}, {n} prompt tokens)"
        eng.cache.check_invariants()
