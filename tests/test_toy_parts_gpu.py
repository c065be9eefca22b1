"""A toy architecture defined here, in the test, built and stepped without a change to the
framework's files: a mixer with state of its own (a decaying sum kept in a state slot), layers
that differ from one another, a run order that names a layer twice and lets one entry read
another entry's cache. It is compared with a plain whole-sequence computation under several ways
of cutting the work. The toy parts use torch for their arithmetic; they are test code, not a model."""
import math
from dataclasses import dataclass

import pytest
import torch

import plain_model
from replay_util import first_bad_row, rel_err, run_cut, run_schedule
from tiny_configs import random_ids

pytestmark = pytest.mark.gpu

from infinilm_b200.config import ModelConfig, config_from_json, register_architecture, unregister_architecture  # noqa: E402
from infinilm_b200.engine import Engine  # noqa: E402
from infinilm_b200.parts import (CacheNeed, LayerSpec, Mixer, ModelSpec, PartSpec, RunStep, WeightSpec,  # noqa: E402
                                 register_part, unregister_part)
from infinilm_b200.weights import random_tensors  # noqa: E402


class DecayMixer(Mixer):
    """y_t = s_t, s_t = decay * s_{t-1} + W x_t; s lives in a per-request state slot (float32)."""

    def __init__(self, params, prefix, dtype):
        super().__init__(params, prefix, dtype)
        self.h, self.decay = int(params["hidden"]), float(params["decay"])

    def weight_specs(self):
        return [WeightSpec("mix.weight", (self.h, self.h), init=("normal", 0.05))]

    def set_weights(self, t):
        self.w = t["mix.weight"].float()

    def cache_need(self):
        return CacheNeed("state", shape=(self.h,), dtype="float32")

    def forward(self, x, ctx, cache):
        xs = x.float() @ self.w.t()
        out = torch.empty_like(xs)
        rs, ws = cache.read_slots.long().tolist(), cache.write_slots.long().tolist()
        a = 0
        for e, n in enumerate(ctx.h_qlen):
            s = cache.storage[rs[e]].clone()
            for t in range(a, a + n):
                s = self.decay * s + xs[t]
                out[t] = s
            if cache.writable:
                cache.storage[ws[e]] = s
            a += n
        return out.to(x.dtype)


@dataclass
class ToyConfig(ModelConfig):
    n_heads: int = 0
    n_kv_heads: int = 0
    head_dim: int = 0
    inter: int = 0
    decay: float = 0.5
    eps: float = 1e-5

    @classmethod
    def from_json(cls, raw):
        return cls(architecture="ToyForCausalLM", model_type="toy", vocab_size=raw["vocab_size"], hidden_size=raw["hidden_size"],
                   max_position_embeddings=raw["max_position_embeddings"], torch_dtype=raw["torch_dtype"], raw=dict(raw),
                   n_heads=raw["n_heads"], n_kv_heads=raw["n_kv_heads"], head_dim=raw["head_dim"], inter=raw["inter"],
                   decay=raw["decay"], eps=raw["eps"])


ORDER = [RunStep(0), RunStep(1), RunStep(0), RunStep(1, cache_from=1)]
BRANCH = 0.6


def describe_toy(cfg: ToyConfig) -> ModelSpec:
    H = cfg.hidden_size

    def norm(p):
        return PartSpec("rmsnorm", {"size": H, "eps": cfg.eps}, p)
    rope = PartSpec("rope", {"rot_dim": cfg.head_dim, "theta": 10000.0})
    l0 = LayerSpec("prenorm_residual", norm("toy.l0.n1"), PartSpec("toy_decay", {"hidden": H, "decay": cfg.decay}, "toy.l0.mixer"),
                   norm("toy.l0.n2"), PartSpec("swiglu", {"hidden": H, "intermediate": cfg.inter}, "toy.l0.mlp"),
                   {"residual_scale": BRANCH})
    l1 = LayerSpec("prenorm_residual", norm("toy.l1.n1"),
                   PartSpec("attention", {"hidden": H, "n_heads": cfg.n_heads, "n_kv_heads": cfg.n_kv_heads,
                                          "head_dim": cfg.head_dim, "position": rope}, "toy.l1.attn"),
                   norm("toy.l1.n2"), PartSpec("swiglu", {"hidden": H, "intermediate": 2 * cfg.inter}, "toy.l1.mlp"),
                   {"residual_scale": BRANCH})
    return ModelSpec(PartSpec("token_embedding", {"vocab": cfg.vocab_size, "hidden": H, "scale": 2.0}, "toy.embed"),
                     [l0, l1], list(ORDER), norm("toy.norm"),
                     PartSpec("linear_head", {"vocab": cfg.vocab_size, "hidden": H, "scale": 0.5, "tied_to": "toy.embed.weight"}, "toy.head"))


RAW = {"architectures": ["ToyForCausalLM"], "model_type": "toy", "vocab_size": 211, "hidden_size": 96, "max_position_embeddings": 256,
       "torch_dtype": "float32", "n_heads": 6, "n_kv_heads": 2, "head_dim": 16, "inter": 120, "decay": 0.7, "eps": 1e-5,
       "tie_word_embeddings": True}


@pytest.fixture()
def toy():
    register_part("mixer", "toy_decay", DecayMixer)
    register_architecture(["ToyForCausalLM", "toy"], ToyConfig, describe_toy)
    yield
    unregister_architecture("ToyForCausalLM")
    unregister_part("mixer", "toy_decay")


def plain_toy(w, ids, round_bf16):
    """The toy model on whole sequences, from plain_model's parts and the recurrence above."""
    cfg = {"num_attention_heads": 6, "num_key_value_heads": 2, "head_dim": 16, "hidden_size": 96, "rope_theta": 10000.0,
           "max_position_embeddings": 256}
    T = len(ids)
    pos = torch.arange(T)
    h = plain_model.embed(torch.tensor(ids), w["toy.embed.weight"], 2.0, round_bf16)
    kv_of = {}
    for i, st in enumerate(ORDER):
        p = f"toy.l{st.layer}"
        x = plain_model.rms_norm(h, w[f"{p}.n1.weight"], 1e-5)
        if st.layer == 0:
            xs = x @ w[f"{p}.mixer.mix.weight"].float().t()
            s = torch.zeros(96)
            rows = []
            for t in range(T):
                s = 0.7 * s + xs[t]
                rows.append(s.clone())
            branch = torch.stack(rows)
        else:
            a = f"{p}.attn"
            q = plain_model.linear(x, w[f"{a}.q_proj.weight"]).view(T, 6, 16)
            k = plain_model.linear(x, w[f"{a}.k_proj.weight"]).view(T, 2, 16)
            v = plain_model.linear(x, w[f"{a}.v_proj.weight"]).view(T, 2, 16)
            cos, sin = plain_model.rope_tables(cfg, pos)
            q, k = plain_model.apply_rope(q, cos, sin, 16), plain_model.apply_rope(k, cos, sin, 16)
            if st.cache_from is None:
                kv_of[i] = (k, v)
            else:
                k, v = kv_of[st.cache_from]
            branch = plain_model.linear(plain_model.attention_scores(q, k, v), w[f"{a}.o_proj.weight"])
        h = h + BRANCH * branch
        h = h + BRANCH * plain_model.swiglu_mlp(w, f"{p}.mlp", plain_model.rms_norm(h, w[f"{p}.n2.weight"], 1e-5))
    h = plain_model.rms_norm(h, w["toy.norm.weight"], 1e-5)
    return plain_model.linear(h, w["toy.embed.weight"], None, 0.5)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_architecture_builds_and_steps(cuda_device, toy, dtype):
    cfg = config_from_json(RAW)
    assert isinstance(cfg, ToyConfig)
    w = random_tensors(cfg, 4, "cpu", tie=True)
    assert "toy.l0.mixer.mix.weight" in w and "toy.head.weight" not in w
    eng = Engine.from_tensors(cfg, w, dtype=dtype, page_size=16, num_pages=24, max_seqs=4, max_batch_tokens=256)
    # two state caches (layer 0 runs twice) in one group, one paged cache (entry 3 reads entry 1's)
    kinds = [(g.need.kind, g.entries) for g in eng.cache.groups]
    assert kinds == [("state", [0, 2]), ("paged_kv", [1])]
    tol = {"float32": 2e-5, "bfloat16": 2.5e-2}[dtype]
    ids = random_ids(90, 211, 1)
    ref = plain_toy(w, ids, dtype == "bfloat16")
    for cuts in ([90], [58] + [1] * 32, [16, 7, 2, 5, 3, 17, 2, 1, 31, 6]):
        got = run_cut(eng, ids, cuts)
        bad = first_bad_row(got, ref, tol)
        assert bad is None, f"cuts {cuts[:4]}..: first wrong position {bad}, rel err {rel_err(got, ref):.3e}"
    # mixed requests: state slots and pages of finished requests are used again
    reqs = {k: random_ids(n, 211, 10 + i) for i, (k, n) in enumerate({"a": 40, "b": 70, "c": 33, "d": 60}.items())}
    sched = [[("a", 16), ("b", 30)], [("a", 1), ("b", 1), ("c", 33)], [("a", 23), ("b", 39)], [("d", 2)], [("d", 57)], [("d", 1)]]
    got = run_schedule(eng, reqs, sched)
    for k, r in reqs.items():
        bad = first_bad_row(got[k], plain_toy(w, r, dtype == "bfloat16"), tol)
        assert bad is None, f"request {k}: first wrong position {bad}"
    assert not eng.cache.live and eng.cache.slots.n_free == 4


def test_unknown_part_kind_is_named(cuda_device):
    from infinilm_b200.parts import build_part
    with pytest.raises(KeyError, match="toy_decay"):
        build_part("mixer", PartSpec("toy_decay", {}), torch.float32)
