"""A toy architecture defined here, in the test, built and stepped without a change to the
framework's files: a mixer with state of its own (a decaying sum kept in a state slot), a
feed-forward that routes every token to one of several experts, a position encoding of its own
(rotation angles that grow with the square root of the pair index, damped), layers that differ
from one another, a run order that names a layer twice and lets one entry read another entry's
cache. It is compared with a plain whole-sequence computation under several ways of cutting the
work. The toy parts use torch for their arithmetic; they are test code, not a model."""
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
from infinilm_b200.parts import (CacheNeed, FeedForward, LayerSpec, Mixer, ModelSpec, PartSpec, PositionEncoding, RunStep,  # noqa: E402
                                 WeightSpec, register_part, unregister_part)
from infinilm_b200.weights import random_tensors  # noqa: E402


class DecayMixer(Mixer):
    """y_t = s_t, s_t = decay * s_{t-1} + W x_t; s lives in a per-request state slot (float32). A step of single
    tokens reads and writes the slots with device-side gathers only, so it can be replayed as a graph."""
    graph_safe = True

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
        if ctx.n_decode == ctx.n_entries:          # one token per entry: no host loop, nothing read back
            s = self.decay * cache.storage.index_select(0, cache.read_slots.long()) + xs
            if cache.writable:
                cache.storage.index_copy_(0, cache.write_slots.long(), s)
            return s.to(x.dtype)
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


def sqrt_inv_freq(rot_dim: int, base: float):
    return [base / math.sqrt(i + 1.0) for i in range(rot_dim // 2)]


class SqrtPosition(PositionEncoding):
    """A rotary encoding with its own table: angle = position * base / sqrt(i + 1), cos/sin times `damp`.
    The attention mixer applies whatever table the position part it was given exposes."""

    def __init__(self, params, prefix, dtype):
        super().__init__(params, prefix, dtype)
        self.rot_dim, self.mscale = int(params["rot_dim"]), float(params["damp"])
        self._table = sqrt_inv_freq(self.rot_dim, float(params["base"]))

    def to_device(self, device):
        self.inv_freq = torch.tensor(self._table, dtype=torch.float64).to(torch.float32).to(device)


class Top1Experts(FeedForward):
    """Every token goes to the expert with the largest router logit (f32), a SwiGLU of its own; the output is the
    expert's, times the logit's sigmoid. A function of the token's row alone, so any cutting gives the same. A step of
    single tokens runs every expert on every row and keeps the chosen one's result (no row lists on the host), so it
    can be replayed as a graph."""
    graph_safe = True

    def __init__(self, params, prefix, dtype):
        super().__init__(params, prefix, dtype)
        self.h, self.inter, self.n = int(params["hidden"]), int(params["intermediate"]), int(params["experts"])

    def weight_specs(self):
        specs = [WeightSpec("router.weight", (self.n, self.h), init=("normal", 0.3))]
        for e in range(self.n):
            specs += [WeightSpec(f"experts.{e}.gate.weight", (self.inter, self.h), init=("normal", 0.05)),
                      WeightSpec(f"experts.{e}.up.weight", (self.inter, self.h), init=("normal", 0.05)),
                      WeightSpec(f"experts.{e}.down.weight", (self.h, self.inter), init=("normal", 0.05))]
        return specs

    def set_weights(self, t):
        self.w = {k: v.float() for k, v in t.items()}

    def forward(self, x, ctx):
        xf = x.float()
        logits = xf @ self.w["router.weight"].t()
        top, which = logits.max(dim=1)
        out = torch.zeros_like(xf)
        if ctx.n_decode == ctx.n_entries:
            for e in range(self.n):
                y = torch.nn.functional.silu(xf @ self.w[f"experts.{e}.gate.weight"].t()) * (xf @ self.w[f"experts.{e}.up.weight"].t())
                out += (y @ self.w[f"experts.{e}.down.weight"].t()) * (torch.sigmoid(top) * (which == e))[:, None]
            return out.to(x.dtype)
        for e in range(self.n):
            rows = (which == e).nonzero().flatten()
            if rows.numel():
                xe = xf[rows]
                y = torch.nn.functional.silu(xe @ self.w[f"experts.{e}.gate.weight"].t()) * (xe @ self.w[f"experts.{e}.up.weight"].t())
                out[rows] = (y @ self.w[f"experts.{e}.down.weight"].t()) * torch.sigmoid(top[rows])[:, None]
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
N_EXPERTS, POS_BASE, POS_DAMP = 3, 0.7, 0.9


def describe_toy(cfg: ToyConfig) -> ModelSpec:
    H = cfg.hidden_size

    def norm(p):
        return PartSpec("rmsnorm", {"size": H, "eps": cfg.eps}, p)
    rope = PartSpec("toy_sqrt", {"rot_dim": cfg.head_dim - 4, "base": POS_BASE, "damp": POS_DAMP})
    l0 = LayerSpec("prenorm_residual", norm("toy.l0.n1"), PartSpec("toy_decay", {"hidden": H, "decay": cfg.decay}, "toy.l0.mixer"),
                   norm("toy.l0.n2"), PartSpec("toy_top1", {"hidden": H, "intermediate": cfg.inter, "experts": N_EXPERTS}, "toy.l0.moe"),
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
    register_part("feed_forward", "toy_top1", Top1Experts)
    register_part("position", "toy_sqrt", SqrtPosition)
    register_architecture(["ToyForCausalLM", "toy"], ToyConfig, describe_toy)
    yield
    unregister_architecture("ToyForCausalLM")
    unregister_part("mixer", "toy_decay")
    unregister_part("feed_forward", "toy_top1")
    unregister_part("position", "toy_sqrt")


def plain_top1(w, p, x, margins):
    """The routed feed-forward on whole sequences; appends each token's routing margin (top logit minus the
    second, over the top's size) to `margins`."""
    logits = x @ w[f"{p}.router.weight"].float().t()
    srt = logits.sort(dim=1, descending=True).values
    margins += ((srt[:, 0] - srt[:, 1]) / srt[:, 0].abs().clamp_min(1e-6)).tolist()
    out = torch.zeros_like(x)
    for t in range(x.shape[0]):
        e = int(logits[t].argmax())
        y = torch.nn.functional.silu(x[t] @ w[f"{p}.experts.{e}.gate.weight"].float().t()) * (x[t] @ w[f"{p}.experts.{e}.up.weight"].float().t())
        out[t] = (y @ w[f"{p}.experts.{e}.down.weight"].float().t()) * torch.sigmoid(logits[t, e])
    return out


def plain_toy(w, ids, round_bf16, margins=None):
    """The toy model on whole sequences, from plain_model's parts and the recurrences above."""
    margins = [] if margins is None else margins
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
            ang = pos.float()[:, None] * torch.tensor(sqrt_inv_freq(12, POS_BASE), dtype=torch.float64).float()[None, :]
            cos, sin = torch.cos(ang) * POS_DAMP, torch.sin(ang) * POS_DAMP
            q, k = plain_model.apply_rope(q, cos, sin, 12), plain_model.apply_rope(k, cos, sin, 12)
            if st.cache_from is None:
                kv_of[i] = (k, v)
            else:
                k, v = kv_of[st.cache_from]
            branch = plain_model.linear(plain_model.attention_scores(q, k, v), w[f"{a}.o_proj.weight"])
        h = h + BRANCH * branch
        x2 = plain_model.rms_norm(h, w[f"{p}.n2.weight"], 1e-5)
        h = h + BRANCH * (plain_top1(w, f"{p}.moe", x2, margins) if st.layer == 0 else plain_model.swiglu_mlp(w, f"{p}.mlp", x2))
    h = plain_model.rms_norm(h, w["toy.norm.weight"], 1e-5)
    return plain_model.linear(h, w["toy.embed.weight"], None, 0.5)


# A token whose two best router logits are nearly equal may go to another expert when the arithmetic changes (bfloat16
# against the plain float32 computation): that is a property of routing, not a fault. So each case names the smallest
# routing margin it relies on, the test checks it on the plain computation, and the bfloat16 case uses a weight seed
# and lengths for which every margin is wide (found by search on the CPU).
SCENARIOS = {
    "float32": dict(seed=4, n=90, cuts=([90], [58] + [1] * 32, [16, 7, 2, 5, 3, 17, 2, 1, 31, 6]), margin=1e-4,
                    lens={"a": 40, "b": 70, "c": 33, "d": 60},
                    sched=[[("a", 16), ("b", 30)], [("a", 1), ("b", 1), ("c", 33)], [("a", 23), ("b", 39)], [("d", 2)], [("d", 57)], [("d", 1)]]),
    "bfloat16": dict(seed=73, n=40, cuts=([40], [24] + [1] * 16, [7, 2, 5, 3, 17, 2, 1, 3]), margin=0.05,
                     lens={"a": 12, "b": 20, "c": 9},
                     sched=[[("a", 5), ("b", 9)], [("a", 1), ("b", 1), ("c", 9)], [("a", 6), ("b", 10)]]),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_architecture_builds_and_steps(cuda_device, toy, dtype):
    sc = SCENARIOS[dtype]
    cfg = config_from_json(RAW)
    assert isinstance(cfg, ToyConfig)
    w = random_tensors(cfg, sc["seed"], "cpu", tie=True)
    assert "toy.l0.mixer.mix.weight" in w and "toy.l0.moe.experts.2.down.weight" in w and "toy.head.weight" not in w
    eng = Engine.from_tensors(cfg, w, dtype=dtype, page_size=16, num_pages=24, max_seqs=4, max_batch_tokens=256)
    # two state caches (layer 0 runs twice) in one group, one paged cache (entry 3 reads entry 1's)
    kinds = [(g.need.kind, g.entries) for g in eng.cache.groups]
    assert kinds == [("state", [0, 2]), ("paged_kv", [1])]
    tol = {"float32": 2e-5, "bfloat16": 2.5e-2}[dtype]
    margins = []
    ids = random_ids(sc["n"], 211, 1)
    ref = plain_toy(w, ids, dtype == "bfloat16", margins)
    for cuts in sc["cuts"]:
        got = run_cut(eng, ids, list(cuts))
        bad = first_bad_row(got, ref, tol)
        assert bad is None, f"cuts {cuts[:4]}..: first wrong position {bad}, rel err {rel_err(got, ref):.3e}"
    # mixed requests: state slots and pages of finished requests are used again
    reqs = {k: random_ids(n, 211, 10 + i) for i, (k, n) in enumerate(sc["lens"].items())}
    refs = {k: plain_toy(w, r, dtype == "bfloat16", margins) for k, r in reqs.items()}
    assert min(margins) >= sc["margin"], f"this case needs routing margins of {sc['margin']}, the plain computation has {min(margins):.2e}"
    got = run_schedule(eng, reqs, sc["sched"])
    for k in reqs:
        bad = first_bad_row(got[k], refs[k], tol)
        assert bad is None, f"request {k}: first wrong position {bad}"
    assert not eng.cache.live and eng.cache.slots.n_free == 4


def test_toy_architecture_decodes_under_graph_replay(cuda_device, toy):
    """Three requests of the toy architecture (state slots, a routed feed-forward, a layer that runs twice, a shared
    cache) decode together with the steps replayed as CUDA graphs: the state slots and block tables come from the
    step's device arrays, padding rows write to the scratch slot and the scratch page."""
    sc = SCENARIOS["float32"]
    cfg = config_from_json(RAW)
    w = random_tensors(cfg, sc["seed"], "cpu", tie=True)
    from infinilm_b200.engine import StepEntry
    eng = Engine.from_tensors(cfg, w, dtype="float32", page_size=16, num_pages=24, max_seqs=4, max_batch_tokens=256)
    assert eng.model.graph_safe and eng.cache.has_state
    eng.enable_graphs()
    reqs = {k: random_ids(n, 211, 30 + i) for i, (k, n) in enumerate({"a": 44, "b": 31, "c": 57}.items())}
    refs = {k: plain_toy(w, r, False) for k, r in reqs.items()}
    n_dec = 24
    seqs = {k: eng.open(k) for k in reqs}
    got = {k: [] for k in reqs}
    for k, r in reqs.items():                      # prompts: eager steps
        n = len(r) - n_dec
        got[k].append(eng.step([StepEntry(seqs[k], r[:n], list(range(n)))]).clone())
    for j in range(n_dec):                         # three single tokens a step (padded to a bucket of four): replayed
        ks = list(reqs)
        lg = eng.step([StepEntry(seqs[k], [reqs[k][len(reqs[k]) - n_dec + j]], [0]) for k in ks]).clone()
        for i, k in enumerate(ks):
            got[k].append(lg[i:i + 1])
    assert any(g.graph is not None for g in eng.runner._graphs.values()), "no step was replayed"
    for k in reqs:
        out = torch.cat(got[k], 0)
        bad = first_bad_row(out, refs[k], 2e-5)
        assert bad is None, f"request {k}: first wrong position {bad}, rel err {rel_err(out, refs[k]):.3e}"
        eng.close(seqs[k])
    eng.synchronize()
    # the zero state (slot 0) was never written, whatever the padding rows did
    for grp in eng.cache.groups:
        if grp.need.kind == "state":
            for st in grp.storage.values():
                assert float(st[0].abs().max()) == 0.0


def test_toy_experts_all_used(toy):
    """The routed feed-forward of the cases above really routes: every expert gets tokens."""
    cfg = config_from_json(RAW)
    w = random_tensors(cfg, 4, "cpu", tie=True)
    x = plain_model.rms_norm(plain_model.embed(torch.tensor(random_ids(90, 211, 1)), w["toy.embed.weight"], 2.0, False), w["toy.l0.n2.weight"], 1e-5)
    which = (x @ w["toy.l0.moe.router.weight"].float().t()).argmax(dim=1)
    assert sorted(set(which.tolist())) == list(range(N_EXPERTS))


def test_unknown_part_kind_is_named(cuda_device):
    from infinilm_b200.parts import build_part
    with pytest.raises(KeyError, match="toy_decay"):
        build_part("mixer", PartSpec("toy_decay", {}), torch.float32)
