"""A plain, slow MiniCPM4 in float32 on the CPU: whole sequences, no cache, one function for each
part. It imports nothing from infinilm_b200; tests compare the engine with it.

It rests on the formulas: InfiniLM's own model code cannot be imported or compiled here (its
Python package needs `infinicore`, and its C++ includes `infinicore/*.hpp`; neither is installed),
so there is no run of the reference behind these functions. Each function cites the lines of
InfiniLM (paths within that project) that fix what it computes; the arithmetic inside RMSNorm,
RoPE and attention is inside InfiniCore there, and is written here from the standard formulas.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def cfg_get(cfg: dict, key: str, default=None):
    v = cfg.get(key, default)
    return default if v is None else v


def head_dim_of(cfg: dict) -> int:
    # csrc/models/minicpm4/minicpm4_for_causal_lm.cpp:144-146: head_dim defaults to hidden/heads.
    return int(cfg_get(cfg, "head_dim", cfg["hidden_size"] // cfg["num_attention_heads"]))


def rotary_dim_of(cfg: dict) -> int:
    # csrc/config/model_config.cpp:41-57.
    hd = head_dim_of(cfg)
    f = float(cfg_get(cfg, "partial_rotary_factor", 1.0))
    if f <= 0.0 or f >= 1.0:
        return hd
    r = min(max(int(round(hd * f)), 2), hd)
    return max(r - (r % 2), 2)


def embed(ids: torch.Tensor, table: torch.Tensor, scale_emb: float, round_bf16: bool) -> torch.Tensor:
    """python/infinilm/modeling_utils.py:258-263: the table is multiplied by scale_emb at load
    time in the model dtype; csrc/models/minicpm4/minicpm4_for_causal_lm.cpp:92: plain gather."""
    x = table.float()[ids] * scale_emb
    return x.bfloat16().float() if round_bf16 else x


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """csrc/models/minicpm4/minicpm4_for_causal_lm.cpp:43,45,86: RMSNorm(hidden_size, rms_norm_eps);
    y = x / sqrt(mean(x^2) + eps) * w."""
    var = x.pow(2).mean(dim=-1, keepdim=True)
    return x * torch.rsqrt(var + eps) * w.float()


def rope_tables(cfg: dict, positions: torch.Tensor):
    """cos and sin [T, rot/2]. csrc/layers/rotary_embedding/rope_scaling_creators.cpp:23-47 (LongRoPE
    takes short_factor, long_factor, original_max_position_embeddings, factor);
    csrc/layers/rotary_embedding/rotary_embedding.cpp:90-113 (head_dim, rotary_dim, max positions,
    theta). inv_freq_i = 1 / (f_i * theta^(2i/rot)); f = long_factor when max_position_embeddings
    exceeds the original maximum, else short_factor; cos/sin scaled by sqrt(1 + ln(s)/ln(orig))."""
    rot = rotary_dim_of(cfg)
    theta = float(cfg_get(cfg, "rope_theta", 10000.0))
    i = torch.arange(rot // 2, dtype=torch.float64)
    freq = theta ** (2.0 * i / rot)
    mscale = 1.0
    rs = cfg.get("rope_scaling")
    kind = None if rs is None else rs.get("rope_type", rs.get("type", "default"))
    if kind == "longrope":
        orig, mx = int(rs["original_max_position_embeddings"]), int(cfg["max_position_embeddings"])
        fac = torch.tensor(rs["long_factor"] if mx > orig else rs["short_factor"], dtype=torch.float64)
        freq = freq * fac
        s = mx / orig
        if rs.get("factor") is not None and float(rs["factor"]) != 1.0:
            s = float(rs["factor"])
        if s > 1.0:
            mscale = math.sqrt(1.0 + math.log(s) / math.log(orig))
    inv_freq = (1.0 / freq).float()
    ang = positions.float()[:, None] * inv_freq[None, :]
    return torch.cos(ang) * mscale, torch.sin(ang) * mscale


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, rot: int) -> torch.Tensor:
    """x [T, heads, head_dim]; rotate-half pairing (i, i+rot/2) (csrc/config/model_config.hpp:139,
    GPT_NEOX); dims beyond rot pass through (csrc/config/model_config.cpp:41-57)."""
    half = rot // 2
    x1, x2, rest = x[..., :half], x[..., half:rot], x[..., rot:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s, rest], dim=-1)


def attention_scores(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: Optional[int] = None) -> torch.Tensor:
    """q [T, nh, hd], k/v [T, nkv, hd] of one whole sequence -> [T, nh*hd].
    csrc/layers/attention/attention.cpp:41 (scale 1/sqrt(head_dim));
    csrc/layers/attention/backends/static_attn.cpp:82-94 (query head j reads kv head j/(nh/nkv);
    scale*Q*K^T, causal softmax, times V)."""
    T, nh, hd = q.shape
    nkv = k.shape[1]
    rep = nh // nkv
    kk = k.repeat_interleave(rep, dim=1)
    vv = v.repeat_interleave(rep, dim=1)
    s = torch.einsum("thd,shd->hts", q, kk) / math.sqrt(hd)
    idx = torch.arange(T)
    mask = idx[None, :] > idx[:, None]
    if window is not None:
        mask = mask | (idx[None, :] < idx[:, None] - window + 1)
    s = s.masked_fill(mask[None], float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.einsum("hts,shd->thd", p, vv).reshape(T, nh * hd)


def linear(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor] = None, alpha: float = 1.0) -> torch.Tensor:
    """csrc/layers/quantization/none_quantization.cpp:26-46: alpha * x W^T (+ b)."""
    y = alpha * (x @ w.float().t())
    return y if b is None else y + b.float()


def attention_block(cfg: dict, w: Dict[str, torch.Tensor], p: str, x: torch.Tensor, positions: torch.Tensor,
                    window: Optional[int] = None) -> torch.Tensor:
    """csrc/layers/attention/attention.cpp:96-137: q,k,v projections, view as heads, RoPE on q and k,
    attention, o_proj."""
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], head_dim_of(cfg)
    T = x.shape[0]

    def b(n):
        return w.get(f"{p}.{n}.bias")
    q = linear(x, w[f"{p}.q_proj.weight"], b("q_proj")).view(T, nh, hd)
    k = linear(x, w[f"{p}.k_proj.weight"], b("k_proj")).view(T, nkv, hd)
    v = linear(x, w[f"{p}.v_proj.weight"], b("v_proj")).view(T, nkv, hd)
    cos, sin = rope_tables(cfg, positions)
    rot = rotary_dim_of(cfg)
    q, k = apply_rope(q, cos, sin, rot), apply_rope(k, cos, sin, rot)
    a = attention_scores(q, k, v, window)
    return linear(a, w[f"{p}.o_proj.weight"], b("o_proj"))


def swiglu_mlp(w: Dict[str, torch.Tensor], p: str, x: torch.Tensor) -> torch.Tensor:
    """csrc/layers/mlp/mlp.cpp:30-37: down(silu(gate(x)) * up(x))."""
    g = linear(x, w[f"{p}.gate_proj.weight"], w.get(f"{p}.gate_proj.bias"))
    u = linear(x, w[f"{p}.up_proj.weight"], w.get(f"{p}.up_proj.bias"))
    return linear(torch.nn.functional.silu(g) * u, w[f"{p}.down_proj.weight"], w.get(f"{p}.down_proj.bias"))


def decoder_layer(cfg: dict, w: Dict[str, torch.Tensor], i: int, h: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
    """csrc/models/minicpm4/minicpm4_for_causal_lm.cpp:59-71 with the branch scale of :12-20,27,33:
    h += s * Attn(norm(h)); h += s * MLP(norm(h)), s = scale_depth / sqrt(num_hidden_layers)."""
    s = float(cfg_get(cfg, "scale_depth", 1.0)) / math.sqrt(cfg["num_hidden_layers"])
    p = f"model.layers.{i}"
    eps = float(cfg["rms_norm_eps"])
    h = h + s * attention_block(cfg, w, f"{p}.self_attn", rms_norm(h, w[f"{p}.input_layernorm.weight"], eps), positions)
    h = h + s * swiglu_mlp(w, f"{p}.mlp", rms_norm(h, w[f"{p}.post_attention_layernorm.weight"], eps))
    return h


def lm_head(cfg: dict, w: Dict[str, torch.Tensor], h: torch.Tensor) -> torch.Tensor:
    """csrc/models/minicpm4/minicpm4_for_causal_lm.cpp:117-125: logits = (dim_model_base/hidden) * h W^T;
    python/infinilm/modeling_utils.py:342-351: an absent lm_head.weight is the unscaled embedding."""
    wt = w["lm_head.weight"] if "lm_head.weight" in w else w["model.embed_tokens.weight"]
    alpha = 1.0
    if cfg.get("dim_model_base") is not None:
        alpha = float(cfg["dim_model_base"]) / float(cfg["hidden_size"])
    return linear(h, wt, None, alpha)


def forward(cfg: dict, w: Dict[str, torch.Tensor], ids: List[int], round_embedding_bf16: bool = False,
            return_hidden: bool = False):
    """Logits [T, vocab] of one whole sequence (csrc/models/minicpm4/minicpm4_for_causal_lm.cpp:89-101,123-127)."""
    with torch.no_grad():
        t = torch.tensor(ids, dtype=torch.long)
        pos = torch.arange(len(ids))
        h = embed(t, w["model.embed_tokens.weight"], float(cfg_get(cfg, "scale_emb", 1.0)), round_embedding_bf16)
        hs = [h]
        for i in range(cfg["num_hidden_layers"]):
            h = decoder_layer(cfg, w, i, h, pos)
            hs.append(h)
        h = rms_norm(h, w["model.norm.weight"], float(cfg["rms_norm_eps"]))
        logits = lm_head(cfg, w, h)
    return (logits, hs) if return_hidden else logits


def greedy_generate(cfg: dict, w: Dict[str, torch.Tensor], prompt: List[int], n_new: int) -> List[int]:
    ids = list(prompt)
    out = []
    for _ in range(n_new):
        nxt = int(torch.argmax(forward(cfg, w, ids)[-1]).item())
        out.append(nxt)
        ids.append(nxt)
    return out


# -- sampling, as plain as it gets ---------------------------------------------------------------
def sample_plain(logits: torch.Tensor, temperature: float, top_k: int, top_p: float, u: float) -> int:
    """One token from one row of logits. InfiniLM: csrc/engine/rank_worker.cpp:487-497 calls
    random_sample_(logits, random_val, top_p, top_k, temperature); top_k == 1 is greedy
    (python/infinilm/llm/sampling_params.py:13-16). Keep the top_k most likely tokens, of those the
    smallest set whose mass reaches top_p (ties at the edge all kept), renormalise, and walk the kept
    tokens in index order until the running mass passes u times the kept mass."""
    V = logits.numel()
    if top_k == 1 or temperature == 0.0:
        return int(torch.argmax(logits).item())
    p = torch.softmax(logits.double() / temperature, dim=-1)
    keep = torch.ones(V, dtype=torch.bool)
    if 0 < top_k < V:
        kth = torch.sort(p, descending=True).values[top_k - 1]
        keep &= p >= kth
    if top_p < 1.0:
        pk = torch.where(keep, p, torch.zeros_like(p))
        sp, _ = torch.sort(pk, descending=True)
        cum = torch.cumsum(sp, 0)
        n = int((cum < top_p * pk.sum()).sum().item()) + 1
        thr = sp[min(n, V) - 1]
        keep &= p >= thr
    pk = torch.where(keep, p, torch.zeros_like(p))
    target = u * pk.sum()
    cum = torch.cumsum(pk, 0)
    hit = torch.nonzero(keep & (cum > target))
    if hit.numel() == 0:                          # u so close to 1 that rounding leaves nothing: the mode
        return int(torch.argmax(logits).item())
    return int(hit[0].item())
