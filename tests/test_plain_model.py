"""The plain implementation checked against properties that do not depend on it: causality, the
meaning of grouped heads, the relative-position property of the rotation, a window, an explicit
loop for attention, and the sampler's rules (CPU)."""
import math

import pytest
import torch

import plain_model
from tiny_configs import TINY, make_weights, random_ids, tiny_a, tiny_b


@pytest.mark.parametrize("name", ["a", "b", "c", "d"])
def test_causal_and_deterministic(name):
    raw = TINY[name]()
    w = make_weights(raw, 0)
    ids = random_ids(24, raw["vocab_size"], 1)
    full = plain_model.forward(raw, w, ids)
    assert full.shape == (24, raw["vocab_size"]) and torch.isfinite(full).all()
    # a later token does not change earlier logits; a prefix gives the same logits
    ids2 = list(ids)
    ids2[20] = (ids2[20] + 1) % raw["vocab_size"]
    assert torch.equal(plain_model.forward(raw, w, ids2)[:20], full[:20])
    assert torch.allclose(plain_model.forward(raw, w, ids[:11]), full[:11], atol=1e-6)
    assert not torch.allclose(plain_model.forward(raw, w, ids2)[20:], full[20:])


def test_attention_against_a_loop():
    g = torch.Generator().manual_seed(0)
    T, nh, nkv, hd = 9, 6, 3, 8
    q, k, v = torch.randn(T, nh, hd, generator=g), torch.randn(T, nkv, hd, generator=g), torch.randn(T, nkv, hd, generator=g)
    for window in (None, 4):
        got = plain_model.attention_scores(q, k, v, window).view(T, nh, hd)
        for t in range(T):
            lo = 0 if window is None else max(0, t - window + 1)
            for j in range(nh):
                s = torch.tensor([float(q[t, j] @ k[u, j // 2]) / math.sqrt(hd) for u in range(lo, t + 1)])
                ref = (torch.softmax(s, 0)[:, None] * v[lo:t + 1, j // 2]).sum(0)
                assert torch.allclose(got[t, j], ref, atol=1e-6)


def test_rotation_depends_on_distance_only():
    cfg = {"hidden_size": 32, "num_attention_heads": 1, "head_dim": 32, "rope_theta": 10000.0, "max_position_embeddings": 512}
    g = torch.Generator().manual_seed(1)
    q, k = torch.randn(1, 1, 32, generator=g), torch.randn(1, 1, 32, generator=g)

    def score(pq, pk):
        cq, sq = plain_model.rope_tables(cfg, torch.tensor([pq]))
        ck, sk = plain_model.rope_tables(cfg, torch.tensor([pk]))
        return float((plain_model.apply_rope(q, cq, sq, 32) * plain_model.apply_rope(k, ck, sk, 32)).sum())
    assert score(17, 5) == pytest.approx(score(112, 100), abs=1e-4)
    assert score(17, 5) != pytest.approx(score(17, 6), abs=1e-4)
    # partial rotation leaves the tail alone; position 0 is the identity
    c0, s0 = plain_model.rope_tables(cfg, torch.tensor([0]))
    assert torch.equal(plain_model.apply_rope(q, c0, s0, 32), q)
    c, s = plain_model.rope_tables({**cfg, "partial_rotary_factor": 0.5}, torch.tensor([9]))
    assert c.shape[-1] == 8 and torch.equal(plain_model.apply_rope(q, c, s, 16)[..., 16:], q[..., 16:])


def test_longrope_tables():
    raw = tiny_b()
    cos, sin = plain_model.rope_tables(raw, torch.tensor([3]))
    rs = raw["rope_scaling"]
    m = math.sqrt(1 + math.log(256 / 64) / math.log(64))
    inv = 1.0 / (torch.tensor(rs["long_factor"], dtype=torch.float64) * 1e6 ** (torch.arange(16, dtype=torch.float64) * 2 / 32))
    assert torch.allclose(cos[0], (torch.cos(3 * inv.float()) * m), atol=1e-6)
    raw["max_position_embeddings"] = 64                       # not extended: short factors, no scale
    cos, _ = plain_model.rope_tables(raw, torch.tensor([3]))
    inv = 1.0 / (torch.tensor(rs["short_factor"], dtype=torch.float64) * 1e6 ** (torch.arange(16, dtype=torch.float64) * 2 / 32))
    assert torch.allclose(cos[0], torch.cos(3 * inv.float()), atol=1e-6)


def test_scale_factors_act_where_they_should():
    raw = tiny_a()
    w = make_weights(raw, 2)
    ids = random_ids(6, raw["vocab_size"], 3)
    base = plain_model.forward(raw, w, ids)
    assert torch.allclose(plain_model.forward({**raw, "dim_model_base": 64}, w, ids), 2 * base, atol=1e-6)
    l0 = plain_model.forward({**raw, "scale_depth": 0.0}, w, ids)      # no branch is added: logits of the embedding alone
    h = plain_model.rms_norm(plain_model.embed(torch.tensor(ids), w["model.embed_tokens.weight"], 12.0, False),
                             w["model.norm.weight"], 1e-6)
    assert torch.allclose(l0, 0.5 * h @ w["model.embed_tokens.weight"].float().t(), atol=1e-5)
    assert plain_model.greedy_generate(raw, w, ids, 3)[:1] == [int(torch.argmax(base[-1]))]


def test_plain_sampler_rules():
    logits = torch.tensor([0.0, 3.0, 1.0, 3.0, -2.0, 2.0])
    assert plain_model.sample_plain(logits, 1.0, 1, 1.0, 0.9) == 1                 # greedy: lowest index among ties
    assert plain_model.sample_plain(logits, 0.0, 0, 1.0, 0.9) == 1
    picks = {plain_model.sample_plain(logits, 1.0, 2, 1.0, u / 50) for u in range(50)}
    assert picks == {1, 3}                                                         # top-2 with a tie at the edge kept
    picks = {plain_model.sample_plain(logits, 1.0, 3, 1.0, u / 200) for u in range(200)}
    assert picks == {1, 3, 5}
    p = torch.softmax(logits, 0)
    picks = {plain_model.sample_plain(logits, 1.0, 0, float(p[1] + p[3]) - 1e-3, u / 200) for u in range(200)}
    assert picks == {1, 3}                                                         # nucleus: smallest set reaching top_p
    assert plain_model.sample_plain(logits, 1.0, 0, 1.0, 0.0) == 0 and plain_model.sample_plain(logits, 1.0, 0, 1.0, 0.999999) == 5
    hot = [plain_model.sample_plain(logits, 0.05, 0, 1.0, u / 100) for u in range(1, 100)]
    assert set(hot) == {1, 3}                                                      # low temperature concentrates on the maxima
