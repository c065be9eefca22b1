"""The benchmark's layer geometry (MiniCPM4-8B sizes: hidden 4096, 32 heads on 2 kv heads, head_dim 128, intermediate
16384, vocabulary 73448) on two layers with random weights: the bfloat16 engine against the float32 engine of the same
weights. The plain implementation is too slow for these sizes; the float32 path (FFMA products, plain attention,
float32 cache) is the oracle here, and it is tied to the plain implementation by the tests at tiny sizes.

The cases cross every kernel that the benchmark times: the weight-streaming products with their fused epilogues
(1..16 rows), the library products and the tcgen05 output head (17..256 rows), the TMA decode attention at group 16,
the tensor-memory prefill attention at head_dim 128, and CUDA-graph replay of decode steps at batch 8 and 64. The
method is InfiniLM's own: logits after the prompt and after every decode step, one backend against another
(`test/models/llama/test_forward_validation.py:128-622`)."""
import pytest
import torch

from replay_util import TOL, first_bad_row, rel_err, run_schedule
from tiny_configs import random_ids

pytestmark = pytest.mark.gpu

from infinilm_b200.config import config_from_json  # noqa: E402
from infinilm_b200.engine import Engine, StepEntry  # noqa: E402
from infinilm_b200.weights import random_tensors  # noqa: E402

RAW = {
    "architectures": ["MiniCPMForCausalLM"], "model_type": "minicpm",
    "num_hidden_layers": 2, "hidden_size": 4096, "num_attention_heads": 32, "num_key_value_heads": 2,
    "head_dim": 128, "intermediate_size": 16384, "vocab_size": 73448,
    "rope_theta": 10000.0, "max_position_embeddings": 32768,
    "rope_scaling": {"rope_type": "longrope", "short_factor": [1.0 + 0.05 * i for i in range(64)],
                     "long_factor": [1.0 + 0.25 * i for i in range(64)], "original_max_position_embeddings": 32768},
    "scale_emb": 12, "dim_model_base": 256, "scale_depth": 1.4, "rms_norm_eps": 1e-6,
    "tie_word_embeddings": False, "torch_dtype": "bfloat16", "eos_token_id": [2, 73440],
}
V = RAW["vocab_size"]


@pytest.fixture(scope="module")
def engines(cuda_device):
    cfg = config_from_json(RAW)
    w = random_tensors(cfg, 0, "cuda")
    kw = dict(page_size=16, num_pages=2000, max_seqs=64, max_batch_tokens=4096)
    e16 = Engine.from_tensors(cfg, w, dtype="bfloat16", **kw)
    e32 = Engine.from_tensors(cfg, w, dtype="float32", **kw)
    del w
    yield e16, e32
    e16.synchronize()
    del e16, e32
    torch.cuda.empty_cache()


def _agree(got, ref, what):
    """Per row: the largest difference against the largest float32 logit of that row; and the same argmax wherever the
    float32 top-2 margin is wider than the rounding allows."""
    got, ref = got.float(), ref.float()
    bad = first_bad_row(got, ref, TOL["bfloat16"])
    assert bad is None, f"{what}: first wrong row {bad} of {got.shape[0]}, rel err {rel_err(got, ref):.3e}"
    top2 = torch.topk(ref, 2, dim=-1).values
    sure = (top2[:, 0] - top2[:, 1]) > 4 * TOL["bfloat16"] * ref.abs().amax(dim=-1)
    assert bool((got.argmax(-1) == ref.argmax(-1))[sure].all()), f"{what}: argmax differs on a row with a wide margin"
    return int(sure.sum())


def _wanted(n):
    """Every 61st place and the last 40: enough to see a wrong tile or page, small enough for the head at 8B width."""
    return sorted(set(range(0, n, 61)) | set(range(max(0, n - 40), n)))


def _run(eng, ids, cuts, graphs=False, want_all=False):
    """Feeds ids in portions; logits at the wanted places of each portion (all places of single-token steps)."""
    eng.runner.use_graphs = graphs
    seq = eng.open("r")
    outs, a = [], 0
    for c in cuts:
        want = list(range(c)) if (want_all or c == 1) else _wanted(c)
        outs.append(eng.step([StepEntry(seq, ids[a:a + c], want)]).clone())
        a += c
    eng.close(seq)
    eng.runner.use_graphs = False
    return torch.cat(outs, 0)


def test_whole_prompt_and_single_tokens(engines):
    """A prompt of 2,100 tokens in one step (prefill attention over many key tiles, library products), then 32 tokens
    one by one (weight-streaming products with fused epilogues, split-KV attention through TMA), eager and replayed."""
    e16, e32 = engines
    ids = random_ids(2132, V, 1)
    cuts = [2100] + [1] * 32
    ref = _run(e32, ids, cuts)
    got = _run(e16, ids, cuts)
    n_sure = _agree(got, ref, "prompt of 2,100 then 32 single tokens")
    assert n_sure > 0
    replayed = _run(e16, ids, cuts, graphs=True)
    _agree(replayed, ref, "the same with decode steps replayed as graphs")
    assert first_bad_row(replayed, got, TOL["bfloat16"]) is None
    e16.synchronize()


def test_changing_portions(engines):
    """Portions of changing size, across the 16-row and 256-row borders of the matrix-product kernels."""
    e16, e32 = engines
    ids = random_ids(700, V, 2)
    cuts = [300, 16, 17, 2, 64, 1, 33, 256, 5, 3, 1, 2]
    assert sum(cuts) == 700
    got = _run(e16, ids, cuts, want_all=True)
    _agree(got, _run(e32, ids, cuts, want_all=True), "changing portions")
    # and against the same tokens run whole: how they were cut does not show beyond rounding
    whole = _run(e16, ids, [700], want_all=True)
    assert first_bad_row(got, whole, TOL["bfloat16"]) is None
    e16.synchronize()


def test_mixed_requests_with_reused_pages(cuda_device):
    """Four live requests, portions of some beside single tokens of others, in a pool so small that pages come back."""
    cfg = config_from_json(RAW)
    w = random_tensors(cfg, 1, "cuda")
    lens = {"p": 3, "q": 130, "r": 260, "s": 200, "t": 90, "u": 150}
    reqs = {k: random_ids(n, V, 50 + i) for i, (k, n) in enumerate(lens.items())}
    sched = [
        [("p", 3), ("q", 64)],
        [("q", 65), ("r", 100), ("s", 2)],
        [("q", 1), ("r", 100), ("s", 100)],                     # q ends
        [("r", 1), ("s", 97), ("t", 30)],
        [("r", 59), ("s", 1), ("t", 1), ("u", 20)],              # r, s end
        [("t", 59), ("u", 1)],                                   # t ends
        [("u", 1)], [("u", 64)], [("u", 64)],
    ]
    outs = {}
    for dtype in ("float32", "bfloat16"):
        eng = Engine.from_tensors(cfg, w, dtype=dtype, page_size=16, num_pages=40, max_seqs=4, max_batch_tokens=512)
        outs[dtype] = run_schedule(eng, reqs, sched)
        assert not eng.cache.live and eng.cache.free_pages() == {0: 40}
        eng.synchronize()
        del eng
    for k in reqs:
        _agree(outs["bfloat16"][k], outs["float32"][k], f"mixed request {k}")


@pytest.mark.parametrize("batch", [8, 64])
def test_decode_steps_at_batch(engines, batch):
    """Batches of 8 and 64 requests (contexts of 40 to 300 tokens) decoding together, eager and replayed as graphs:
    8 rows go through the weight-streaming kernels, 64 through the library products and the tcgen05 output head."""
    e16, e32 = engines
    prompts = [random_ids(40 + (37 * i) % 260, V, 300 + i) for i in range(batch)]
    new = [random_ids(6, V, 900 + i) for i in range(batch)]

    def run(eng, graphs):
        eng.runner.use_graphs = graphs
        seqs = [eng.open(f"b{i}") for i in range(batch)]
        for lo in range(0, batch, 8):               # prompts, eight requests a step
            eng.step([StepEntry(seqs[i], prompts[i], []) for i in range(lo, min(lo + 8, batch))])
        outs = []
        for j in range(6):
            outs.append(eng.step([StepEntry(seqs[i], [new[i][j]], [0]) for i in range(batch)]).clone())
        for s in seqs:
            eng.close(s)
        eng.runner.use_graphs = False
        return torch.cat(outs, 0)
    ref = run(e32, False)
    eager = run(e16, False)
    _agree(eager, ref, f"decode at batch {batch}")
    replayed = run(e16, True)
    _agree(replayed, ref, f"decode at batch {batch}, replayed")
    assert any(g.graph is not None for g in e16.runner._graphs.values())
    e16.synchronize()
