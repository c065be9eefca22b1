"""Command line in InfiniLM's manner: the option names and meanings of its `BaseConfig` where it
has them (`python/infinilm/base_config.py:182-345,395-418`), used as `examples/test_infer.py:124-188`
uses them: build an `LLM`, generate for `--batch-size` copies of one prompt, print the answers
and the time.

    python -m infinilm_b200 --model DIR --enable-paged-attn --max-new-tokens 32 --prompt-len 64
    python -m infinilm_b200 --write-random-model DIR --config config.json --seed 0

Options of other devices, parallelism, MoE, quantization, drafts and the server do not exist here.
"""
from __future__ import annotations

import argparse
import json
import logging
import sys
import time

logger = logging.getLogger("infinilm_b200")


def parse_list(value: str):
    """An int or a list of ints, in InfiniLM's spellings (`python/infinilm/base_config.py:11-43`): "1", "[1,2,4]", "1,2,4"."""
    value = value.strip()
    try:
        if value.startswith("[") and value.endswith("]"):
            got = json.loads(value)
            return [int(x) for x in got] if isinstance(got, list) else int(got)
        if "," in value:
            return [int(x.strip()) for x in value.split(",")]
        return int(value)
    except (ValueError, TypeError):
        raise argparse.ArgumentTypeError(f"value must be an int or list[int], got: {value}") from None


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="infinilm_b200", description=__doc__,
                                formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--model", type=str, help="model folder (config.json + safetensors)")
    p.add_argument("--device", type=str, default="auto", help="auto, nvidia or cuda[:N] (CUDA only)")
    p.add_argument("--dtype", type=str, default=None, choices=["float32", "bfloat16", "float16"],
                   help="compute dtype (default: the folder's torch_dtype; float16 runs as bfloat16)")
    p.add_argument("--attn", type=str, default="default", choices=["default", "paged-attn", "flash-attn"],
                   help="accepted for scripts written for InfiniLM; the paged kernels of this package always run")
    p.add_argument("--enable-graph", action="store_true", help="replay decode steps as CUDA graphs")
    p.add_argument("--enable-paged-attn", action="store_true", help="use paged cache (the only cache here)")
    p.add_argument("--disable-prefix-caching", dest="enable_prefix_caching", action="store_false", default=False,
                   help="prefix reuse is not built; this flag is accepted and changes nothing")
    p.add_argument("--num-blocks", type=int, default=512, help="number of KV cache blocks")
    p.add_argument("--block-size", type=int, default=256, help="size of each KV cache block")
    p.add_argument("--skip-load", action="store_true", help="skip loading model weights (seeded random weights)")
    p.add_argument("--batch-size", type=int, default=1, help="copies of the prompt to generate for")
    p.add_argument("--max-batch-size", type=int, default=8, help="maximum number of live requests")
    p.add_argument("--max-new-tokens", type=int, default=512, help="maximum number of new tokens to generate")
    p.add_argument("--input-len", type=parse_list, default=10, help="input sequence length(s) of the benchmark tool: 256 | 256,1024 | [256,1024]")
    p.add_argument("--output-len", type=parse_list, default=20, help="output sequence length(s) of the benchmark tool")
    p.add_argument("--prompt", type=str, default="How are you", help="default prompt text")
    p.add_argument("--top-k", type=int, default=1)
    p.add_argument("--top-p", type=float, default=1.0)
    p.add_argument("--temperature", type=float, default=1.0)
    p.add_argument("--ignore-eos", action="store_true", help="keep generating past the end-of-sequence token")
    p.add_argument("--warmup", action="store_true", help="run one short generation before the timed one")
    p.add_argument("--log-level", type=str, default="INFO", choices=["DEBUG", "INFO", "WARNING", "ERROR", "CRITICAL"])
    # ours
    p.add_argument("--prompt-ids", type=str, default=None, help="prompt as comma-separated token ids")
    p.add_argument("--prompt-len", type=int, default=None, help="prompt of this many seeded random token ids")
    p.add_argument("--seed", type=int, default=0, help="seed of sampling, random prompts and random weights")
    p.add_argument("--chunk-size", type=int, default=2048, help="largest prompt portion in one step")
    p.add_argument("--max-num-batched-tokens", type=int, default=None, help="token budget of one step")
    p.add_argument("--admission", type=str, default="worst_case", choices=["worst_case", "optimistic"])
    p.add_argument("--write-random-model", type=str, default=None, metavar="DIR",
                   help="write config.json and model.safetensors with random weights to DIR and exit")
    p.add_argument("--config", type=str, default=None, help="config.json for --write-random-model")
    return p


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    logging.basicConfig(level=getattr(logging, args.log_level), format="%(asctime)s - %(name)s - %(levelname)s - %(message)s")
    if args.write_random_model:
        if not args.config:
            print("--write-random-model needs --config", file=sys.stderr)
            return 2
        from .config.registry import config_from_json
        from .weights.random_init import write_model_folder
        with open(args.config) as f:
            cfg = config_from_json(json.load(f))
        write_model_folder(cfg, args.seed, args.write_random_model)
        print(f"wrote {args.write_random_model}")
        return 0
    if not args.model:
        print("--model is required", file=sys.stderr)
        return 2
    from .llm import LLM, SamplingParams
    device = "cuda" if args.device in ("auto", "nvidia") else args.device
    llm = LLM(args.model, device=device, dtype=args.dtype, max_batch_size=max(args.max_batch_size, args.batch_size),
              max_tokens=args.max_new_tokens, num_blocks=args.num_blocks, block_size=args.block_size,
              temperature=args.temperature, top_p=args.top_p, top_k=args.top_k, enable_graph=args.enable_graph,
              attn_backend=args.attn, skip_load=args.skip_load, enable_prefix_caching=False,
              max_num_batched_tokens=args.max_num_batched_tokens, chunk_size=args.chunk_size, seed=args.seed,
              admission=args.admission)
    sp = SamplingParams(temperature=args.temperature, top_p=args.top_p, top_k=args.top_k,
                        max_tokens=args.max_new_tokens, ignore_eos=args.ignore_eos)
    kw = {}
    if args.prompt_ids is not None:
        kw["prompt_token_ids"] = [[int(x) for x in args.prompt_ids.split(",")]] * args.batch_size
    elif args.prompt_len is not None:
        import torch
        g = torch.Generator().manual_seed(args.seed)
        ids = torch.randint(0, llm.model_config.vocab_size, (args.prompt_len,), generator=g).tolist()
        kw["prompt_token_ids"] = [ids] * args.batch_size
    else:
        conv = [{"role": "user", "content": args.prompt}]
        kw["messages"] = [conv for _ in range(args.batch_size)]
    if args.warmup:
        w = sp.clone()
        w.max_tokens = min(4, sp.max_tokens)
        llm.generate(sampling_params=w, **kw)
    t1 = time.time()
    print("=================== start generate ====================")
    try:
        outputs = llm.generate(sampling_params=sp, **kw)
    finally:
        llm.close()
    t2 = time.time()
    n_new = 0
    for i, o in enumerate(outputs):
        print(f"Request {i}:")
        print("===Query===")
        print(o.prompt if o.prompt is not None else o.prompt_token_ids)
        print("===Response===")
        print(o.outputs[0].text if o.outputs[0].text else o.outputs[0].token_ids)
        print(f"(finish_reason: {o.finish_reason.value if o.finish_reason else None})\n")
        n_new += len(o.outputs[0].token_ids)
    print(f"total_time: {round((t2 - t1) * 1000, 2)} ms, {n_new} new tokens, {n_new / max(t2 - t1, 1e-9):.1f} tok/s")
    return 0


def bench_main(argv=None) -> int:
    """The benchmark tool in InfiniLM's manner (`examples/bench.py:592-696,731-745`): for every combination of
    --input-len and --output-len at --batch-size, generate for that many copies of a prompt and print the time to the first
    token and the prefill and decode throughputs as InfiniLM defines them (`python/infinilm/infer_engine.py:720-726`:
    prefill tok/s = batch * input_len / time of the first step(s); decode tok/s = batch * (n - 1) / time of the others).
    The prompt is seeded random token ids of the asked length (InfiniLM repeats a text to length; random weights have no text)."""
    args = build_parser().parse_args(argv)
    logging.basicConfig(level=getattr(logging, args.log_level), format="%(asctime)s - %(name)s - %(levelname)s - %(message)s")
    if not args.model:
        print("--model is required", file=sys.stderr)
        return 2
    import torch

    from .llm import LLM, SamplingParams
    ins = args.input_len if isinstance(args.input_len, list) else [args.input_len]
    outs = args.output_len if isinstance(args.output_len, list) else [args.output_len]
    device = "cuda" if args.device in ("auto", "nvidia") else args.device
    need_pages = args.batch_size * ((max(ins) + max(outs) + args.block_size - 1) // args.block_size + 1)
    llm = LLM(args.model, device=device, dtype=args.dtype, max_batch_size=max(args.max_batch_size, args.batch_size),
              max_tokens=max(outs), num_blocks=max(args.num_blocks, need_pages), block_size=args.block_size,
              enable_graph=args.enable_graph, attn_backend=args.attn, skip_load=args.skip_load,
              max_num_batched_tokens=args.max_num_batched_tokens, chunk_size=args.chunk_size, seed=args.seed, admission=args.admission)
    results = []
    try:
        for n_in in ins:
            for n_out in outs:
                if n_in + n_out > llm.model_config.max_position_embeddings:
                    print(f"[bench] input_len={n_in} + output_len={n_out} passes max_position_embeddings; skipped")
                    continue
                g = torch.Generator().manual_seed(args.seed + n_in)
                ids = torch.randint(0, llm.model_config.vocab_size, (n_in,), generator=g).tolist()
                sp = SamplingParams(temperature=args.temperature, top_p=args.top_p, top_k=args.top_k, max_tokens=n_out, ignore_eos=True)
                for timed in ([False, True] if args.warmup else [True]):
                    reqs = [llm.add_request(ids, sp if timed else SamplingParams(top_k=1, max_tokens=min(4, n_out), ignore_eos=True))
                            for _ in range(args.batch_size)]
                    torch.cuda.synchronize()
                    t0 = time.perf_counter()
                    while any(len(r.output_token_ids) < 1 for r in reqs):       # the prompts' steps, to every request's first token
                        llm.step()
                    torch.cuda.synchronize()
                    t1 = time.perf_counter()
                    while not all(r.finished for r in reqs):
                        llm.step()
                    torch.cuda.synchronize()
                    t2 = time.perf_counter()
                if any(len(r.output_token_ids) != n_out for r in reqs):
                    print("[bench] a request did not produce output_len tokens", file=sys.stderr)
                    return 1
                B = args.batch_size
                rec = {"batch_size": B, "input_len": n_in, "output_len": n_out, "ttft_ms": (t1 - t0) * 1e3,
                       "prefill_tok_s": B * n_in / (t1 - t0),
                       "itl_ms": (t2 - t1) * 1e3 / max(n_out - 1, 1), "decode_tok_s": B * (n_out - 1) / (t2 - t1) if n_out > 1 else 0.0}
                results.append(rec)
                print(f"\n Generation completed in {round((t2 - t0) * 1000, 2)} ms")
                print(f" Batchsize={B}  Per_Batch_Input_Len={n_in}  Per_Batch_New_Tokens={n_out}")
                print(f" Prefill TTFT: {round(rec['ttft_ms'], 2)} ms  Throughput: {round(rec['prefill_tok_s'], 2)} tok/s")
                if n_out > 1:
                    print(f" Decode  Avg ITL: {round(rec['itl_ms'], 2)} ms   Throughput: {round(rec['decode_tok_s'], 2)} tok/s")
    finally:
        llm.close()
    print(json.dumps({"bench": results}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
