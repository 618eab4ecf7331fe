"""Command line of the engine, in the manner of the reference's scripts (argparse, the same option
names where it has them: ``--max-running``, ``--requests``, ``--trials``, ``--out``;
benchmarks/compare/run_omniserve.py:44-61, omniserve/server.py:185-192).

    python -m omniserver_b200.cli generate --model DIR --prompt-ids 5,17,3 --max-new-tokens 16
    python -m omniserver_b200.cli generate --model DIR --prompt-file prompts.jsonl --temperature 0.8 --seed 1 --out out.json
    python -m omniserver_b200.cli random-model --config config.json --seed 0 --out DIR
    python -m omniserver_b200.cli replay --model DIR --dtype float32 --out LOGITS_DIR --max-tokens 4096 < steps.jsonl
    python -m omniserver_b200.cli bench decode --model 2b --batch 8 --steps 64 --trials 3 [--profile]
    python -m omniserver_b200.cli bench prefill --model 7b --tokens 2048
    python -m omniserver_b200.cli bench mixed --model 7b --requests 64 --max-running 64

Prompts are token ids: the tokenizer is outside the engine. ``--prompt-file`` holds one JSON list
of ids per line.
"""

from __future__ import annotations

import argparse
import json
import sys
import time
from typing import List

from .config.engine_config import DEFAULT_PAGE_SIZE


def _prompts(args) -> List[List[int]]:
    out: List[List[int]] = []
    for p in args.prompt_ids or []:
        out.append([int(t) for t in p.replace(" ", "").split(",") if t])
    if args.prompt_file:
        with open(args.prompt_file) as f:
            for line in f:
                line = line.strip()
                if line:
                    out.append([int(t) for t in json.loads(line)])
    if args.requests and out:
        out = [out[i % len(out)] for i in range(args.requests)]
    if not out:
        raise SystemExit("generate: give --prompt-ids or --prompt-file")
    return out


def cmd_generate(args) -> int:
    import torch

    from . import EngineConfig, LLMEngine, Request, SamplingParams, SchedulerConfig
    prompts = _prompts(args)
    ec = EngineConfig(dtype=args.dtype, page_size=args.page_size, max_cache_tokens=args.max_cache_tokens,
                      max_requests=max(args.max_running, 1) + 1, device=args.device, cuda_graphs=not args.no_cuda_graph)
    sc = SchedulerConfig(max_running=args.max_running, max_prefill_per_step=args.max_prefill_per_step,
                         max_prefill_tokens=args.max_prefill_tokens, max_seq_len=args.max_seq_len)
    t0 = time.perf_counter()
    with torch.inference_mode():
        eng = LLMEngine.from_model_dir(args.model, ec, sc, seed=args.seed)
        load_s = time.perf_counter() - t0
        trials = []
        outs = {}
        for trial in range(max(1, args.trials)):
            ids = []
            for i, p in enumerate(prompts):
                sp = SamplingParams(max_new_tokens=args.max_new_tokens, temperature=args.temperature,
                                    stop_token_ids=list(args.stop_token_ids or []), ignore_eos=args.ignore_eos)
                ids.append(eng.add_request(Request(prompt=p, sampling=sp, request_id=f"req-{trial}-{i}")))
            t1 = time.perf_counter()
            outs = eng.run_until_complete()
            torch.cuda.synchronize()
            wall = time.perf_counter() - t1
            toks = sum(len(outs[i]) for i in ids)
            trials.append({"wall_s": wall, "tokens": toks, "tok_per_s": toks / wall, "req_per_s": len(ids) / wall})
            last_ids = ids
    result = {"backend": "omniserver_b200", "dtype": args.dtype, "n_requests": len(prompts), "load_s": round(load_s, 3),
              "trials": trials, "outputs": [outs[i] for i in last_ids], "stats": eng.stats()}
    text = json.dumps(result, indent=2 if args.out else None)
    if args.out:
        with open(args.out, "w") as f:
            f.write(text)
        med = sorted(t["tok_per_s"] for t in trials)[len(trials) // 2]
        print(f"[omniserver_b200] {len(prompts)} reqs x{len(trials)} trials -> median {med:.1f} tok/s")
    else:
        print(text)
    return 0


def cmd_random_model(args) -> int:
    from .weights import write_random_model
    with open(args.config) as f:
        cfg = json.load(f)
    d = write_random_model(cfg, args.seed, args.out, store_dtype=args.store_dtype, std=args.std, norm_noise=args.norm_noise)
    print(f"wrote {d}/config.json and {d}/model.safetensors (seed {args.seed}, {args.store_dtype})")
    return 0


def cmd_replay(args) -> int:
    from .replay import main as replay_main
    argv = ["--model", args.model, "--dtype", args.dtype, "--out", args.out, "--max-tokens", str(args.max_tokens),
            "--page-size", str(args.page_size)]
    return replay_main(argv)


def cmd_bench(args) -> int:
    """Throughput of random-weight models of the architecture's sizes (see omniserver_b200/benchmark.py); JSON out."""
    import torch

    from . import benchmark as bm
    if not torch.cuda.is_available():
        raise SystemExit("bench: no CUDA device is visible")
    pk = bm.read_peaks(args.peaks) if args.peaks else (*bm.FALLBACK_PEAKS, "fallback")
    if args.what == "mixed":
        b = bm.Bench(args.model, args.layers, args.max_running, args.prompt_hi, args.max_new_tokens + 64, args.page_size, pk,
                     graphs=not args.no_cuda_graph, pool_tokens=args.max_running * (args.prompt_hi + args.max_new_tokens + 64) + 4096,
                     max_requests=args.max_running)
        out = b.mixed(args.requests, args.prompt_lo, args.prompt_hi, args.max_new_tokens, args.chunk, args.max_running,
                      trials=args.trials)
    elif args.what == "prefill":
        b = bm.Bench(args.model, args.layers, 1, args.tokens, 64, args.page_size, pk, graphs=not args.no_cuda_graph)
        out = b.prefill(args.tokens, trials=args.trials)
        if args.profile:
            out["kernels"] = b.profile(1, prefill_tokens=args.tokens)["prefill"]
    else:
        b = bm.Bench(args.model, args.layers, args.batch, args.ctx, args.max_new_tokens, args.page_size, pk,
                     graphs=not args.no_cuda_graph)
        r = b.decode(args.batch, args.steps, args.warmup, trials=args.trials)
        out = {"tokens_per_s": round(r["tokens_per_s"], 1), "ms_per_step": round(r["ms_per_step"], 4), "trials_ms": r["trials_ms"],
               "bytes_per_step": r["bytes_per_step"], "achieved_gbs": round(r["achieved_gbs"], 1), "frac": round(r["frac"], 4),
               "launches": r["launches"]}
        if args.profile:
            out["kernels"] = b.profile(args.batch)["decode"]
    out["config"] = bm.config_of(b, args.batch if args.what == "decode" else (args.max_running if args.what == "mixed" else 1))
    out["peaks"] = {"hbm_gbs": pk[0], "bf16_tflops": pk[1], "of": pk[2]}
    text = json.dumps(out, indent=2 if args.out else None)
    if args.out:
        with open(args.out, "w") as f:
            f.write(text)
    else:
        print(text)
    return 0


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="omniserver_b200", description=__doc__.split("\n\n")[0])
    sub = ap.add_subparsers(dest="command", required=True)

    g = sub.add_parser("generate", help="generate tokens for prompts given as token ids")
    g.add_argument("--model", required=True, help="folder with config.json and model*.safetensors")
    g.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    g.add_argument("--prompt-ids", action="append", help="comma-separated token ids; may be given several times")
    g.add_argument("--prompt-file", help="file with one JSON list of token ids per line")
    g.add_argument("--requests", type=int, default=0, help="repeat the prompts round-robin up to this many requests")
    g.add_argument("--trials", type=int, default=1)
    g.add_argument("--max-new-tokens", type=int, default=128)
    g.add_argument("--temperature", type=float, default=0.0, help="0 means greedy")
    g.add_argument("--seed", type=int, default=0)
    g.add_argument("--stop-token-ids", type=int, nargs="*")
    g.add_argument("--ignore-eos", action="store_true")
    g.add_argument("--max-running", type=int, default=8)
    g.add_argument("--max-prefill-per-step", type=int, default=1)
    g.add_argument("--max-prefill-tokens", type=int, default=8192)
    g.add_argument("--max-seq-len", type=int, default=4096)
    g.add_argument("--page-size", type=int, default=DEFAULT_PAGE_SIZE)
    g.add_argument("--max-cache-tokens", type=int, default=32768)
    g.add_argument("--no-cuda-graph", action="store_true", help="launch decode steps kernel by kernel")
    g.add_argument("--device", default="cuda:0")
    g.add_argument("--out", type=str, default=None)
    g.set_defaults(fn=cmd_generate)

    r = sub.add_parser("random-model", help="write a model folder with random weights from a config.json and a seed")
    r.add_argument("--config", required=True)
    r.add_argument("--seed", type=int, default=0)
    r.add_argument("--out", required=True)
    r.add_argument("--store-dtype", default="bfloat16", choices=["bfloat16", "float32", "float16"])
    r.add_argument("--std", type=float, default=0.02)
    r.add_argument("--norm-noise", type=float, default=0.0)
    r.set_defaults(fn=cmd_random_model)

    b = sub.add_parser("bench", help="throughput with random weights: decode steps, a prompt, or a mixed run")
    b.add_argument("what", choices=["decode", "prefill", "mixed"])
    b.add_argument("--model", default="2b", choices=["2b", "7b", "72b"], help="layer sizes of the Qwen2-VL text decoder")
    b.add_argument("--layers", type=int, default=None, help="fewer layers than the model has")
    b.add_argument("--batch", type=int, default=8)
    b.add_argument("--ctx", type=int, default=2048, help="tokens each request holds when decoding starts")
    b.add_argument("--tokens", type=int, default=2048, help="prompt length of 'prefill'")
    b.add_argument("--steps", type=int, default=64)
    b.add_argument("--warmup", type=int, default=8)
    b.add_argument("--trials", type=int, default=3)
    b.add_argument("--requests", type=int, default=64)
    b.add_argument("--max-running", type=int, default=64)
    b.add_argument("--prompt-lo", type=int, default=128)
    b.add_argument("--prompt-hi", type=int, default=4096)
    b.add_argument("--chunk", type=int, default=2048, help="most prompt tokens per step of 'mixed'")
    b.add_argument("--max-new-tokens", type=int, default=256)
    b.add_argument("--page-size", type=int, default=DEFAULT_PAGE_SIZE)
    b.add_argument("--no-cuda-graph", action="store_true")
    b.add_argument("--profile", action="store_true", help="time per class of kernels inside real steps")
    b.add_argument("--peaks", default=None, help="a MEASURED_PEAKS.json (hbm_gbs, bf16_tflops) for the fractions")
    b.add_argument("--out", type=str, default=None)
    b.set_defaults(fn=cmd_bench)

    p = sub.add_parser("replay", help="feed token ids from stdin step by step and write logits (see bin/trace_run)")
    p.add_argument("--model", required=True)
    p.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    p.add_argument("--out", required=True)
    p.add_argument("--max-tokens", type=int, required=True)
    p.add_argument("--page-size", type=int, default=DEFAULT_PAGE_SIZE)
    p.set_defaults(fn=cmd_replay)
    return ap


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    return args.fn(args)


if __name__ == "__main__":
    sys.exit(main())
