"""Benchmark of the engine's headline metric: decoded tokens per second on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers L] [--impl ours|reference]

Default run: the Qwen2-VL-2B text decoder's layer sizes with random weights (seed 2), bfloat16,
a batch of 8 requests each holding a 2,048-token context, pages of 16 tokens.  A "step" is one
decode step of the whole batch.  It prints one JSON line:

* ``value``: decoded tokens per second, timed with CUDA events around K steps of the step
  function plus sampling (the device time of the steps including the gaps between kernels);
* ``e2e``: the same through the Python entry point (LLMEngine.step): scheduler, host token ids in
  (pinned staging buffer, one host-to-device copy per step) and sampled ids out;
* ``prefill``: one 2,048-token prompt through the step function; ``frac`` = flops / time / bf16 peak;
* ``roofline``: bytes a decode step has to read (every weight once, the live requests' keys and
  values) / its time, against the measured copy bandwidth;
* ``points``: decode at batch 1 and 64.

Peaks come from MEASURED_PEAKS.json beside this file when present, else 6.65 TB/s and 1.59 PFLOP/s.
Weights (3 GB) and caches are far larger than the L2 (126 MB), so no flush is needed between steps.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

MODEL_2B = {
    "architectures": ["Qwen2VLForConditionalGeneration"], "model_type": "qwen2_vl",
    "hidden_size": 1536, "num_hidden_layers": 28, "num_attention_heads": 12, "num_key_value_heads": 2,
    "head_dim": 128, "intermediate_size": 8960, "vocab_size": 151936, "rms_norm_eps": 1e-6,
    "rope_theta": 1000000.0, "rope_scaling": {"type": "mrope", "mrope_section": [16, 24, 24]},
    "tie_word_embeddings": True, "hidden_act": "silu", "use_sliding_window": False,
    "max_position_embeddings": 4096,
}
FULL_LAYERS = 28
CONTEXT = 2048
NEW_TOKENS = 256
PAGE_SIZE = 16       # tokens per cache page (--page-size)
SEED = 2


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    hbm, tf, src = 6650.0, 1590.0, "fallback"
    if os.path.isfile(p):
        try:
            with open(p) as f:
                d = json.load(f)
            hbm = float(d.get("hbm_gbs", hbm))
            tf = float(d.get("bf16_tflops", tf))
            src = "measured"
        except Exception:
            pass
    return hbm, tf, src


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc = None
        self.path = os.path.join(tempfile.gettempdir(), "osb_bench_clocks_%d.csv" % os.getpid())

    def start(self):
        try:
            self.f = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=self.f, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.f.close()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        with open(self.path) as f:
            for line in f:
                parts = [x.strip() for x in line.split(",")]
                if len(parts) < 6:
                    continue
                try:
                    sm.append(float(parts[0]))
                    mx.append(float(parts[1]))
                except ValueError:
                    continue
                for n, v in zip(names, parts[2:6]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
        if sm:
            out = {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}
        return out


def model_numbers(cfg, layers):
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    per_layer = H * (nh + 2 * nkv) * hd + (nh + 2 * nkv) * hd + nh * hd * H + 2 * I * H + I * H + 2 * H
    params = layers * per_layer + V * H + H
    kv_per_token = layers * 2 * nkv * hd * 2            # bytes, bf16
    weight_bytes = params * 2
    return dict(per_layer=per_layer, params=params, kv_per_token=kv_per_token, weight_bytes=weight_bytes)


def prefill_flops(cfg, layers, T):
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    gemm = 2 * T * (H * (nh + 2 * nkv) * hd + nh * hd * H + 3 * I * H)
    attn = 2 * 2 * nh * hd * (T * (T + 1) // 2)         # causal QK^T and PV
    return layers * (gemm + attn) + 2 * H * V            # head at one row


def run_ours(args):
    import torch
    if not torch.cuda.is_available():
        print(json.dumps({"error": "no CUDA device"}))
        return 1
    from omniserver_b200 import EngineConfig, LLMEngine, Request, SamplingParams, SchedulerConfig, build_runner, ops
    from omniserver_b200.engine.step import StepEntry
    from omniserver_b200.sampling import Sampler

    hbm_peak, tf_peak, peak_src = peaks()
    cfg = dict(MODEL_2B)
    cfg["num_hidden_layers"] = args.layers
    nums = model_numbers(cfg, args.layers)
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    g = torch.Generator().manual_seed(SEED)
    max_batch = max(args.batch, 1 if args.no_points else 64)
    ctx_total = CONTEXT + NEW_TOKENS
    pool_tokens = max_batch * (-(-ctx_total // 64) * 64) + 4096
    ec = EngineConfig(dtype="bfloat16", page_size=PAGE_SIZE, max_cache_tokens=pool_tokens, max_requests=max_batch + 2,
                      check_device_errors=False, cuda_graphs=not args.no_graphs)
    t0 = time.time()
    runner = build_runner(config=cfg, seed=SEED, engine_config=ec, random_on_device=True)
    torch.cuda.synchronize()
    build_s = time.time() - t0
    K = ops.kernels()
    sampler_k = K

    def new_prompt(n):
        return torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist()

    # ------------------------------------------------------------------ prefill: one 2,048-token prompt
    def prefill_once(rid):
        runner.start_request(rid)
        lg = runner.step([StepEntry(rid, new_prompt(CONTEXT), want=[CONTEXT - 1])])
        return lg

    with torch.inference_mode():
        for i in range(0 if args.only == "decode" else 3):
            prefill_once(f"pw{i}")
            runner.end_request(f"pw{i}")
        torch.cuda.synchronize()
        times = []
        for i in range(1 if args.only == "decode" else 5):
            toks = new_prompt(CONTEXT)
            torch.cuda.nvtx.range_push("timed_prefill")
            runner.start_request(f"p{i}")
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            runner.step([StepEntry(f"p{i}", toks, want=[CONTEXT - 1])])
            e1.record()
            torch.cuda.synchronize()
            torch.cuda.nvtx.range_pop()
            times.append(e0.elapsed_time(e1))
            runner.end_request(f"p{i}")
        pre_ms = statistics.median(times)
    pflops = prefill_flops(cfg, args.layers, CONTEXT)
    prefill = {"value": round(CONTEXT / (pre_ms / 1e3), 1), "tokens": CONTEXT, "ms": round(pre_ms, 3),
               "frac": round(pflops / (pre_ms / 1e3) / (tf_peak * 1e12), 4), "tflops": round(pflops / (pre_ms / 1e3) / 1e12, 1),
               "peak_tflops": tf_peak, "of": peak_src}

    # ------------------------------------------------------------------ decode through the step function
    def decode_run(B, steps, warmup, sample_clocks=False):
        """Decode steps through the step function, the way the engine drives it: the sampled tokens stay on
        the device for the next step's embedding lookup and are read on the host one step later, so the
        host's planning of step t+1 overlaps the device's work on step t. Every step copies its metadata
        from pinned host memory and brings its tokens back to the host."""
        rids = [f"d{B}_{i}" for i in range(B)]
        sampler = Sampler(SEED)
        with torch.inference_mode():
            for r in rids:
                runner.start_request(r)
                lg = runner.step([StepEntry(r, new_prompt(CONTEXT), want=[CONTEXT - 1])], copy_logits=False)
                sampler.sample_async(lg, None, runner.last_token, runner.logit_slots).result()
            entries = [StepEntry(r, [0], want=[0], from_device=True) for r in rids]

            def launch():
                lg = runner.step(entries, copy_logits=False)
                return sampler.sample_async(lg, None, runner.last_token, runner.logit_slots)

            def run(n):
                prev, got = None, 0
                for _ in range(n):
                    h = launch()
                    if prev is not None:
                        got += len(prev.result())
                    prev = h
                got += len(prev.result())
                return got

            run(warmup)
            torch.cuda.synchronize()
            clocks = ClockSampler() if sample_clocks else None
            if clocks:
                clocks.start()
                time.sleep(0.3)
            l0 = K.launches
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            torch.cuda.nvtx.range_push("timed_decode")
            e0.record()
            got = run(steps)
            e1.record()
            torch.cuda.synchronize()
            torch.cuda.nvtx.range_pop()
            assert got == steps * B
            ms = e0.elapsed_time(e1) / steps
            launches = K.launches - l0
            ck = clocks.stop() if clocks else None
            ctx_mid = CONTEXT + warmup + steps / 2
            for r in rids:
                runner.end_request(r)
        return ms, launches, ck, ctx_mid

    ms, launches, clocks, ctx_mid = decode_run(args.batch, args.steps, args.warmup, sample_clocks=True)
    value = args.batch / (ms / 1e3)
    step_bytes = nums["weight_bytes"] + args.batch * ctx_mid * nums["kv_per_token"]
    achieved = step_bytes / (ms / 1e3) / 1e9
    roofline = {"bound": "hbm", "achieved": round(achieved, 1), "peak": hbm_peak, "unit": "GB/s",
                "frac": round(achieved / hbm_peak, 4), "bytes_per_step": int(step_bytes), "of": peak_src}

    points = {}
    if not args.no_points and args.only == "all":
        for B in (1, 64):
            pms, _, _, _ = decode_run(B, max(8, args.steps // 2), max(3, args.warmup // 2))
            points[f"decode_b{B}"] = round(B / (pms / 1e3), 1)

    # ------------------------------------------------------------------ end to end through LLMEngine
    e2e = None
    with torch.inference_mode():
        # all prompts enter in one step, so that every request decodes in every timed step
        eng = LLMEngine(runner, SchedulerConfig(max_running=args.batch, max_prefill_per_step=args.batch,
                                                max_prefill_tokens=CONTEXT * args.batch, max_seq_len=4096), seed=SEED)
        n_new = args.warmup + args.steps + 1
        for i in range(args.batch if args.only == "all" else 0):
            eng.add_request(Request(prompt=new_prompt(CONTEXT),
                                    sampling=SamplingParams(max_new_tokens=n_new, ignore_eos=True)))
        while any(s.num_streamed < 1 + args.warmup for s in eng.sequences()):
            eng.step()
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        n_steps = e2e_tokens = 0
        while eng.has_unfinished():
            e2e_tokens += sum(len(d.new_token_ids) for d in eng.step())     # tokens that reached the host
            n_steps += 1
        torch.cuda.synchronize()
        e2e_s = max(time.perf_counter() - t1, 1e-9)
    e2e = {"value": round(e2e_tokens / e2e_s, 1), "unit": "tokens/s", "h2d_bytes_per_step": runner.last_h2d_bytes,
           "d2h_bytes_per_step": 4 * args.batch, "steps": n_steps, "tokens": e2e_tokens}

    line = {
        "metric": "decode tokens/s (Qwen2-VL-2B text decoder, batch %d, 2048-token contexts)" % args.batch,
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: uniform random token ids, random weights (seed 2)",
        "config": {"model": "Qwen2-VL-2B text decoder (random weights)", "layers": args.layers,
                   "layers_of_model": FULL_LAYERS, "hidden_size": 1536, "heads": 12, "kv_heads": 2, "head_dim": 128,
                   "intermediate_size": 8960, "vocab_size": 151936, "tied_head": True, "global_batch": args.batch,
                   "seq_len": CONTEXT, "new_tokens": NEW_TOKENS, "page_size": PAGE_SIZE, "parallelism": "single GPU",
                   "l2": "inputs (3 GB of weights) larger than L2, no flush"},
        "clocks": clocks, "e2e": e2e, "gpu_launches": launches, "prefill": prefill, "roofline": roofline,
        "points": points, "build_s": round(build_s, 1),
    }
    print(json.dumps(line))
    return 0


def run_reference(args):
    # The reference has no setup.py/pyproject.toml, so pip cannot install it; its generation path
    # also needs a downloaded checkpoint with tokenizer and vLLM's FlashAttention binary.
    print(json.dumps({"impl": "reference", "unavailable":
                      "omniserve has no setup.py/pyproject.toml (pip install fails) and its runner needs a downloaded "
                      "Qwen2-VL checkpoint and tokenizer, which do not exist offline"}))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=FULL_LAYERS)
    ap.add_argument("--page-size", type=int, default=PAGE_SIZE, help="tokens per cache page")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 and 64 points")
    ap.add_argument("--no-graphs", action="store_true", help="launch every kernel of a decode step from the host")
    ap.add_argument("--only", default="all", choices=["all", "decode"],
                    help="'decode': skip the prefill repeats, the points and the end-to-end run (for profiling)")
    args = ap.parse_args()
    globals()["PAGE_SIZE"] = args.page_size
    if args.impl == "reference":
        return run_reference(args)
    if args.gpus != 1:
        print("bench.py: this engine runs on one GPU; --gpus %d is not supported" % args.gpus)
        return 2
    if args.warmup < 3:
        args.warmup = 3
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
