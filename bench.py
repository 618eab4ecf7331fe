"""Benchmark of the engine's headline metric: decoded tokens per second on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--model 2b|7b|72b] [--layers L]
                    [--workload decode|mixed] [--profile] [--impl ours|reference]

Default run: the Qwen2-VL-2B text decoder's layer sizes with random weights (seed 2), bfloat16,
a batch of 8 requests each holding a 2,048-token context, pages of 16 tokens.  A "step" is one
decode step of the whole batch.  It prints one JSON line:

* ``value``: decoded tokens per second, timed with CUDA events around K steps of the step
  function plus sampling (the device time of the steps including the gaps between kernels): the
  median of --trials such runs;
* ``e2e``: the same through the Python entry point (LLMEngine.step): scheduler, host token ids in
  (pinned staging buffer, one host-to-device copy per step) and sampled ids out;
* ``prefill``: one 2,048-token prompt through the step function; ``frac`` = flops / time / bf16 peak, the time from
  the call to the logits with the device idle before (``back_to_back_ms``: per step when four follow one another);
* ``roofline``: bytes a decode step has to read (every weight once, the live requests' keys and
  values) / its time, against the measured copy bandwidth;
* ``points``: decode at batch 1 and 64 (tokens/s, ms per step, fraction of the roofline), and for the 7B and
  72B sizes of the same architecture: the 7B decode point and mixed continuous-batching run (64 requests,
  prompts of 128 to 4,096 tokens, 256 new tokens, portions of 2,048), the 72B decode points and prefill;
* ``roofline.kernels`` / ``prefill.kernels``: time, achieved rate and fraction per class of kernels (matrix
  products, attention, ...) from events recorded inside real steps.

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
PAGE_SIZE = 32       # tokens per cache page (--page-size); the engine's default
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
    """Our arm: the measurements of omniserver_b200.benchmark (the same code as ``python -m omniserver_b200.cli bench``)
    put together into the one JSON line of the contract."""
    import torch
    if not torch.cuda.is_available():
        print(json.dumps({"error": "no CUDA device"}))
        return 1
    from omniserver_b200 import benchmark as bm
    torch.cuda.set_device(0)
    pk = bm.read_peaks(os.path.join(ROOT, "MEASURED_PEAKS.json"))
    model = args.model
    big = model == "72b"
    batches = (1, 8, 16) if big else (1, 8, 64)
    batch = args.batch
    points_on = not args.no_points and args.only == "all"
    max_batch = max([batch] + (list(batches) if points_on else []))
    new_tokens = 128 if big else NEW_TOKENS
    b = bm.Bench(model, args.layers, max_batch, CONTEXT, new_tokens, args.page_size, pk, graphs=not args.no_graphs)
    fast = args.only == "decode"
    prefill = b.prefill(CONTEXT, trials=1 if fast else 5, warmup=0 if fast else 3)
    main = b.decode(batch, args.steps, args.warmup, trials=1 if fast else args.trials, clocks=True)
    points = {}
    e2e = None
    kernels = None
    if not fast:
        e2e = b.e2e_decode(batch, args.steps, args.warmup)     # (before the points: same state of the process as `value`)
    if points_on:
        for B in sorted(batches, reverse=True):
            if B != batch:
                r = b.decode(B, max(8, args.steps // 2), max(3, args.warmup // 2), trials=args.trials)
                points[f"decode_b{B}"] = round(r["tokens_per_s"], 1)
                points[f"decode_b{B}_ms"] = round(r["ms_per_step"], 4)
                points[f"decode_b{B}_frac"] = round(r["frac"], 4)
    if not fast and (args.profile or points_on):
        kernels = b.profile(batch)
    line = {
        "metric": "decode tokens/s (Qwen2-VL-%s text decoder, batch %d, %d-token contexts)" % (model.upper(), batch, CONTEXT),
        "value": round(main["tokens_per_s"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(main["ms_per_step"], 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: uniform random token ids, random weights (seed %d)" % b.seed,
        "config": bm.config_of(b, batch), "clocks": main["clocks"], "e2e": e2e, "gpu_launches": main["launches"],
        "trials_ms": main["trials_ms"], "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(main["achieved_gbs"], 1), "peak": pk[0], "unit": "GB/s",
                     "frac": round(main["frac"], 4), "bytes_per_step": main["bytes_per_step"], "of": pk[2]},
        "points": points, "build_s": round(b.build_s, 1),
    }
    if kernels is not None:
        line["roofline"]["kernels"] = kernels.get("decode")
        line["prefill"]["kernels"] = kernels.get("prefill")
    b.close()
    # the other sizes of the architecture: the 7B mixed run and decode point, the 72B decode points and prefill
    if points_on and model == "2b" and not args.no_other_sizes:
        try:
            b7 = bm.Bench("7b", None, 64, 4096, 320, args.page_size, pk, graphs=not args.no_graphs,
                          pool_tokens=64 * 4416 + 4096, max_requests=64)
            r = b7.decode(8, max(8, args.steps // 2), max(3, args.warmup // 2), trials=args.trials)
            points.update({"7b_decode_b8": round(r["tokens_per_s"], 1), "7b_decode_b8_ms": round(r["ms_per_step"], 4),
                           "7b_decode_b8_frac": round(r["frac"], 4)})
            m = b7.mixed(trials=args.trials)
            points.update({"7b_mixed_output_tok_s": m["output_tokens_per_s"], "7b_mixed_prefill_tok_s": m["prefill_tokens_per_s"],
                           "7b_mixed_frac": m["roofline_frac"], "7b_mixed_wall_s": m["wall_s"]})
            b7.close()
        except Exception as e:      # a point that cannot be measured is left out, with the reason
            points["7b_error"] = f"{type(e).__name__}: {str(e)[:160]}"
        try:
            need = bm.model_numbers(bm.MODELS["72b"])["stored_bytes"] + 16 * 2304 * bm.model_numbers(bm.MODELS["72b"])["kv_per_token"]
            if bm.free_gpu_bytes() < need + (6 << 30):
                raise MemoryError("%.0f GB free, the 72B sizes need %.0f GB" % (bm.free_gpu_bytes() / 1e9, need / 1e9))
            b72 = bm.Bench("72b", None, 16, CONTEXT, 128, args.page_size, pk, graphs=not args.no_graphs)
            for B in (1, 8, 16):
                r = b72.decode(B, 8, 3, trials=1)
                points.update({f"72b_decode_b{B}": round(r["tokens_per_s"], 1), f"72b_decode_b{B}_ms": round(r["ms_per_step"], 3),
                               f"72b_decode_b{B}_frac": round(r["frac"], 4)})
            p72 = b72.prefill(CONTEXT, trials=3, warmup=1, back_to_back=1)
            points.update({"72b_prefill_tok_s": p72["value"], "72b_prefill_ms": p72["ms"], "72b_prefill_frac": p72["frac"]})
            sustained = bm.read_sustained_tflops(os.path.join(ROOT, "MEASURED_PEAKS.json"))
            if sustained:
                # a step of a quarter of a second runs under the power cap: also against the library's rate there
                points["72b_prefill_frac_of_sustained"] = round(p72["tflops"] / sustained, 4)
            b72.close()
        except Exception as e:
            points["72b_error"] = f"{type(e).__name__}: {str(e)[:160]}"
    if args.workload == "mixed":
        bmx = bm.Bench(model, args.layers, 64, 4096, 320, args.page_size, pk, graphs=not args.no_graphs,
                       pool_tokens=64 * 4416 + 4096, max_requests=64)
        line["mixed"] = bmx.mixed(trials=args.trials)
        bmx.close()
    print(json.dumps(line))
    return 0


def _reference_root():
    """Where the unmodified reference package lies: the copy under baseline/_ref (it travels with the
    repository's snapshot), else a checkout named by OMNISERVE_REFERENCE."""
    for p in (os.path.join(ROOT, "baseline", "_ref"), os.environ.get("OMNISERVE_REFERENCE", "")):
        if p and os.path.isdir(os.path.join(p, "omniserve")):
            return p
    return None


def run_reference(args):
    """The reference arm: omniserve's own LLMEngine -> Scheduler -> MultimodalRunner -> Qwen2LLM ->
    PreallocatedKVCache (Triton norm/activation kernels, vLLM's FlashAttention, cuBLAS), unmodified, on the
    same model sizes, batch, context and step counts. The only code of this file on that path is the adapter
    below, which stands where omniserve's Qwen2VLAdapter loads a checkpoint, a tokenizer and a vision tower
    (none exist offline): it holds the reference's Qwen2LLM in fp16 (its only precision) filled with random
    weights through the reference's own load_from_hf, and hands token ids through. Nothing of
    omniserver_b200 is imported here."""
    def unavailable(why):
        print(json.dumps({"impl": "reference", "unavailable": " ".join(str(why).split())[:400]}))
        return 0

    root = _reference_root()
    if root is None:
        return unavailable("no copy of the reference (baseline/_ref/omniserve) beside bench.py")
    sys.path.insert(0, root)
    try:
        import torch
        if not torch.cuda.is_available():
            return unavailable("no CUDA device is visible to the reference arm")
        from omniserve import LLMEngine, Request, SamplingParams, SchedulerConfig
        from omniserve.model import Qwen2Config, Qwen2LLM, load_from_hf
        from omniserve.model.positions import IMAGE_TOKEN_ID
        from omniserve.models.base import VLMAdapter
        from omniserve.models.qwen2_vl import Qwen2VLAdapter
        from omniserve.runners.multimodal import MultimodalRunner
        from vllm.vllm_flash_attn.flash_attn_interface import flash_attn_varlen_func  # noqa: F401  (its attention)
        import triton  # noqa: F401  (its norm and activation kernels)
    except Exception as e:  # the reason must be the error raised on this machine
        return unavailable(f"importing the reference's stack failed: {type(e).__name__}: {e}")

    hbm_peak, tf_peak, peak_src = peaks()
    cfg = dict(MODEL_2B)
    if args.layers != FULL_LAYERS:
        return unavailable("the reference arm runs the whole model only (omniserve's Qwen2Config is fixed at 28 layers)")
    dev = "cuda"
    torch.cuda.set_device(0)

    class RandomWeightsAdapter(VLMAdapter):
        """Token ids in, token ids out; the model and the position rules are omniserve's own."""

        def __init__(self):
            self.device = dev
            self.image_token_id = IMAGE_TOKEN_ID
            self.eos_ids = set()                    # the timed requests run to max_new_tokens, as in our arm
            rcfg = Qwen2Config()                    # the reference's defaults are the 2B sizes
            for ours, theirs in (("hidden_size", "hidden_size"), ("num_hidden_layers", "num_layers"),
                                 ("num_attention_heads", "num_heads"), ("num_key_value_heads", "num_kv_heads"),
                                 ("head_dim", "head_dim"), ("intermediate_size", "intermediate_size"),
                                 ("vocab_size", "vocab_size")):
                assert getattr(rcfg, theirs) == cfg[ours], (ours, getattr(rcfg, theirs), cfg[ours])
            self._llm = Qwen2LLM(rcfg).half().to(dev)
            g = torch.Generator(device=dev).manual_seed(SEED)
            H, I, V = rcfg.hidden_size, rcfg.intermediate_size, rcfg.vocab_size
            q, kv = rcfg.num_heads * rcfg.head_dim, rcfg.num_kv_heads * rcfg.head_dim

            def rnd(*shape):
                return (torch.randn(shape, generator=g, device=dev, dtype=torch.float32) * 0.02).half()

            sd = {"model.embed_tokens.weight": rnd(V, H), "model.norm.weight": torch.ones(H, device=dev).half()}
            for i in range(rcfg.num_layers):
                p = f"model.layers.{i}."
                sd.update({
                    p + "self_attn.q_proj.weight": rnd(q, H), p + "self_attn.q_proj.bias": rnd(q),
                    p + "self_attn.k_proj.weight": rnd(kv, H), p + "self_attn.k_proj.bias": rnd(kv),
                    p + "self_attn.v_proj.weight": rnd(kv, H), p + "self_attn.v_proj.bias": rnd(kv),
                    p + "self_attn.o_proj.weight": rnd(H, q), p + "mlp.gate_proj.weight": rnd(I, H),
                    p + "mlp.up_proj.weight": rnd(I, H), p + "mlp.down_proj.weight": rnd(H, I),
                    p + "input_layernorm.weight": torch.ones(H, device=dev).half(),
                    p + "post_attention_layernorm.weight": torch.ones(H, device=dev).half()})
            load_from_hf(self._llm, sd)
            self._llm = self._llm.eval()
            self.num_layers, self.num_kv_heads, self.head_dim = rcfg.num_layers, rcfg.num_kv_heads, rcfg.head_dim

        def preprocess(self, images):
            return None, None

        def encode_prompt(self, prompt, grids):
            return list(prompt)

        def embed_tokens(self, input_ids):
            return self._llm.embed_tokens(input_ids)

        def vision_embed(self, pixel_values, grids):
            raise RuntimeError("text-only benchmark")

        # the position rules and the forward are the reference adapter's own bodies, called unchanged
        def prefill_positions(self, input_ids, grids):
            return Qwen2VLAdapter.prefill_positions(self, input_ids, grids)

        def decode_positions(self, write_pos, rope_deltas):
            return Qwen2VLAdapter.decode_positions(self, write_pos, rope_deltas)

        def llm(self, embeds, positions, attn_mask, cache, logits_indices=None):
            return Qwen2VLAdapter.llm(self, embeds, positions, attn_mask, cache, logits_indices=logits_indices)

        def detokenize(self, token_ids):
            return ""

    gen = torch.Generator().manual_seed(SEED)

    def new_prompt(n):
        return torch.randint(0, cfg["vocab_size"], (n,), generator=gen).tolist()

    try:
        t0 = time.time()
        adapter = RandomWeightsAdapter()
        torch.cuda.synchronize()
        build_s = time.time() - t0
    except Exception as e:
        return unavailable(f"building the reference's model failed: {type(e).__name__}: {e}")

    def say(msg):
        print(f"[bench reference] {msg}", file=sys.stderr, flush=True)

    # omniserve's own benchmark packs at most 16,384 prompt tokens into one forward
    # (benchmarks/compare/run_omniserve.py:28-29); its Triton activation kernel indexes rows in 32-bit
    # (omniserve/kernels/fused_ops.py:111-119), which 131,072 packed rows of 17,920 columns overflow.
    PACKED_PREFILL_TOKENS = 16384

    def decode_run(B, steps, warmup, use_graph, sample_clocks=False):
        """B requests of CONTEXT tokens through omniserve's engine; returns device-timed ms per decode step
        (CUDA events around its runner.decode), end-to-end tokens/s through LLMEngine.step (wall clock,
        token ids read on the host every step, as the reference does), and the first prefill step's wall time."""
        per_step = max(1, min(B, PACKED_PREFILL_TOKENS // CONTEXT))
        admit_steps = -(-B // per_step)
        n_new = admit_steps + 2 * (warmup + steps) + 2
        max_len = -(-(CONTEXT + n_new + 1) // 256) * 256       # its cache is one page of max_len tokens per request
        say(f"batch {B}: runner (graph={use_graph}, max_len={max_len})")
        runner = MultimodalRunner(adapter, max_running=B, max_len=max_len, use_graph=use_graph)
        eng = LLMEngine(runner, SchedulerConfig(max_running=B, max_prefill_per_step=per_step,
                                                max_prefill_tokens=per_step * CONTEXT, max_seq_len=4096))
        for _ in range(B):
            eng.add_request(Request(prompt=new_prompt(CONTEXT), sampling=SamplingParams(max_new_tokens=n_new)))
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        eng.step()                                             # up to 8 prompts packed into one prefill; one token each
        torch.cuda.synchronize()
        prefill_s = time.perf_counter() - t1
        while eng.scheduler.waiting:
            eng.step()                                         # the next prompts; the running requests decode beside them
        torch.cuda.synchronize()
        say(f"batch {B}: prompts in")
        seqs = list(eng.scheduler.running)
        assert len(seqs) == B and all(1 <= s.num_output_tokens <= admit_steps for s in seqs)
        for _ in range(warmup):
            runner.decode(seqs)
        torch.cuda.synchronize()
        say(f"batch {B}: warm")
        clocks = ClockSampler() if sample_clocks else None
        if clocks:
            clocks.start()
            time.sleep(0.3)
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
        n0 = seqs[0].num_output_tokens
        for a, b in ev:
            a.record()
            runner.decode(seqs)                                # what LLMEngine.step calls for a decode-only step
            b.record()
        torch.cuda.synchronize()
        ck = clocks.stop() if clocks else None
        assert seqs[0].num_output_tokens == n0 + steps
        ms = statistics.median(a.elapsed_time(b) for a, b in ev)
        for _ in range(warmup):
            eng.step()
        torch.cuda.synchronize()
        t2 = time.perf_counter()
        toks = 0
        for _ in range(steps):
            toks += len(eng.step())                            # one delta per request that produced a token
        torch.cuda.synchronize()
        e2e_s = time.perf_counter() - t2
        assert toks == steps * B and seqs[0].num_output_tokens == n0 + steps + warmup + steps
        say(f"batch {B}: {ms:.3f} ms per decode step, {toks / e2e_s:.0f} tokens/s through its engine")
        del runner, eng
        torch.cuda.empty_cache()
        return ms, toks / e2e_s, prefill_s, ck

    graph = not args.no_graphs
    note = ""
    try:
        try:
            ms, e2e_v, _, clocks = decode_run(args.batch, args.steps, args.warmup, graph, sample_clocks=True)
        except Exception as e:
            if not graph:
                raise
            note = f"its CUDA-graph decode failed ({type(e).__name__}: {str(e)[:120]}); eager decode timed"
            graph = False
            torch.cuda.synchronize()
            ms, e2e_v, _, clocks = decode_run(args.batch, args.steps, args.warmup, graph, sample_clocks=True)
        points = {}
        if not args.no_points:
            for B in (1, 64):
                pms, _, _, _ = decode_run(B, max(8, args.steps // 2), max(3, args.warmup // 2), graph)
                points[f"decode_b{B}"] = round(B / (pms / 1e3), 1)
        # prefill: one 2,048-token prompt through its engine (admission + packed prefill + first token)
        pre = []
        for _ in range(4):
            _, _, ps, _ = decode_run(1, 1, 0, False)
            pre.append(ps * 1e3)
        pre_ms = statistics.median(pre[1:])
    except Exception as e:
        return unavailable(f"running the reference failed: {type(e).__name__}: {e}")

    nums = model_numbers(cfg, FULL_LAYERS)
    ctx_mid = CONTEXT + 1 + args.warmup + args.steps / 2
    step_bytes = nums["weight_bytes"] + args.batch * ctx_mid * nums["kv_per_token"]
    achieved = step_bytes / (ms / 1e3) / 1e9
    pflops = prefill_flops(cfg, FULL_LAYERS, CONTEXT)
    line = {
        "impl": "reference",
        "metric": "decode tokens/s (Qwen2-VL-2B text decoder, batch %d, 2048-token contexts)" % args.batch,
        "value": round(args.batch / (ms / 1e3), 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "fp16",
        "data": "synthetic: uniform random token ids, random weights (seed 2)",
        "config": {"model": "Qwen2-VL-2B text decoder (random weights), omniserve Qwen2LLM", "layers": FULL_LAYERS,
                   "layers_of_model": FULL_LAYERS, "hidden_size": 1536, "heads": 12, "kv_heads": 2, "head_dim": 128,
                   "intermediate_size": 8960, "vocab_size": 151936, "tied_head": True, "global_batch": args.batch,
                   "seq_len": CONTEXT, "new_tokens": NEW_TOKENS, "page_size": "one slot of max_len per request",
                   "parallelism": "single GPU", "decode": "cuda graph" if graph else "eager",
                   "l2": "inputs (3 GB of weights) larger than L2, no flush"},
        "clocks": clocks,
        "e2e": {"value": round(e2e_v, 1), "unit": "tokens/s", "h2d_bytes_per_step": 8 * args.batch * 2,
                "d2h_bytes_per_step": 8 * args.batch, "steps": args.steps, "tokens": args.steps * args.batch},
        "gpu_launches": 0,
        "prefill": {"value": round(CONTEXT / (pre_ms / 1e3), 1), "tokens": CONTEXT, "ms": round(pre_ms, 3),
                    "frac": round(pflops / (pre_ms / 1e3) / (tf_peak * 1e12), 4), "of": peak_src},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": hbm_peak, "unit": "GB/s",
                     "frac": round(achieved / hbm_peak, 4), "of": peak_src},
        "points": points, "build_s": round(build_s, 1),
    }
    if note:
        line["note"] = note
    print(json.dumps(line))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--model", default="2b", choices=["2b", "7b", "72b"], help="layer sizes of the Qwen2-VL text decoder")
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the model has (named in config)")
    ap.add_argument("--trials", type=int, default=3, help="timed runs of --steps decode steps; the median is reported")
    ap.add_argument("--workload", default="decode", choices=["decode", "mixed"],
                    help="'mixed': also 64 requests, prompts of 128..4096 tokens, 256 new tokens, portions of 2,048")
    ap.add_argument("--profile", action="store_true", help="per-kernel-class times inside real steps (no graphs)")
    ap.add_argument("--no-other-sizes", action="store_true", help="skip the 7B and 72B points of the default run")
    ap.add_argument("--page-size", type=int, default=PAGE_SIZE, help="tokens per cache page")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 and 64 points")
    ap.add_argument("--no-graphs", action="store_true", help="launch every kernel of a decode step from the host")
    ap.add_argument("--only", default="all", choices=["all", "decode"],
                    help="'decode': skip the prefill repeats, the points and the end-to-end run (for profiling)")
    args = ap.parse_args()
    globals()["PAGE_SIZE"] = args.page_size
    if args.impl == "reference":
        if args.layers is None:
            args.layers = FULL_LAYERS
        return run_reference(args)
    if args.gpus != 1:
        print("bench.py: this engine runs on one GPU; --gpus %d is not supported" % args.gpus)
        return 2
    if args.warmup < 3:
        args.warmup = 3
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
