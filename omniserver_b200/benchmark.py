"""Measurement of the engine: decode and prefill throughput, a mixed continuous-batching run, and the share of the
roofline that the steps and their kernel classes reach.  ``bench.py`` at the repository's root and
``python -m omniserver_b200.cli bench {decode,prefill,mixed}`` both call this module.

The workloads are the reference's (benchmarks/compare/run_omniserve.py:27-42: a fixed set of requests through
LLMEngine, median of trials; benchmarks/bench_chunked_prefill.py:83-96: a long prompt in chunks beside decoding
requests; benchmarks/profile_engine.py:26-54: time per phase of a step) with random weights and uniform random token
ids in place of a checkpoint and a dataset.  Sizes are those of the Qwen2-VL text decoders (2B, 7B, 72B).

Timing: CUDA events on the launching stream around whole steps (with their gaps), after warm-up, median of trials.
Bytes a decode step has to read: every weight once plus the keys and values of the live requests; flops of a prompt:
the matrix products plus causal attention.  Peaks are given by the caller (measured copy bandwidth and library GEMM
throughput); a fraction is achieved / peak.
"""

from __future__ import annotations

import gc
import json
import os
import statistics
import subprocess
import tempfile
import time
from typing import Any, Dict, List, Optional

_BASE = {
    "architectures": ["Qwen2VLForConditionalGeneration"], "model_type": "qwen2_vl", "rms_norm_eps": 1e-6,
    "rope_theta": 1000000.0, "rope_scaling": {"type": "mrope", "mrope_section": [16, 24, 24]}, "hidden_act": "silu",
    "use_sliding_window": False, "head_dim": 128,
}
#: layer sizes of the text decoders of Qwen2-VL 2B / 7B / 72B, and the seed their random weights are drawn from
MODELS: Dict[str, Dict[str, Any]] = {
    "2b": dict(_BASE, hidden_size=1536, num_hidden_layers=28, num_attention_heads=12, num_key_value_heads=2,
               intermediate_size=8960, vocab_size=151936, tie_word_embeddings=True, max_position_embeddings=4096),
    "7b": dict(_BASE, hidden_size=3584, num_hidden_layers=28, num_attention_heads=28, num_key_value_heads=4,
               intermediate_size=18944, vocab_size=152064, tie_word_embeddings=False, max_position_embeddings=8192),
    "72b": dict(_BASE, hidden_size=8192, num_hidden_layers=80, num_attention_heads=64, num_key_value_heads=8,
                intermediate_size=29568, vocab_size=152064, tie_word_embeddings=False, max_position_embeddings=8192),
}
SEEDS = {"2b": 2, "7b": 3, "72b": 4}
FALLBACK_PEAKS = (6650.0, 1590.0)      # GB/s, TFLOP/s: an earlier measurement on this kind of GPU


def read_peaks(path: Optional[str]):
    """(copy bandwidth GB/s, bf16 GEMM TFLOP/s, "measured" | "fallback") from a MEASURED_PEAKS.json, if there is one."""
    hbm, tf = FALLBACK_PEAKS
    if path and os.path.isfile(path):
        try:
            with open(path) as f:
                d = json.load(f)
            return float(d.get("hbm_gbs", hbm)), float(d.get("bf16_tflops", tf)), "measured"
        except Exception:
            pass
    return hbm, tf, "fallback"


def read_sustained_tflops(path: Optional[str]) -> Optional[float]:
    """The bf16 GEMM rate that the same file gives for a loop of seconds under the power cap, if it has one: the
    denominator for a step that itself runs long enough to be power-limited."""
    try:
        with open(path) as f:
            v = json.load(f).get("bf16_tflops_sustained")
        return float(v) if v else None
    except Exception:
        return None


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self) -> None:
        self.proc = None
        self.path = os.path.join(tempfile.gettempdir(), "osb_bench_clocks_%d.csv" % os.getpid())

    def start(self) -> None:
        try:
            self.f = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=self.f, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.f.close()
        sm, mx, reasons = [], [], set()
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
                for n, v in zip(self.NAMES, parts[2:6]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
        if sm:
            out = {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}
        return out


def model_numbers(cfg: Dict[str, Any], layers: Optional[int] = None) -> Dict[str, int]:
    """Parameters and bytes of a configuration (bf16): what a decode step reads, what a cached token holds."""
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    L = cfg["num_hidden_layers"] if layers is None else layers
    per_layer = H * (nh + 2 * nkv) * hd + (nh + 2 * nkv) * hd + nh * hd * H + 2 * I * H + I * H + 2 * H
    head = V * H                       # the head's matrix is read once per step, tied or not
    stored = L * per_layer + V * H + H + (0 if cfg.get("tie_word_embeddings") else V * H)
    return dict(per_layer=per_layer, read_params=L * per_layer + head + H, stored_params=stored,
                weight_bytes=(L * per_layer + head + H) * 2, stored_bytes=stored * 2, kv_per_token=L * 2 * nkv * hd * 2,
                layer_weight_bytes=L * per_layer * 2, head_bytes=head * 2)


def prefill_flops(cfg: Dict[str, Any], layers: int, T: int, start: int = 0, logit_rows: int = 1) -> Dict[str, int]:
    """Flops of T prompt tokens appended at position ``start``: matrix products, causal attention, head rows."""
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    gemm = 2 * T * (H * (nh + 2 * nkv) * hd + nh * hd * H + 3 * I * H)
    keys = T * start + T * (T + 1) // 2                 # (query, key) pairs under the causal mask
    attn = 2 * 2 * nh * hd * keys
    head = 2 * H * V * logit_rows
    return dict(gemm=layers * gemm, attention=layers * attn, head=head, total=layers * (gemm + attn) + head)


#: which class a kernel launch is counted under in the per-class times
KERNEL_CLASS = (
    ("attn", "attention"), ("paged_attn", "attention"), ("stream_", "gemm"), ("gemm", "gemm"), ("library_gemm", "gemm"),
    ("silu_mul", "gemm"), ("add_rmsnorm", "norm"), ("rope", "rope"), ("advance_cursor", "rope"), ("embed", "embedding"),
    ("scatter_rows", "embedding"), ("argmax", "sampling"), ("sample", "sampling"), ("plan", "host"),
)


def kernel_class(what: str) -> str:
    for prefix, cls in KERNEL_CLASS:
        if what.startswith(prefix):
            return cls
    return "other"


class Bench:
    """One model on one GPU and the measurements on it."""

    def __init__(self, model: str, layers: Optional[int], max_batch: int, context: int, new_tokens: int, page_size: int,
                 peaks, graphs: bool = True, pool_tokens: Optional[int] = None, max_requests: Optional[int] = None):
        import torch

        from . import EngineConfig, build_runner, ops
        self.torch = torch
        self.name = model
        self.cfg = dict(MODELS[model])
        self.full_layers = self.cfg["num_hidden_layers"]
        self.layers = layers or self.full_layers
        self.cfg["num_hidden_layers"] = self.layers
        self.seed = SEEDS[model]
        self.context, self.new_tokens, self.page_size = context, new_tokens, page_size
        self.hbm_peak, self.tf_peak, self.peak_src = peaks
        self.nums = model_numbers(self.cfg)
        self.gen = torch.Generator().manual_seed(self.seed)
        if pool_tokens is None:
            pool_tokens = max_batch * (-(-(context + new_tokens) // 64) * 64) + 4096
        ec = EngineConfig(dtype="bfloat16", page_size=page_size, max_cache_tokens=pool_tokens,
                          max_requests=(max_requests or max_batch) + 2, check_device_errors=False, cuda_graphs=graphs)
        t0 = time.time()
        self.runner = build_runner(config=self.cfg, seed=self.seed, engine_config=ec, random_on_device=True)
        torch.cuda.synchronize()
        self.build_s = time.time() - t0
        self.K = ops.kernels()

    def close(self) -> None:
        self.runner = None
        gc.collect()
        self.torch.cuda.empty_cache()

    def new_prompt(self, n: int) -> List[int]:
        return self.torch.randint(0, self.cfg["vocab_size"], (n,), generator=self.gen).tolist()

    # ------------------------------------------------------------------ prefill: one prompt through the step function
    def prefill(self, tokens: int = 2048, trials: int = 5, warmup: int = 3, back_to_back: int = 4) -> Dict[str, Any]:
        """One prompt of ``tokens`` tokens through the step function. ``ms`` is the time from the call to the logits,
        the device idle before it (so the host's planning of the step counts: what a first token waits for).
        ``back_to_back_ms`` is the time per step when ``back_to_back`` such steps of different requests are launched
        one behind the other, as a loaded engine runs them: the host plans a step while the one before computes."""
        from .engine.step import StepEntry
        torch, runner = self.torch, self.runner
        times, b2b = [], []
        with torch.inference_mode():
            for i in range(warmup + trials):
                toks = self.new_prompt(tokens)
                runner.start_request(f"p{i}")
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                runner.step([StepEntry(f"p{i}", toks, want=[tokens - 1])])
                e1.record()
                torch.cuda.synchronize()
                runner.end_request(f"p{i}")
                if i >= warmup:
                    times.append(e0.elapsed_time(e1))
            for i in range(trials if back_to_back > 1 else 0):
                prompts = [self.new_prompt(tokens) for _ in range(back_to_back)]
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for j, toks in enumerate(prompts):
                    runner.start_request(f"b{i}_{j}")
                    runner.step([StepEntry(f"b{i}_{j}", toks, want=[tokens - 1])])
                    runner.end_request(f"b{i}_{j}")     # its pages go to the next prompt; the stream keeps the order
                e1.record()
                torch.cuda.synchronize()
                b2b.append(e0.elapsed_time(e1) / back_to_back)
        ms = statistics.median(times)
        fl = prefill_flops(self.cfg, self.layers, tokens)
        out = {"value": round(tokens / (ms / 1e3), 1), "tokens": tokens, "ms": round(ms, 3),
               "frac": round(fl["total"] / (ms / 1e3) / (self.tf_peak * 1e12), 4),
               "tflops": round(fl["total"] / (ms / 1e3) / 1e12, 1), "peak_tflops": self.tf_peak, "of": self.peak_src,
               "trials": len(times)}
        if b2b:
            m2 = statistics.median(b2b)
            out.update({"back_to_back_ms": round(m2, 3), "back_to_back_steps": back_to_back,
                        "back_to_back_frac": round(fl["total"] / (m2 / 1e3) / (self.tf_peak * 1e12), 4)})
        return out

    # ------------------------------------------------------------------ decode through the step function
    def decode(self, B: int, steps: int, warmup: int, trials: int = 3, clocks: bool = False) -> Dict[str, Any]:
        """Decode steps the way the engine drives them: the sampled tokens stay on the device for the next step's
        embedding lookup and are read on the host one step later, so the host's planning of step t+1 overlaps the
        device's work on step t. Every step copies its metadata from pinned host memory and brings its tokens back.
        ``trials`` timed runs of ``steps`` steps each on the same requests; the median run is reported."""
        from .engine.step import StepEntry
        from .sampling import Sampler
        torch, runner, K = self.torch, self.runner, self.K
        rids = [f"d{B}_{i}" for i in range(B)]
        sampler = Sampler(self.seed)
        with torch.inference_mode():
            for r in rids:
                runner.start_request(r)
                lg = runner.step([StepEntry(r, self.new_prompt(self.context), want=[self.context - 1])], copy_logits=False)
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
                return got + len(prev.result())

            run(warmup)
            torch.cuda.synchronize()
            sampler_proc = ClockSampler() if clocks else None
            if sampler_proc:
                sampler_proc.start()
            # the prompts' prefills just before ran the tensor cores at the power limit; the decode steps are timed
            # after a short pause, at the clocks a decoding GPU has and not at those that burst left behind
            time.sleep(0.3)
            per_step, launches = [], 0
            for _ in range(max(1, trials)):
                l0 = K.launches
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                torch.cuda.synchronize()
                e0.record()
                got = run(steps)
                e1.record()
                torch.cuda.synchronize()
                assert got == steps * B
                per_step.append(e0.elapsed_time(e1) / steps)
                launches = K.launches - l0
            ck = sampler_proc.stop() if sampler_proc else None
            done = warmup + max(1, trials) * steps
            for r in rids:
                runner.end_request(r)
        ms = statistics.median(per_step)
        ctx_mid = self.context + done / 2
        step_bytes = self.nums["weight_bytes"] + B * ctx_mid * self.nums["kv_per_token"]
        achieved = step_bytes / (ms / 1e3) / 1e9
        return {"batch": B, "ms_per_step": ms, "tokens_per_s": B / (ms / 1e3), "trials_ms": [round(t, 4) for t in per_step],
                "launches": launches, "clocks": ck, "bytes_per_step": int(step_bytes), "achieved_gbs": achieved,
                "frac": achieved / self.hbm_peak}

    # ------------------------------------------------------------------ per-class times inside real steps
    def profile(self, B: int, steps: int = 8, prefill_tokens: int = 2048) -> Dict[str, Any]:
        """Time, bytes or flops and fraction of the peak per class of kernels, from CUDA events recorded behind every
        launch of real steps (launched kernel by kernel: no graphs in this pass). A kernel's time is the time from
        the event behind the launch before it to the event behind its own, so gaps count for the kernel after them
        and the overlap of dependent launches is not seen."""
        from .engine.step import StepEntry
        torch, runner, K = self.torch, self.runner, self.K
        keep = runner.use_graphs
        runner.use_graphs = False
        out: Dict[str, Any] = {}
        try:
            with torch.inference_mode():
                # prefill
                for i in range(3):
                    runner.start_request("pp")
                    if i == 2:
                        K.start_profile()
                    runner.step([StepEntry("pp", self.new_prompt(prefill_tokens), want=[prefill_tokens - 1])])
                    if i == 2:
                        pre = K.stop_profile()
                    runner.end_request("pp")
                fl = prefill_flops(self.cfg, self.layers, prefill_tokens)
                cls: Dict[str, float] = {}
                for what, ms in pre:
                    cls[kernel_class(what)] = cls.get(kernel_class(what), 0.0) + ms
                pk = {}
                for c, ms in sorted(cls.items(), key=lambda kv: -kv[1]):
                    d = {"ms": round(ms, 3)}
                    if c == "gemm":
                        tf = (fl["gemm"] + fl["head"]) / (ms / 1e3) / 1e12
                        d.update(tflops=round(tf, 1), frac=round(tf / self.tf_peak, 3))
                    elif c == "attention":
                        tf = fl["attention"] / (ms / 1e3) / 1e12
                        d.update(tflops=round(tf, 1), frac=round(tf / self.tf_peak, 3))
                    pk[c] = d
                out["prefill"] = pk
                # decode
                rids = [f"q{i}" for i in range(B)]
                for r in rids:
                    runner.start_request(r)
                    runner.step([StepEntry(r, self.new_prompt(self.context), want=[])])
                toks = [1] * B
                for i in range(3 + steps):
                    if i == 3:
                        K.start_profile()
                    lg = runner.step([StepEntry(r, [toks[j]], want=[0]) for j, r in enumerate(rids)], copy_logits=False)
                    K.sample(lg, None, None)
                dec = K.stop_profile()
                for r in rids:
                    runner.end_request(r)
                cls = {}
                for what, ms in dec:
                    cls[kernel_class(what)] = cls.get(kernel_class(what), 0.0) + ms / steps
                kv_bytes = B * (self.context + 3 + steps / 2) * self.nums["kv_per_token"]
                dk = {}
                for c, ms in sorted(cls.items(), key=lambda kv: -kv[1]):
                    d = {"ms": round(ms, 4)}
                    if c == "gemm":
                        gbs = self.nums["weight_bytes"] / (ms / 1e3) / 1e9
                        d.update(gbs=round(gbs, 1), frac=round(gbs / self.hbm_peak, 3))
                    elif c == "attention":
                        gbs = kv_bytes / (ms / 1e3) / 1e9
                        d.update(gbs=round(gbs, 1), frac=round(gbs / self.hbm_peak, 3))
                    dk[c] = d
                out["decode"] = dk
                out["decode_batch"] = B
        finally:
            runner.use_graphs = keep
        return out

    # ------------------------------------------------------------------ end to end through LLMEngine
    def e2e_decode(self, B: int, steps: int, warmup: int) -> Dict[str, Any]:
        """The decode metric through the Python entry point: scheduler, host token ids in (pinned staging buffer, one
        host-to-device copy per step) and sampled ids out."""
        from . import LLMEngine, Request, SamplingParams, SchedulerConfig
        torch, runner = self.torch, self.runner
        with torch.inference_mode():
            # all prompts enter in one step, so that every request decodes in every timed step
            eng = LLMEngine(runner, SchedulerConfig(max_running=B, max_prefill_per_step=B,
                                                    max_prefill_tokens=self.context * B, max_seq_len=8192), seed=self.seed)
            n_new = warmup + steps + 1
            for _ in range(B):
                eng.add_request(Request(prompt=self.new_prompt(self.context),
                                        sampling=SamplingParams(max_new_tokens=n_new, ignore_eos=True)))
            while any(s.num_streamed < 1 + warmup for s in eng.sequences()):
                eng.step()
            torch.cuda.synchronize()
            t1 = time.perf_counter()
            n_steps = tokens = 0
            while eng.has_unfinished():
                tokens += sum(len(d.new_token_ids) for d in eng.step())     # tokens that reached the host
                n_steps += 1
            torch.cuda.synchronize()
            wall = max(time.perf_counter() - t1, 1e-9)
        return {"value": round(tokens / wall, 1), "unit": "tokens/s", "h2d_bytes_per_step": runner.last_h2d_bytes,
                "d2h_bytes_per_step": 4 * B, "steps": n_steps, "tokens": tokens}

    # ------------------------------------------------------------------ mixed continuous batching
    def mixed(self, requests: int = 64, prompt_lo: int = 128, prompt_hi: int = 4096, new_tokens: int = 256,
              chunk: int = 2048, max_running: int = 64, trials: int = 1) -> Dict[str, Any]:
        """The median by wall time of ``trials`` runs of ``mixed_once`` over the same requests (on a shared machine
        under its power cap single runs of the same work were seen to take 3.15 to 3.8 s)."""
        state = self.gen.get_state()
        runs = []
        for _ in range(max(1, trials)):
            self.gen.set_state(state)
            runs.append(self.mixed_once(requests, prompt_lo, prompt_hi, new_tokens, chunk, max_running))
        runs.sort(key=lambda r: r["wall_s"])
        out = dict(runs[len(runs) // 2])
        out["trials"] = len(runs)
        out["wall_s_all"] = [r["wall_s"] for r in runs]
        return out

    def mixed_once(self, requests: int = 64, prompt_lo: int = 128, prompt_hi: int = 4096, new_tokens: int = 256,
                   chunk: int = 2048, max_running: int = 64) -> Dict[str, Any]:
        """``requests`` requests with prompt lengths uniform in [prompt_lo, prompt_hi], ``new_tokens`` greedy tokens
        each, through LLMEngine with continuous batching and prompts cut into portions of at most ``chunk`` tokens
        beside the decoding requests. Reports output and prompt tokens per second over the whole run (wall clock,
        token ids in and out on the host) and the time-weighted fraction of the roofline: per step, the time that
        its bytes (every weight once, the keys and values its requests hold) and its flops (its prompt tokens)
        would take at the peaks, over the time it took on the device."""
        from . import LLMEngine, Request, SamplingParams, SchedulerConfig
        torch, runner = self.torch, self.runner
        lens = torch.randint(prompt_lo, prompt_hi + 1, (requests,), generator=self.gen).tolist()
        with torch.inference_mode():
            eng = LLMEngine(runner, SchedulerConfig(max_running=max_running, max_prefill_per_step=max_running,
                                                    max_prefill_tokens=chunk, max_seq_len=prompt_hi + new_tokens + 64),
                            seed=self.seed)
            for n in lens:
                eng.add_request(Request(prompt=self.new_prompt(n), sampling=SamplingParams(max_new_tokens=new_tokens, ignore_eos=True)))
            torch.cuda.synchronize()
            events = [torch.cuda.Event(enable_timing=True)]
            events[0].record()
            ideal: List[float] = []
            t0 = time.perf_counter()
            out_tokens = 0
            c0 = dict(eng.counters)
            while eng.has_unfinished():
                before = (eng.counters["prefill_tokens"], eng.counters["decode_tokens"])
                out_tokens += sum(len(d.new_token_ids) for d in eng.step())
                p = eng.counters["prefill_tokens"] - before[0]
                d = eng.counters["decode_tokens"] - before[1]
                ev = torch.cuda.Event(enable_timing=True)
                ev.record()
                events.append(ev)
                # what the step that was just launched has to read and compute
                live_kv = sum(s.num_computed for s in eng.scheduler.running)
                nbytes = self.nums["weight_bytes"] + live_kv * self.nums["kv_per_token"]
                flops = 2 * (p + d) * (self.nums["read_params"] - self.cfg["vocab_size"] * self.cfg["hidden_size"])
                ideal.append(max(nbytes / (self.hbm_peak * 1e9), flops / (self.tf_peak * 1e12)) if (p + d) else 0.0)
            torch.cuda.synchronize()
            wall = time.perf_counter() - t0
        device_ms = events[0].elapsed_time(events[-1])
        prefill_tokens = eng.counters["prefill_tokens"] - c0["prefill_tokens"]
        return {"requests": requests, "prompt_tokens": int(sum(lens)), "output_tokens": out_tokens, "chunk": chunk,
                "wall_s": round(wall, 3), "output_tokens_per_s": round(out_tokens / wall, 1),
                "prefill_tokens_per_s": round(prefill_tokens / wall, 1), "steps": len(ideal),
                "preemptions": eng.counters["preemptions"] - c0["preemptions"],
                "roofline_frac": round(sum(ideal) / (device_ms / 1e3), 4), "device_ms": round(device_ms, 1)}


def free_gpu_bytes() -> int:
    import torch
    return int(torch.cuda.mem_get_info()[0])


def config_of(b: Bench, batch: int) -> Dict[str, Any]:
    """The sizes of a run, flat (what a record of the run keeps)."""
    c = b.cfg
    return {"model": f"Qwen2-VL-{b.name.upper()} text decoder (random weights)", "layers": b.layers,
            "layers_of_model": b.full_layers, "hidden_size": c["hidden_size"], "heads": c["num_attention_heads"],
            "kv_heads": c["num_key_value_heads"], "head_dim": c["head_dim"], "intermediate_size": c["intermediate_size"],
            "vocab_size": c["vocab_size"], "tied_head": bool(c["tie_word_embeddings"]), "global_batch": batch,
            "seq_len": b.context, "new_tokens": b.new_tokens, "page_size": b.page_size, "parallelism": "single GPU",
            "l2": "inputs (GBs of weights) larger than L2, no flush"}
