"""Trace replay: feeds given token ids through the model step by step and writes logits.

It samples nothing and has no forward pass, cache or loader of its own: it drives the
framework's model, step function, cache manager and kernels, the ones generation uses.

Input, one JSON object per line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

``entries``: for each request its next tokens and the places among them whose logits are wanted.
All entries of a step run as one batch.  An entry may also carry ``positions`` ([3][n] integers;
default: the tokens continue the request as text) and ``embeds`` ({"rows": [...], "values":
[[...], ...]}: places whose embedding is given).  ``end``: requests that are finished after the
step; what they hold is given back.  For a step in which something is wanted, ``<out>/<step>.f32``
holds the logits [wanted, vocab] as little-endian float32 in the order of the entries and of
``want``.  After every step a line ``done <step>`` is printed and flushed.
"""

from __future__ import annotations

import json
import os
import sys
from typing import Dict, Iterable, Optional

import numpy as np
import torch

from . import ops
from .config import DEFAULT_PAGE_SIZE, EngineConfig
from .engine.llm_engine import build_runner
from .engine.step import ModelRunner, StepEntry


class TraceReplayer:
    def __init__(self, runner: ModelRunner):
        self.runner = runner
        self.live = set()

    def run_step(self, step: dict) -> Optional[torch.Tensor]:
        """Runs one step of the trace; returns the logits [wanted, vocab] (None if nothing is wanted)."""
        entries = []
        for e in step.get("entries", []):
            rid = str(e["id"])
            if rid not in self.live:
                self.runner.start_request(rid)
                self.live.add(rid)
            pos = np.asarray(e["positions"], dtype=np.int64) if e.get("positions") is not None else None
            rows = vals = None
            if e.get("embeds"):
                rows = list(e["embeds"]["rows"])
                vals = torch.tensor(e["embeds"]["values"], dtype=torch.float32)
            entries.append(StepEntry(rid, list(e["tokens"]), want=list(e.get("want", [])), positions=pos,
                                     embed_rows=rows, embed_values=vals))
        logits = None
        if entries:
            out = self.runner.step(entries)
            if self.runner.check_device_errors:
                ops.kernels().check_device_errors()   # a replayed step is checked before the next one (this waits)
            if out.shape[0] > 0:
                logits = out
        for rid in step.get("end", []):
            rid = str(rid)
            if rid in self.live:
                self.runner.end_request(rid)
                self.live.discard(rid)
        return logits


def replay(runner: ModelRunner, lines: Iterable[str], out_dir: str, log=None) -> int:
    os.makedirs(out_dir, exist_ok=True)
    rp = TraceReplayer(runner)
    n = 0
    for line in lines:
        line = line.strip()
        if not line:
            continue
        step = json.loads(line)
        logits = rp.run_step(step)
        if logits is not None:
            arr = logits.detach().to(torch.float32).cpu().numpy().astype("<f4", copy=False)
            tmp = os.path.join(out_dir, f".{step['step']}.f32.tmp")
            arr.tofile(tmp)
            os.replace(tmp, os.path.join(out_dir, f"{step['step']}.f32"))
        print(f"done {step['step']}", flush=True)
        n += 1
    return n


def main(argv=None) -> int:
    import argparse
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder the logits files are written to")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each request rounded up to 64)")
    ap.add_argument("--page-size", type=int, default=DEFAULT_PAGE_SIZE)
    ap.add_argument("--max-requests", type=int, default=64)
    ap.add_argument("--device", default="cuda:0")
    args = ap.parse_args(argv)
    if 64 % args.page_size != 0:
        ap.error("--page-size must divide 64")
    if not torch.cuda.is_available():
        print("trace_run: no CUDA device is visible; this engine runs on a GPU only", file=sys.stderr)
        return 1
    ec = EngineConfig(dtype=args.dtype, page_size=args.page_size, max_cache_tokens=args.max_tokens,
                      max_requests=args.max_requests, device=args.device)
    from . import ops
    ops.kernels()  # builds the kernels at the first call, with progress lines on stderr
    if args.dtype == "float32":
        torch.backends.cuda.matmul.allow_tf32 = False
        torch.backends.cudnn.allow_tf32 = False
    with torch.inference_mode():
        runner = build_runner(model_dir=args.model, engine_config=ec)
        replay(runner, sys.stdin, args.out)
    return 0


if __name__ == "__main__":
    sys.exit(main())
