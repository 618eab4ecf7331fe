"""Builds replay traces (lists of steps) for the four families the tests use, and checks logits."""

from __future__ import annotations

import random
from typing import Dict, List, Sequence, Tuple

import torch


def whole(requests: Dict[str, List[int]]) -> List[dict]:
    """Each request alone, whole prompt in one step, logits at all places."""
    steps = []
    for i, (rid, toks) in enumerate(requests.items()):
        steps.append({"step": i, "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}],
                      "end": [rid]})
    return steps


def tail_decode(requests: Dict[str, List[int]], tail: int = 32) -> List[dict]:
    """Most of each request in one step, then the last ``tail`` tokens one by one."""
    steps, n = [], 0
    for rid, toks in requests.items():
        head = max(1, len(toks) - tail)
        steps.append({"step": n, "entries": [{"id": rid, "tokens": toks[:head], "want": list(range(head))}], "end": []})
        n += 1
        for j in range(head, len(toks)):
            steps.append({"step": n, "entries": [{"id": rid, "tokens": [toks[j]], "want": [0]}],
                          "end": [rid] if j == len(toks) - 1 else []})
            n += 1
        if head == len(toks):
            steps[-1]["end"] = [rid]
    return steps


def portions(requests: Dict[str, List[int]], sizes: Sequence[int] = (7, 2, 16, 3, 2, 33, 5, 2, 64, 11)) -> List[dict]:
    """Each request alone in portions of changing size, down to two tokens."""
    steps, n = [], 0
    for rid, toks in requests.items():
        pos, k = 0, 0
        while pos < len(toks):
            m = min(sizes[k % len(sizes)], len(toks) - pos)
            k += 1
            steps.append({"step": n, "entries": [{"id": rid, "tokens": toks[pos:pos + m], "want": list(range(m))}],
                          "end": [rid] if pos + m == len(toks) else []})
            n += 1
            pos += m
    return steps


def mixed(requests: Dict[str, List[int]], seed: int = 0, max_live: int = 4) -> List[dict]:
    """Up to ``max_live`` live requests: portions of some beside single tokens of others; requests
    start as others end, so that pages are used again."""
    rng = random.Random(seed)
    pending = list(requests.items())
    live: Dict[str, Tuple[List[int], int]] = {}
    steps, n = [], 0
    while pending or live:
        while pending and len(live) < max_live:
            rid, toks = pending.pop(0)
            live[rid] = (toks, 0)
        entries, end = [], []
        for rid in list(live):
            toks, pos = live[rid]
            if len(live) > 1 and rng.random() < 0.15:
                continue  # left out of this step, goes on later
            left = len(toks) - pos
            mode = rng.random()
            if mode < 0.45:
                m = 1
            elif mode < 0.6:
                m = 2
            else:
                m = rng.choice([3, 5, 8, 13, 16, 17, 31])
            m = min(m, left)
            entries.append({"id": rid, "tokens": toks[pos:pos + m], "want": list(range(m))})
            pos += m
            live[rid] = (toks, pos)
            if pos == len(toks):
                end.append(rid)
                del live[rid]
        if not entries:
            continue
        steps.append({"step": n, "entries": entries, "end": end})
        n += 1
    return steps


def max_live_tokens(steps: List[dict], round_to: int = 64) -> int:
    """The most tokens live requests hold at any time, each rounded up to ``round_to``."""
    held: Dict[str, int] = {}
    peak = 0
    for st in steps:
        for e in st["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum(-(-v // round_to) * round_to for v in held.values()))
        for rid in st["end"]:
            held.pop(rid, None)
    return peak


def collect(steps: List[dict], outputs: Dict[int, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """Per request: logits [len, V] assembled from the steps' outputs (all places were wanted)."""
    rows: Dict[str, List[torch.Tensor]] = {}
    for st in steps:
        out = outputs.get(st["step"])
        o = 0
        for e in st["entries"]:
            k = len(e["want"])
            if k:
                rows.setdefault(e["id"], []).append(out[o:o + k])
                o += k
    return {rid: torch.cat(v, dim=0) for rid, v in rows.items()}
