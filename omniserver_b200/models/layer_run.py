"""Runs of consecutive layers that one kernel can step at once in a decode step.

A block may describe itself (``Block.decode_descriptor``): the arrangement, and what its parts say about
themselves.  Consecutive schedule entries whose descriptions the persistent decode kernel understands
(pre-norm blocks with RMS norms, rotary grouped-query attention and a SwiGLU feed-forward; the same sizes;
each entry writing a cache of its own in one page group) form a run.  For a step of a few single-token
requests the model hands the run to ``ops.kernels().decode_layers_fused``; for every other step, and for
every other layer, it runs the blocks one by one.  Nothing here is specific to one architecture: it is a
property of the layers' parts, found by asking them.
"""

from __future__ import annotations

from typing import Any, Dict, List, Optional, Tuple

import torch

from .. import ops
from ..parts.base import Block, CacheBinding


class FusedLayerRun:
    """Schedule entries [start, end) as one kernel launch."""

    def __init__(self, start: int, descs: List[Dict[str, Any]], bindings: List[CacheBinding]):
        self.start, self.end = start, start + len(descs)
        m, f = descs[0]["mixer"], descs[0]["ffn"]
        self.nh, self.nkv, self.hd, self.scale = m["nh"], m["nkv"], m["hd"], m["scale"]
        self.position = m["position"]
        self.group = bindings[0].group
        self.I = f["intermediate_size"]
        self.H = descs[0]["norm_attn"].shape[0]
        self._layers = [dict(norm_attn=d["norm_attn"], w_qkv=d["mixer"]["w_qkv"], b_qkv=d["mixer"]["b_qkv"],
                             w_o=d["mixer"]["w_o"], norm_ffn=d["norm_ffn"], w_gate_up=d["ffn"]["w_gate_up"],
                             w_down=d["ffn"]["w_down"], k_cache=b.k_cache, v_cache=b.v_cache, eps_attn=d["eps_attn"],
                             eps_ffn=d["eps_ffn"], window=d["mixer"]["window"]) for d, b in zip(descs, bindings)]
        self._table: Optional[torch.Tensor] = None

    @staticmethod
    def key(desc: Optional[Dict[str, Any]], binding: CacheBinding) -> Optional[Tuple]:
        """Entries with equal keys can share a run; None: this entry is in no run."""
        if desc is None or desc.get("block") != "prenorm_rms" or not binding.writes or binding.k_cache is None:
            return None
        m, f = desc["mixer"], desc["ffn"]
        if m.get("kind") != "gqa_rope" or f.get("kind") != "swiglu":
            return None
        tensors = [desc["norm_attn"], desc["norm_ffn"], m["w_qkv"], m["w_o"], f["w_gate_up"], f["w_down"], binding.k_cache]
        if any(t is None or t.dtype != torch.bfloat16 for t in tensors):
            return None
        return (m["nh"], m["nkv"], m["hd"], m["scale"], id(m["position"]), m["b_qkv"] is None, f["intermediate_size"],
                desc["norm_attn"].shape[0], binding.group, tuple(binding.k_cache.shape))

    def accepts(self, ctx: Any, x: torch.Tensor) -> bool:
        if ctx.decode_index is None:
            return False
        rot = self.position.rotary(ctx.position_tables(self.position))
        return rot is not None and ops.kernels().can_decode_layers_fused(
            x, self.H, self.nh, self.nkv, self.hd, self.I, ctx.n_decode, ctx.n_multi, rot.rot_dim)

    def forward(self, ctx: Any, x: torch.Tensor, residual: Optional[torch.Tensor]) -> Tuple[torch.Tensor, torch.Tensor]:
        k = ops.kernels()
        if self._table is None:
            self._table = k.decode_layers_table(self._layers, x.device)
        rot = self.position.rotary(ctx.position_tables(self.position))
        g = self.group
        return k.decode_layers_fused(self._table, len(self._layers), x, residual, self.I, ctx.block_tables[g],
                                     ctx.slot_maps[g], ctx.cu_q, ctx.seq_lens, ctx.decode_index, self.nh, self.nkv,
                                     self.hd, self.scale, ctx.max_kv_len, rot.cos, rot.sin, rot.rot_dim,
                                     ctx.scratch)


def find_runs(blocks: List[Block], schedule: List[Any], bindings: List[CacheBinding], min_len: int = 2
              ) -> Dict[int, FusedLayerRun]:
    """Maximal runs of schedule entries that one kernel can take, by their first entry. A layer that the
    schedule names twice is in no run (its second turn would need the first one's output order kept)."""
    seen: Dict[int, int] = {}
    for e in schedule:
        seen[e.layer] = seen.get(e.layer, 0) + 1
    keys = []
    descs = []
    for e, b in zip(schedule, bindings):
        d = blocks[e.layer].decode_descriptor() if seen[e.layer] == 1 and e.cache_of is None else None
        descs.append(d)
        keys.append(FusedLayerRun.key(d, b))
    runs: Dict[int, FusedLayerRun] = {}
    i = 0
    while i < len(keys):
        j = i
        if keys[i] is not None:
            while j + 1 < len(keys) and keys[j + 1] == keys[i]:
                j += 1
            if j + 1 - i >= min_len:
                runs[i] = FusedLayerRun(i, descs[i:j + 1], bindings[i:j + 1])
        i = j + 1
    return runs
