"""Mixers. Grouped-query attention over the paged cache.

Per layer, as the reference computes it (omniserve/model/qwen2_llm.py:75-113): one fused
projection to q, k, v (all three biased), rotary encoding of q and k, the rotated keys and
the values appended to the cache, causal attention of the new queries over all cached keys
of the same request (scale head_dim^-1/2, query head h reads kv head h // (nh/nkv)), and
an output projection without bias.  A window (keys p-w+1..p) is a parameter of the part.
"""

from __future__ import annotations

from typing import Any, List, Optional

import torch

from .. import ops
from .base import CacheBinding, KVCacheNeed, Mixer, ParamSpec, PositionEncoding, register_mixer
from .linear import Linear


class GQAAttention(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, prefix: str,
                 position: Optional[PositionEncoding] = None, qkv_bias: bool = True, out_bias: bool = False,
                 window: Optional[int] = None, scale: Optional[float] = None):
        if num_heads % num_kv_heads:
            raise ValueError(f"num_heads {num_heads} is not a multiple of num_kv_heads {num_kv_heads}")
        self.hidden_size, self.nh, self.nkv, self.hd = int(hidden_size), int(num_heads), int(num_kv_heads), int(head_dim)
        self.prefix = prefix
        self.position = position
        self.window = int(window) if window else None
        self.scale = float(scale) if scale is not None else self.hd ** -0.5
        self.qkv = Linear("qkv", hidden_size, (self.nh * self.hd, self.nkv * self.hd, self.nkv * self.hd),
                          ("q_proj", "k_proj", "v_proj"), bias=qkv_bias)
        self.out = Linear("o", self.nh * self.hd, (hidden_size,), ("o_proj",), bias=out_bias)

    def param_specs(self) -> List[ParamSpec]:
        return self.qkv.param_specs() + self.out.param_specs()

    def bind(self, tensors) -> None:
        self.qkv.bind(tensors)
        self.out.bind(tensors)

    def cache_needs(self) -> List[object]:
        return [KVCacheNeed(self.nkv, self.hd, self.window)]

    def forward(self, ctx: Any, x: torch.Tensor, binding: CacheBinding) -> torch.Tensor:
        return self._attend(ctx, self.qkv(x, ctx.act_dtype), binding)

    def _rotary(self, ctx: Any):
        """(the step's tables of this mixer's encoding, the same as rotary operands or None)."""
        if self.position is None:
            return None, None
        tables = ctx.position_tables(self.position)
        return tables, self.position.rotary(tables)

    def forward_prenorm(self, ctx: Any, x: torch.Tensor, residual, norm, binding: CacheBinding):
        # a few rows (a decode step): the norm inside the kernel of the q/k/v projection, if the norm has such a kernel
        fused = norm.fused_linear(x, residual, self.qkv, ctx.act_dtype)
        if fused is None:
            return super().forward_prenorm(ctx, x, residual, norm, binding)
        qkv, residual = fused
        return self._attend(ctx, qkv, binding), residual

    def _attend(self, ctx: Any, qkv: torch.Tensor, binding: CacheBinding) -> torch.Tensor:
        k = ops.kernels()
        tables, rot = self._rotary(ctx)
        if self.position is not None and rot is None:
            # an encoding that is no rotation of element pairs changes q and k itself, before the cache write
            self.position.apply(ctx, tables, qkv, self.nh, self.nkv, self.hd)
        g = binding.group
        rot_dim = rot.rot_dim if rot is not None else 0
        # A step of single-token requests lets the decode attention kernel rotate q and k and store
        # the new key and value itself; otherwise a kernel of its own does that for all tokens first.
        fuse = (rot_dim > 0 and binding.writes and ctx.decode_index is not None
                and k.can_fuse_rope_decode(qkv, binding.k_cache, self.nh, self.nkv, self.hd, ctx.n_decode, ctx.n_multi))
        if not fuse:
            k.rope_kv_write(qkv, rot.cos if rot_dim else None, rot.sin if rot_dim else None,
                            binding.k_cache, binding.v_cache, ctx.slot_maps[g] if binding.writes else None,
                            self.nh, self.nkv, self.hd, rot_dim)
        a = k.paged_attention(qkv, binding.k_cache, binding.v_cache, ctx.block_tables[g], ctx.cu_q, ctx.seq_lens,
                              ctx.tok_seq, self.nh, self.nkv, self.hd, self.scale, self.window,
                              ctx.max_q_len, ctx.max_kv_len, ctx.act_dtype, decode_index=ctx.decode_index,
                              n_decode=ctx.n_decode, n_multi=ctx.n_multi, scratch=ctx.scratch,
                              rope=(rot.cos, rot.sin, ctx.slot_maps[g], rot_dim) if fuse else None,
                              order=ctx.attn_order, uneven=ctx.kv_uneven, units=ctx.prefill_units)
        return self.out(a, ctx.act_dtype)


register_mixer("gqa_attention", GQAAttention)
