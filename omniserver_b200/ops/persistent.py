"""The persistent decode kernels (``csrc/decode_fused.cu``): one CTA per SM, weights streamed through shared
memory, for decode steps of up to ``FUSED_MAX_ROWS`` rows. A mixin of ``ops.CudaKernels``, which provides
``lib``, ``_stream()``, ``_ok()``, ``err_flag()``, ``_scratch()`` and the switches ``fuse_*``."""

from __future__ import annotations

import ctypes
import struct
from typing import Optional, Sequence, Tuple

import torch

from ._common import _check, _cuda_contig, _p


class PersistentDecodeOps:
    FUSED_MAX_ROWS = 8
    STREAM_LINEAR_MAX_ROWS = 16    # the projection kernel (with or without its norm) has a form with two column tiles
    FFN_MAX_ROWS = 16              # and so has the feed-forward half
    SCRATCH_ROWS = 16
    STREAM_LINEAR_MAX_N = 4096     # rows of W up to which the streaming projection without norm is used
    FUSED_MAX_SPLITS = 16

    def _fused_state(self, device: torch.device, width: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """What the persistent decode kernels of one device share: the words of their grid barrier and
        an activation scratch of SCRATCH_ROWS rows. They run one after the other on one stream."""
        idx = device.index if device.index is not None else torch.cuda.current_device()
        st = self._fused.get(idx)
        if st is None or st[1].numel() < self.SCRATCH_ROWS * width:
            with torch.inference_mode(False):
                bar = st[0] if st is not None else torch.zeros(64, dtype=torch.int32, device=device)
                act = torch.empty(self.SCRATCH_ROWS * width, dtype=torch.bfloat16, device=device)
            if st is not None:
                self._retired.append(st[1])      # a captured graph may still write to it
            st = self._fused[idx] = (bar, act)
        return st

    def can_norm_linear_decode(self, x: torch.Tensor, norm_weight: torch.Tensor, w: torch.Tensor,
                               bias: Optional[torch.Tensor]) -> bool:
        """Whether ``norm_linear_decode`` takes these operands."""
        return (self.fuse_norm_linear_decode and x.dim() == 2 and 0 < x.shape[0] <= self.STREAM_LINEAR_MAX_ROWS
                and x.dtype == norm_weight.dtype == w.dtype == torch.bfloat16
                and (bias is None or bias.dtype == torch.bfloat16)
                and bool(self.lib.osb_norm_linear_decode_supported(x.shape[1])))

    def norm_linear_decode(self, x: torch.Tensor, residual: Optional[torch.Tensor], norm_weight: torch.Tensor, eps: float,
                           w: torch.Tensor, bias: Optional[torch.Tensor]) -> Tuple[torch.Tensor, torch.Tensor]:
        """(norm(residual + x) * norm_weight) @ w^T (+ bias) for up to 16 rows as one kernel that has its rows of
        w on their way while it normalises; returns (y, the new fp32 residual stream, a new tensor)."""
        for name, t in (("x", x), ("norm_weight", norm_weight), ("w", w)):
            _cuda_contig(name, t, torch.bfloat16)
        B, H = x.shape
        N = w.shape[0]
        _check(self.can_norm_linear_decode(x, norm_weight, w, bias) and w.shape == (N, H) and norm_weight.shape == (H,),
               "norm_linear_decode: x [B<=16,H] bf16, w [N,H] bf16 at a width it is built for")
        if residual is not None:
            _cuda_contig("residual", residual, torch.float32)
            _check(residual.shape == x.shape, "norm_linear_decode: residual [B,H]")
        if bias is not None:
            _cuda_contig("bias", bias, torch.bfloat16)
            _check(bias.shape == (N,), "norm_linear_decode: bias [N]")
        res_out = torch.empty((B, H), dtype=torch.float32, device=x.device)
        y = torch.empty((B, N), dtype=torch.bfloat16, device=x.device)
        rc = self.lib.osb_norm_linear_decode(_p(y), _p(res_out), _p(x), _p(residual), _p(norm_weight), ctypes.c_float(eps),
                                             _p(w), _p(bias), _p(self.err_flag(x.device)), B, N, H, self._stream())
        self._ok(rc, "norm_linear_decode")
        return y, res_out

    def can_attn_decode_fused(self, x: torch.Tensor, norm_weight: torch.Tensor, w_qkv: torch.Tensor,
                              b_qkv: Optional[torch.Tensor], w_o: torch.Tensor, k_cache: torch.Tensor, nh: int, nkv: int,
                              hd: int, n_decode: int, n_multi: int, rot: int) -> bool:
        """Whether ``attn_decode_fused`` takes this step: single-token requests only, as many rows as
        requests, a rotary span, bf16, sizes it is built for."""
        return (self.fuse_attn_decode and x.dim() == 2 and 0 < x.shape[0] <= self.FUSED_MAX_ROWS
                and n_multi == 0 and n_decode == x.shape[0] and rot > 0 and rot % 2 == 0 and nh % nkv == 0
                and nh // nkv <= 8
                and x.dtype == norm_weight.dtype == w_qkv.dtype == w_o.dtype == k_cache.dtype == torch.bfloat16
                and (b_qkv is None or b_qkv.dtype == torch.bfloat16)
                and (k_cache.shape[2] & (k_cache.shape[2] - 1)) == 0
                and bool(self.lib.osb_attn_decode_fused_supported(x.shape[1], nh * hd, hd)))

    def attn_decode_fused(self, x: torch.Tensor, residual: Optional[torch.Tensor], norm_weight: torch.Tensor, eps: float,
                          w_qkv: torch.Tensor, b_qkv: Optional[torch.Tensor], w_o: torch.Tensor, k_cache: torch.Tensor,
                          v_cache: torch.Tensor, block_table: torch.Tensor, cu_q: torch.Tensor, seq_lens: torch.Tensor,
                          decode_index: torch.Tensor, nh: int, nkv: int, hd: int, scale: float, window: Optional[int],
                          max_kv_len: int, rope: Tuple[torch.Tensor, torch.Tensor, torch.Tensor, int],
                          scratch: Optional[dict] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        """The attention half of a layer for a decode step of up to 8 single-token requests as one persistent
        kernel: norm, qkv projection, rotary encoding, cache write, attention over the cache, output projection.
        Returns (y [B,H], the new fp32 residual stream)."""
        for name, t in (("x", x), ("norm_weight", norm_weight), ("w_qkv", w_qkv), ("w_o", w_o), ("k_cache", k_cache),
                        ("v_cache", v_cache)):
            _cuda_contig(name, t, torch.bfloat16)
        B, H = x.shape
        nq = (nh + 2 * nkv) * hd
        _check(w_qkv.shape == (nq, H) and w_o.shape == (H, nh * hd) and norm_weight.shape == (H,),
               "attn_decode_fused: w_qkv [(nh+2nkv)*hd, H], w_o [H, nh*hd], norm_weight [H]")
        _check(k_cache.dim() == 4 and k_cache.shape == v_cache.shape and k_cache.shape[1] == nkv and k_cache.shape[3] == hd,
               "attn_decode_fused: caches [pages, nkv, page_size, hd]")
        if residual is not None:
            _cuda_contig("residual", residual, torch.float32)
            _check(residual.shape == x.shape, "attn_decode_fused: residual [B,H]")
        if b_qkv is not None:
            _cuda_contig("b_qkv", b_qkv, torch.bfloat16)
        cos, sin, slot_map, rot = rope
        for name, t in (("block_table", block_table), ("cu_q", cu_q), ("seq_lens", seq_lens), ("decode_index", decode_index),
                        ("slot_map", slot_map)):
            _cuda_contig(name, t, torch.int32)
        _cuda_contig("cos", cos, torch.float32)
        _cuda_contig("sin", sin, torch.float32)
        # as many splits of the keys as give every SM one (request, kv head, split); a split is at least 16 keys
        n_sm = torch.cuda.get_device_properties(x.device).multi_processor_count
        nsplits = max(1, min(n_sm // (B * nkv), (max(int(max_kv_len), 1) + 15) // 16, self.FUSED_MAX_SPLITS))
        bar, act = self._fused_state(x.device, max(nq + nh * hd, 1))
        qkv, attn = act[:B * nq].view(B, nq), act[self.FUSED_MAX_ROWS * nq:self.FUSED_MAX_ROWS * nq + B * nh * hd]
        part_o = self._scratch(scratch, "attn_part_o", B * nh * nsplits * hd, x.device)
        part_ml = self._scratch(scratch, "attn_part_ml", B * nh * nsplits * 2, x.device)
        counters = self._scratch(scratch, "attn_counters", B * nkv, x.device, zero_int=True)
        res_out = torch.empty((B, H), dtype=torch.float32, device=x.device)
        y = torch.empty((B, H), dtype=torch.bfloat16, device=x.device)
        rc = self.lib.osb_attn_decode_fused(
            _p(y), _p(res_out), _p(x), _p(residual), _p(norm_weight), ctypes.c_float(eps), _p(w_qkv), _p(b_qkv), _p(w_o),
            _p(qkv), _p(attn), _p(bar), _p(self.err_flag(x.device)), B, H, _p(k_cache), _p(v_cache), _p(block_table),
            block_table.shape[1], _p(cu_q), _p(seq_lens), _p(decode_index), nh, nkv, hd, k_cache.shape[2], k_cache.shape[0],
            ctypes.c_float(scale), int(window) if window else 0, _p(part_o), _p(part_ml), _p(counters), nsplits,
            _p(cos), _p(sin), _p(slot_map), int(rot), self._stream())
        self._ok(rc, "attn_decode_fused")
        return y, res_out

    LAYER_DESC = struct.Struct("<9Q2f4i")

    def decode_layers_table(self, layers: Sequence[dict], device: torch.device) -> torch.Tensor:
        """The device table that ``decode_layers_fused`` walks: one record per layer from a dict with the tensors
        norm_attn, w_qkv, b_qkv (or None), w_o, norm_ffn, w_gate_up, w_down, k_cache, v_cache and the numbers
        eps_attn, eps_ffn, window (or None). The tensors must stay alive as long as the table is used."""
        _check(self.LAYER_DESC.size == int(self.lib.osb_decode_layer_desc_bytes()), "layer record layout differs from the library's")
        raw = bytearray()
        for d in layers:
            for name in ("norm_attn", "w_qkv", "w_o", "norm_ffn", "w_gate_up", "w_down", "k_cache", "v_cache"):
                _cuda_contig(name, d[name], torch.bfloat16)
            if d["b_qkv"] is not None:
                _cuda_contig("b_qkv", d["b_qkv"], torch.bfloat16)
            ps = d["k_cache"].shape[2]
            _check((ps & (ps - 1)) == 0, "decode_layers_table: the page size must be a power of two")
            ptr = lambda t: 0 if t is None else t.data_ptr()
            raw += self.LAYER_DESC.pack(ptr(d["norm_attn"]), ptr(d["w_qkv"]), ptr(d["b_qkv"]), ptr(d["w_o"]), ptr(d["norm_ffn"]),
                                        ptr(d["w_gate_up"]), ptr(d["w_down"]), ptr(d["k_cache"]), ptr(d["v_cache"]),
                                        float(d["eps_attn"]), float(d["eps_ffn"]), int(d["window"] or 0),
                                        d["k_cache"].shape[0], ps.bit_length() - 1, 0)
        with torch.inference_mode(False):
            return torch.frombuffer(raw, dtype=torch.uint8).clone().to(device)

    def can_decode_layers_fused(self, x: torch.Tensor, H: int, nh: int, nkv: int, hd: int, I: int, n_decode: int,
                                n_multi: int, rot: int) -> bool:
        """Whether ``decode_layers_fused`` takes this step (see ``can_attn_decode_fused``)."""
        return (self.fuse_decode_layers and x.dim() == 2 and x.dtype == torch.bfloat16 and x.shape[1] == H
                and 0 < x.shape[0] <= self.FUSED_MAX_ROWS and n_multi == 0 and n_decode == x.shape[0]
                and rot > 0 and rot % 2 == 0 and nh % nkv == 0 and nh // nkv <= 8
                and bool(self.lib.osb_decode_layers_fused_supported(H, nh * hd, I, hd)))

    def decode_layers_fused(self, table: torch.Tensor, n_layers: int, x: torch.Tensor, residual: Optional[torch.Tensor],
                            I: int, block_table: torch.Tensor, slot_map: torch.Tensor, cu_q: torch.Tensor,
                            seq_lens: torch.Tensor, decode_index: torch.Tensor, nh: int, nkv: int, hd: int, scale: float,
                            max_kv_len: int, cos: torch.Tensor, sin: torch.Tensor, rot: int,
                            scratch: Optional[dict] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        """``n_layers`` pre-norm layers (attention half, feed-forward half) of a decode step of up to 8 single-token
        requests as ONE persistent kernel. Returns (the last half's output [B,H], the fp32 residual stream)."""
        _cuda_contig("x", x, torch.bfloat16)
        B, H = x.shape
        nq = (nh + 2 * nkv) * hd
        if residual is not None:
            _cuda_contig("residual", residual, torch.float32)
            _check(residual.shape == x.shape, "decode_layers_fused: residual [B,H]")
        for name, t in (("block_table", block_table), ("cu_q", cu_q), ("seq_lens", seq_lens), ("decode_index", decode_index),
                        ("slot_map", slot_map)):
            _cuda_contig(name, t, torch.int32)
        _cuda_contig("cos", cos, torch.float32)
        _cuda_contig("sin", sin, torch.float32)
        _check(table.numel() == n_layers * self.LAYER_DESC.size, "decode_layers_fused: one record per layer")
        n_sm = torch.cuda.get_device_properties(x.device).multi_processor_count
        nsplits = max(1, min(n_sm // (B * nkv), (max(int(max_kv_len), 1) + 15) // 16, self.FUSED_MAX_SPLITS))
        bar, act = self._fused_state(x.device, nq + nh * hd + I)
        R = self.FUSED_MAX_ROWS
        qkv, attn, mid = act[:R * nq], act[R * nq:R * (nq + nh * hd)], act[R * (nq + nh * hd):]
        part_o = self._scratch(scratch, "attn_part_o", B * nh * nsplits * hd, x.device)
        part_ml = self._scratch(scratch, "attn_part_ml", B * nh * nsplits * 2, x.device)
        counters = self._scratch(scratch, "attn_counters", B * nkv, x.device, zero_int=True)
        res = torch.empty((2, B, H), dtype=torch.float32, device=x.device)
        y = torch.empty((B, H), dtype=torch.bfloat16, device=x.device)
        rc = self.lib.osb_decode_layers_fused(
            _p(table), n_layers, _p(y), _p(res[0]), _p(res[1]), _p(x), _p(residual), _p(qkv), _p(attn), _p(mid), _p(bar),
            _p(self.err_flag(x.device)), B, H, I, _p(block_table), block_table.shape[1], _p(slot_map), _p(cu_q), _p(seq_lens),
            _p(decode_index), nh, nkv, hd, ctypes.c_float(scale), _p(part_o), _p(part_ml), _p(counters), nsplits, _p(cos),
            _p(sin), int(rot), self._stream())
        self._ok(rc, "decode_layers_fused")
        return y, res[1]

    def can_ffn_decode_fused(self, x: torch.Tensor, norm_weight: torch.Tensor, w_gate_up: torch.Tensor,
                             w_down: torch.Tensor) -> bool:
        """Whether ``ffn_decode_fused`` takes these operands (else: norm, ``gate_up_silu``, ``linear``)."""
        return (self.fuse_ffn_decode and x.dim() == 2 and 0 < x.shape[0] <= self.FFN_MAX_ROWS
                and x.dtype == norm_weight.dtype == w_gate_up.dtype == w_down.dtype == torch.bfloat16
                and bool(self.lib.osb_ffn_decode_fused_supported(x.shape[1], w_down.shape[1])))

    def ffn_decode_fused(self, x: torch.Tensor, residual: Optional[torch.Tensor], norm_weight: torch.Tensor, eps: float,
                         w_gate_up: torch.Tensor, w_down: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """down(silu(gate(h)) * up(h)) with h = norm(residual + x) * norm_weight, for up to 16 rows, as one
        persistent kernel that streams both weight matrices; returns (y, the new fp32 residual stream)."""
        for name, t in (("x", x), ("norm_weight", norm_weight), ("w_gate_up", w_gate_up), ("w_down", w_down)):
            _cuda_contig(name, t, torch.bfloat16)
        B, H = x.shape
        I = w_down.shape[1]
        _check(self.can_ffn_decode_fused(x, norm_weight, w_gate_up, w_down) and w_gate_up.shape == (2 * I, H)
               and w_down.shape == (H, I) and norm_weight.shape == (H,),
               "ffn_decode_fused: x [B<=16,H] bf16, w_gate_up [2I,H], w_down [H,I] at sizes it is built for")
        if residual is not None:
            _cuda_contig("residual", residual, torch.float32)
            _check(residual.shape == x.shape, "ffn_decode_fused: residual [B,H]")
        bar, act = self._fused_state(x.device, I)
        res_out = torch.empty((B, H), dtype=torch.float32, device=x.device)
        y = torch.empty((B, H), dtype=torch.bfloat16, device=x.device)
        rc = self.lib.osb_ffn_decode_fused(_p(y), _p(res_out), _p(x), _p(residual), _p(norm_weight), ctypes.c_float(eps),
                                           _p(w_gate_up), _p(w_down), _p(act), _p(bar), _p(self.err_flag(x.device)),
                                           B, H, I, self._stream())
        self._ok(rc, "ffn_decode_fused")
        return y, res_out
