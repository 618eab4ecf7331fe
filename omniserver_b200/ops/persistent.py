"""The weight-streaming decode kernels (``csrc/decode_stream.cu``): one CTA per SM, weights streamed through
shared memory, for decode steps of up to 16 rows at any layer sizes that are multiples of 128. A mixin of
``ops.CudaKernels``, which provides ``lib``, ``_stream()``, ``_ok()``, ``err_flag()`` and the switches."""

from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch

from ._common import _check, _cuda_contig, _p


class PersistentDecodeOps:
    STREAM_MAX_ROWS = 16           # the streaming kernels have forms with one and with two column tiles of 8 rows
    #: rows of W up to which a plain projection of a few rows runs in the streaming kernel; larger matrices (the
    #: head over the vocabulary) stay with the skinny GEMM, which spreads them over many short CTAs
    STREAM_LINEAR_MAX_N = 16384

    def _stream_state(self, device: torch.device, width: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """What the streaming kernels of one device share: the words of their grid barrier and an activation
        scratch of STREAM_MAX_ROWS rows. They run one after the other on one stream."""
        idx = device.index if device.index is not None else torch.cuda.current_device()
        st = self._fused.get(idx)
        if st is None or st[1].numel() < self.STREAM_MAX_ROWS * width:
            with torch.inference_mode(False):
                bar = st[0] if st is not None else torch.zeros(64, dtype=torch.int32, device=device)
                act = torch.empty(self.STREAM_MAX_ROWS * width, dtype=torch.bfloat16, device=device)
            if st is not None:
                self._retired.append(st[1])      # a captured graph may still write to it
            st = self._fused[idx] = (bar, act)
        return st

    def can_stream_linear(self, x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor],
                          norm_weight: Optional[torch.Tensor] = None) -> bool:
        """Whether ``stream_linear`` takes these operands: a few bf16 rows over a K that is a multiple of 128
        (with a norm in front: rows that fit in shared memory beside the weight tiles)."""
        return (x.dim() == 2 and 0 < x.shape[0] <= self.STREAM_MAX_ROWS and x.dtype == w.dtype == torch.bfloat16
                and (bias is None or bias.dtype == torch.bfloat16)
                and (norm_weight is None or norm_weight.dtype == torch.bfloat16)
                and bool(self.lib.osb_stream_linear_supported(x.shape[0], x.shape[1], 0 if norm_weight is None else 1)))

    def stream_linear(self, x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
                      norm: Optional[Tuple[Optional[torch.Tensor], torch.Tensor, float]] = None, gated: bool = False):
        """y = f(x) w^T (+ bias) for up to 16 bf16 rows as one kernel that streams w once. ``norm`` = (residual or
        None, norm weight, eps): f(x) = rmsnorm(residual + x) * weight, computed by the kernel while its rows of w
        are already on their way, and the result is (y, the new fp32 residual stream). ``gated``: w is [2N, K] with
        the gate rows first and y = silu(f(x) Wg^T) * (f(x) Wu^T)."""
        _cuda_contig("x", x, torch.bfloat16)
        _cuda_contig("w", w, torch.bfloat16)
        B, K = x.shape
        N = w.shape[0] // 2 if gated else w.shape[0]
        _check(w.dim() == 2 and w.shape[1] == K and (not gated or (w.shape[0] % 2 == 0 and bias is None)),
               "stream_linear: x [B,K], w [N,K] (gated: [2N,K], no bias)")
        residual = norm_weight = res_out = None
        eps = 0.0
        if norm is not None:
            residual, norm_weight, eps = norm
            _cuda_contig("norm_weight", norm_weight, torch.bfloat16)
            _check(norm_weight.shape == (K,), "stream_linear: norm weight [K]")
            if residual is not None:
                _cuda_contig("residual", residual, torch.float32)
                _check(residual.shape == x.shape, "stream_linear: residual [B,K]")
            res_out = torch.empty((B, K), dtype=torch.float32, device=x.device)
        _check(self.can_stream_linear(x, w, bias, norm_weight), "stream_linear: up to 16 bf16 rows, K a multiple of 128 "
               "(with a norm: rows that fit in shared memory)")
        if bias is not None:
            _cuda_contig("bias", bias, torch.bfloat16)
            _check(bias.shape == (N,), "stream_linear: bias [N]")
        y = torch.empty((B, N), dtype=torch.bfloat16, device=x.device)
        rc = self.lib.osb_stream_linear(_p(y), _p(res_out), _p(x), _p(residual), _p(norm_weight), ctypes.c_float(eps),
                                        _p(w), _p(bias), _p(self.err_flag(x.device)), B, N, K, 1 if gated else 0,
                                        self._stream())
        self._ok(rc, "stream_linear")
        return (y, res_out) if norm is not None else y

    #: rows up to this length are normalised inside ``stream_linear``; longer ones by the norm kernel in front of it
    STREAM_NORM_INSIDE_WIDTH = 2048

    def prefer_norm_inside(self, x: torch.Tensor) -> bool:
        """Whether add + norm are better done inside ``stream_linear`` than by the norm kernel in front of it.
        Measured on a B200 with the q/k/v projection behind the norm (us, 1 / 8 / 16 rows): width 1,536: 3.9 / 4.2 /
        6.8 inside against 5.2 / 4.6 / 7.6 apart; width 3,584: 13.6 / 15.1 / 25.1 against 12.2 / 13.2 / 15.7; width
        8,192: 46 / 49 / - against 35 / 36 / 37. Rows of up to 2,048 elements are normalised out of registers in one
        pass by every CTA; longer ones take two passes and leave less shared memory for the weight tiles."""
        return x.shape[1] <= self.STREAM_NORM_INSIDE_WIDTH

    def can_stream_ffn(self, x: torch.Tensor, norm_weight: torch.Tensor, w_gate_up: torch.Tensor,
                       w_down: torch.Tensor) -> bool:
        """Whether ``stream_ffn`` takes these operands (else: norm, ``gate_up_silu``, ``linear``)."""
        return (self.fuse_ffn_decode and x.dim() == 2 and 0 < x.shape[0] <= self.STREAM_MAX_ROWS
                and x.dtype == norm_weight.dtype == w_gate_up.dtype == w_down.dtype == torch.bfloat16
                and bool(self.lib.osb_stream_ffn_supported(x.shape[0], x.shape[1], w_down.shape[1])))

    #: ``stream_ffn`` is preferred over the separate kernels up to these sizes
    STREAM_FFN_PREFER_ROWS = 8
    STREAM_FFN_PREFER_WIDTH = 3584

    def prefer_stream_ffn(self, x: torch.Tensor, w_gate_up: Optional[torch.Tensor] = None) -> bool:
        """Whether the one-kernel feed-forward half is the faster form for these rows. Measured on a B200 against
        add + norm, gate/up with the activation, down as three streaming kernels (us, 1 / 8 / 16 rows): width 1,536:
        17.6 / 18.5 / 25.4 against 20.2 / 19.7 / 21.8; width 3,584: 70 / 73 / 94 against 78 / 78 / 82; width 4,096 (and
        14,336 between): - / 69.5 / - against - / 65.2 / -; width 8,192: 296 / 299 / - against 230 / 235 / 239. The one kernel keeps the normalised rows in shared memory beside its
        weight tiles: with 16 rows (two column tiles) or rows of 8,192 elements too little is left for the tiles.
        Where the gate/up matrix is large enough for the few-rows tcgen05 kernel (64 MB: the 7B size) the norm
        kernel and that kernel for both products are faster still: a 7B decode step of 1 / 8 requests 2.996 / 3.216
        -> 2.966 / 3.153 ms (72B, which never took the one kernel, 24.24 / 25.55 -> 24.09 / 25.36 ms)."""
        if (w_gate_up is not None and getattr(self, "fewrows_tc", False)
                and w_gate_up.numel() >= self.LARGE_MATRIX_ELEMS):
            return False
        return x.shape[0] <= self.STREAM_FFN_PREFER_ROWS and x.shape[1] <= self.STREAM_FFN_PREFER_WIDTH

    def stream_ffn(self, x: torch.Tensor, residual: Optional[torch.Tensor], norm_weight: torch.Tensor, eps: float,
                   w_gate_up: torch.Tensor, w_down: torch.Tensor, wait_limit: int = 0, bar_extra: int = 0
                   ) -> Tuple[torch.Tensor, torch.Tensor]:
        """down(silu(gate(h)) * up(h)) with h = norm(residual + x) * norm_weight, for up to 16 rows, as one kernel
        that streams both weight matrices and in which all CTAs meet once; returns (y, the new fp32 residual
        stream). ``wait_limit`` / ``bar_extra``: only for the test that makes the CTAs' wait for one another run
        out (so many polls of the counter; so many arrivals more than there are CTAs)."""
        for name, t in (("x", x), ("norm_weight", norm_weight), ("w_gate_up", w_gate_up), ("w_down", w_down)):
            _cuda_contig(name, t, torch.bfloat16)
        B, H = x.shape
        I = w_down.shape[1]
        _check(self.can_stream_ffn(x, norm_weight, w_gate_up, w_down) and w_gate_up.shape == (2 * I, H)
               and w_down.shape == (H, I) and norm_weight.shape == (H,),
               "stream_ffn: x [B<=16,H] bf16, w_gate_up [2I,H], w_down [H,I], H and I multiples of 128, rows that fit "
               "in shared memory")
        if residual is not None:
            _cuda_contig("residual", residual, torch.float32)
            _check(residual.shape == x.shape, "stream_ffn: residual [B,H]")
        bar, act = self._stream_state(x.device, I)
        res_out = torch.empty((B, H), dtype=torch.float32, device=x.device)
        y = torch.empty((B, H), dtype=torch.bfloat16, device=x.device)
        rc = self.lib.osb_stream_ffn(_p(y), _p(res_out), _p(x), _p(residual), _p(norm_weight), ctypes.c_float(eps),
                                     _p(w_gate_up), _p(w_down), _p(act), _p(bar), _p(self.err_flag(x.device)),
                                     B, H, I, int(wait_limit), int(bar_extra), self._stream())
        self._ok(rc, "stream_ffn")
        return y, res_out
