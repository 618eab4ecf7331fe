"""Python face of the CUDA kernels: argument checks, output allocation, launch.

Every function here runs a kernel of ``csrc/`` on the current CUDA stream (or,
for large bf16 matrix products, the vendor library's GEMM, which is where the
reference's engine uses a library too: nn.Linear, omniserve/model/qwen2_llm.py:82-83,120-121,167).
Tensors must live on a CUDA device; there is no CPU path.  The kernels take
float32 and bfloat16 storage in any combination the signatures below allow.

The object that does the work is ``kernels()``; model code calls it as
``ops.kernels().<op>(...)``.
"""

from __future__ import annotations

import collections
import contextlib
import ctypes
from typing import Dict, Optional, Tuple

import numpy as np
import torch

from . import library
from .library import KernelLibraryError

from ._common import _DEVICE_ERR, _STATUS, KernelError, _check, _cuda_contig, _dt, _p
from .persistent import PersistentDecodeOps


class CudaKernels(PersistentDecodeOps):
    """Launches the hand-written kernels. One instance per process."""

    #: rows up to which the bf16 weight-streaming GEMM is used instead of the tiled tensor-core GEMM
    #: (measured on B200: it wins up to 16 rows, the library GEMM from 32 rows on)
    SKINNY_MAX_ROWS = 16
    #: matrices from 64 MB on: at up to 16 rows they go to the few-rows tcgen05 kernel (the head over the vocabulary,
    #: with its fp32 logits, to the library from 9 rows) instead of the streaming and skinny kernels
    LARGE_MATRIX_ELEMS = 1 << 25
    FEWROWS_MAX_ROWS_KERNEL = 128         # what ``gemm_fewrows`` takes
    FEWROWS_GATED_MIN_ROWS = 1            # a large gate/up matrix with its activation goes there from this many rows
    #: splits of a request's keys that one thread-block cluster of the decode attention merges
    CLUSTER_MAX_SPLITS = 8

    def __init__(self) -> None:
        self.lib = library.load()
        # the library GEMM (used for medium row counts) must accumulate in fp32, also across its K splits
        torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
        self._err: Dict[int, torch.Tensor] = {}
        self._err_pending: Dict[int, collections.deque] = {}   # copies of the flags on their way to the host
        self._err_hosts: Dict[int, list] = {}                   # pinned landing places not in use
        self.launches = 0  # kernels of this library launched so far
        self.counts: collections.Counter = collections.Counter()   # ... by entry point: which path the steps took
        self.skinny_warps = 0  # 0: the skinny GEMM picks its K split from the shape
        #: bf16 products with more rows than SKINNY_MAX_ROWS: the tcgen05/TMEM/TMA kernel (True) or the
        #: vendor library's GEMM (False)
        self.use_tcgen05 = True
        self.decode_clusters = True   # decode attention: merge a request's splits inside a cluster
        self.tc_prefill = True        # prompt attention on tcgen05 where the head size allows (64, 128)
        self.stream_max_splits = 32   # of the keys of one (request, kv head); batch 1 measured 2 % faster with 32 than 16
        self.stream_max_splits_long = 64   # ... of very long requests
        self.decode_stream = True     # decode attention that streams K and V into MMA registers (head size 64, 128)
        self.stream_target_ctas = 148  # CTAs of that kernel the GPU holds at once (one per SM)
        self.stream_cluster_sizes = (2, 4)   # split counts merged inside a thread-block cluster
        # Rows from which a plain projection runs in this repository's tcgen05 kernels. Measured, the vendor
        # library is 15-40 % faster on plain products at every row count (it spreads shapes with few tiles over
        # all SMs), so they go to the library; the fused SwiGLU product, which the library cannot do in one
        # kernel, is 35-40 % faster here at many rows and still ahead of library + activation kernel at 64 rows
        # (15.6 vs 16.2 us; at 24 rows the library pair wins, 14.0 vs 19.1 us).
        self.tcgen05_min_rows = 1 << 30
        self.tcgen05_min_rows_swiglu = 64
        # from this many rows two CTAs share a 256-row tile (cta_group::2); measured cross-over with the
        # one-CTA kernel: about 2,000 rows for the fused SwiGLU form, 4,000 for the others
        self.tcgen05_pair_min_rows = 4096
        # up to this many rows: the tcgen05 kernel with W on the M side (csrc/gemm_fewrows_tc.cu) for the gate/up
        # product with its activation (from 17 rows; a large matrix from one row) and for the plain products that
        # ``prefer_gemm_fewrows`` names
        self.fewrows_tc = True
        self.fewrows_max_rows = 64
        if torch.cuda.is_available():
            self.lib.osb_gemm_fewrows_tc_prepare()   # its questions to the device, before any graph is captured
        self._pinned_stream: Optional[ctypes.c_void_p] = None
        # decode steps of up to 16 rows: the weight-streaming kernels (csrc/decode_stream.cu) for the feed-forward
        # half, for a projection with the norm in front of it, and for a plain projection
        self.fuse_ffn_decode = True
        self.fuse_norm_linear_decode = True
        self.stream_linear_decode = True
        self._fused: dict = {}
        self._retired: list = []
        self._prof: Optional[list] = None    # while profiling: (kernel name, event behind its launch)
        self.tcgen05_pair_min_rows_swiglu = 2048

    # ------------------------------------------------------------------ plumbing
    def _stream(self) -> ctypes.c_void_p:
        if self._pinned_stream is not None:
            return self._pinned_stream
        return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    @contextlib.contextmanager
    def pinned_stream(self):
        """Inside the block every launch goes to the stream that is current at its start: one lookup
        of the current stream instead of one per launch. The caller must not switch streams inside."""
        prev = self._pinned_stream
        self._pinned_stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        try:
            yield
        finally:
            self._pinned_stream = prev

    def err_flag(self, device: torch.device) -> torch.Tensor:
        idx = device.index if device.index is not None else torch.cuda.current_device()
        if idx not in self._err:
            with torch.inference_mode(False):  # a lasting tensor: must stay writable outside inference mode
                self._err[idx] = torch.zeros(1, dtype=torch.int32, device=device)
        return self._err[idx]

    def _ok(self, rc: int, what: str) -> None:
        self.launches += 1
        self.counts[what] += 1
        if rc != 0:
            why = _STATUS.get(rc, f"CUDA error {rc}")
            raise KernelError(f"{what}: {why}")
        if self._prof is not None:
            self._mark(what)

    # ------------------------------------------------------------------ per-kernel times (measurement only)
    def _mark(self, what: str) -> None:
        if self._prof is not None:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self._prof.append((what, ev))

    def start_profile(self) -> None:
        """From here on an event is recorded behind every launch (kernel by kernel, no graphs)."""
        self._prof = []
        self._mark("start")

    def stop_profile(self) -> list:
        """[(kernel name, ms since the event before it)] of the launches since ``start_profile``; waits for them."""
        prof, self._prof = self._prof or [], None
        torch.cuda.synchronize()
        return [(what, prof[i - 1][1].elapsed_time(ev)) for i, (what, ev) in enumerate(prof) if i > 0]

    def check_device_errors(self) -> None:
        """Raise if a kernel recorded a bad index since the last check (synchronises)."""
        for flag in self._err.values():
            v = int(flag.item())
            if v != 0:
                flag.zero_()
                for bar, _ in self._fused.values():
                    bar.zero_()     # a CTA that gave up at a grid barrier leaves the counter between two multiples
                raise KernelError("device-side check failed: " + _DEVICE_ERR.get(v, f"code {v}"))

    def check_device_errors_async(self) -> None:
        """The same without waiting for the device: queues a copy of the error flags behind the work launched so
        far and raises what an earlier such copy has brought back, so an error shows a step or two late."""
        for idx, flag in self._err.items():
            pending = self._err_pending.setdefault(idx, collections.deque())
            while pending and pending[0][0].query():
                _, host = pending.popleft()
                v = int(host[0])
                self._err_hosts.setdefault(idx, []).append(host)
                if v != 0:
                    flag.zero_()
                    for bar, _ in self._fused.values():
                        bar.zero_()
                    pending.clear()
                    raise KernelError("device-side check failed: " + _DEVICE_ERR.get(v, f"code {v}"))
            if len(pending) < 4:
                free = self._err_hosts.setdefault(idx, [])
                if free:
                    host = free.pop()
                else:
                    with torch.inference_mode(False):
                        host = torch.zeros(1, dtype=torch.int32, pin_memory=True)
                host.copy_(flag, non_blocking=True)
                ev = torch.cuda.Event()
                ev.record()
                pending.append((ev, host))

    # ------------------------------------------------------------------ embedding
    def embed_lookup(self, table: torch.Tensor, ids: torch.Tensor, out_dtype: torch.dtype,
                     src_slots: Optional[torch.Tensor] = None, last_token: Optional[torch.Tensor] = None
                     ) -> torch.Tensor:
        """table[ids]; where ``src_slots[t] >= 0`` the id is ``last_token[src_slots[t]]`` instead (a token
        sampled on the device that the host has not seen yet)."""
        _cuda_contig("table", table)
        _cuda_contig("ids", ids, torch.int32)
        _check(table.dim() == 2 and ids.dim() == 1, "embed_lookup: table [V,H], ids [T]")
        V, H = table.shape
        T = ids.shape[0]
        if src_slots is not None:
            _cuda_contig("src_slots", src_slots, torch.int32)
            _cuda_contig("last_token", last_token, torch.int32)
            _check(src_slots.shape == (T,), "embed_lookup: src_slots [T]")
        out = torch.empty((T, H), dtype=out_dtype, device=table.device)
        rc = self.lib.osb_embed_lookup(_p(out), _dt(out), _p(table), _dt(table), _p(ids), _p(src_slots),
                                       _p(last_token if src_slots is not None else None), T, H, V,
                                       _p(self.err_flag(table.device)), self._stream())
        self._ok(rc, "embed_lookup")
        return out

    def scatter_rows(self, x: torch.Tensor, rows: torch.Tensor, vals: torch.Tensor) -> None:
        _cuda_contig("x", x)
        _cuda_contig("rows", rows, torch.int32)
        _cuda_contig("vals", vals)
        _check(x.dim() == 2 and vals.dim() == 2 and vals.shape[1] == x.shape[1] and vals.shape[0] == rows.shape[0],
               "scatter_rows: x [T,H], rows [R], vals [R,H]")
        rc = self.lib.osb_scatter_rows(_p(x), _dt(x), _p(rows), _p(vals), _dt(vals), rows.shape[0], x.shape[1],
                                       x.shape[0], _p(self.err_flag(x.device)), self._stream())
        self._ok(rc, "scatter_rows")

    # ------------------------------------------------------------------ norm
    def add_rmsnorm(self, x: torch.Tensor, residual: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                    out_dtype: torch.dtype) -> Tuple[torch.Tensor, torch.Tensor]:
        """residual <- residual + x (or x), fp32, in place when given; returns (norm(residual)*w, residual)."""
        _cuda_contig("x", x)
        _cuda_contig("weight", weight)
        _check(x.dim() == 2 and weight.shape == (x.shape[1],), "add_rmsnorm: x [T,H], weight [H]")
        T, H = x.shape
        if residual is None:
            res_out = torch.empty((T, H), dtype=torch.float32, device=x.device)
            res_in = None
        else:
            _cuda_contig("residual", residual, torch.float32)
            _check(residual.shape == x.shape, "add_rmsnorm: residual must match x")
            res_out = res_in = residual
        y = torch.empty((T, H), dtype=out_dtype, device=x.device)
        rc = self.lib.osb_add_rmsnorm(_p(y), _dt(y), _p(res_out), _p(res_in), _p(x), _dt(x), _p(weight), _dt(weight),
                                      ctypes.c_float(eps), T, H, _p(None), self._stream())
        self._ok(rc, "add_rmsnorm")
        return y, res_out

    def add_rmsnorm_rows(self, x: torch.Tensor, residual: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                         rows: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
        """norm(residual[rows] + x[rows]) * w for the given rows; nothing is written back."""
        _cuda_contig("x", x)
        _cuda_contig("weight", weight)
        _cuda_contig("rows", rows, torch.int32)
        if residual is not None:
            _cuda_contig("residual", residual, torch.float32)
            _check(residual.shape == x.shape, "add_rmsnorm_rows: residual must match x")
        R, H = rows.shape[0], x.shape[1]
        y = torch.empty((R, H), dtype=out_dtype, device=x.device)
        rc = self.lib.osb_add_rmsnorm(_p(y), _dt(y), _p(None), _p(residual), _p(x), _dt(x), _p(weight), _dt(weight),
                                      ctypes.c_float(eps), R, H, _p(rows), self._stream())
        self._ok(rc, "add_rmsnorm_rows")
        return y

    # ------------------------------------------------------------------ matrix product
    def linear(self, x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out_dtype: torch.dtype
               ) -> torch.Tensor:
        """y[M,N] = x[M,K] @ w[N,K]^T (+ bias), fp32 accumulation."""
        _cuda_contig("x", x)
        _cuda_contig("w", w)
        _check(x.dim() == 2 and w.dim() == 2 and x.shape[1] == w.shape[1], "linear: x [M,K], w [N,K]")
        if bias is not None:
            _cuda_contig("bias", bias)
            _check(bias.shape == (w.shape[0],), "linear: bias [N]")
        M, K = x.shape
        N = w.shape[0]
        if x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16:
            if self.can_gemm_fewrows(x, w, out_dtype) and self.prefer_gemm_fewrows(M, N, K):
                return self.gemm_fewrows(x, w, bias)
            if (self.stream_linear_decode and out_dtype == torch.bfloat16 and N <= self.STREAM_LINEAR_MAX_N
                    and self.can_stream_linear(x, w, bias)):
                # a few rows: the weight-streaming kernel without a norm
                return self.stream_linear(x, w, bias)
            return self._linear_bf16(x, w, bias, out_dtype)
        y = torch.empty((M, N), dtype=out_dtype, device=x.device)
        rc = self.lib.osb_gemm_simt(_p(y), _dt(y), _p(x), _dt(x), _p(w), _dt(w), _p(bias),
                                    _dt(bias) if bias is not None else 0, M, N, K, self._stream())
        self._ok(rc, "gemm_simt")
        return y

    def gemm_simt(self, x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out_dtype: torch.dtype
                  ) -> torch.Tensor:
        """The CUDA-core product for any operand types (the 32-bit path's GEMM)."""
        M, K = x.shape
        N = w.shape[0]
        y = torch.empty((M, N), dtype=out_dtype, device=x.device)
        rc = self.lib.osb_gemm_simt(_p(y), _dt(y), _p(x), _dt(x), _p(w), _dt(w), _p(bias),
                                    _dt(bias) if bias is not None else 0, M, N, K, self._stream())
        self._ok(rc, "gemm_simt")
        return y

    def gemm_skinny(self, x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out_dtype: torch.dtype
                    ) -> torch.Tensor:
        """The weight-streaming bf16 product for up to 64 rows (K a multiple of 8)."""
        _cuda_contig("x", x, torch.bfloat16)
        _cuda_contig("w", w, torch.bfloat16)
        M, K = x.shape
        N = w.shape[0]
        _check(w.shape[1] == K and M <= 64 and K % 8 == 0, "gemm_skinny: x [M<=64, K], w [N, K], K % 8 == 0")
        y = torch.empty((M, N), dtype=out_dtype, device=x.device)
        rc = self.lib.osb_gemm_skinny_bf16(_p(y), _dt(y), _p(x), _p(w), _p(bias), _dt(bias) if bias is not None else 0,
                                           M, N, K, 0, self.skinny_warps, self._stream())
        self._ok(rc, "gemm_skinny_bf16")
        return y

    def _linear_bf16(self, x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out_dtype: torch.dtype
                     ) -> torch.Tensor:
        M, K = x.shape
        N = w.shape[0]
        if M <= self.SKINNY_MAX_ROWS and K % 8 == 0 and (M <= 8 or N * K < self.LARGE_MATRIX_ELEMS or N % 8 != 0):
            # (with 9 to 16 rows the kernel's two-column-tile form streams a large matrix, the head over the
            # vocabulary, at 0.71 to 0.74 of the copy rate where the library reaches 0.93)
            return self.gemm_skinny(x, w, bias, out_dtype)
        if (self.use_tcgen05 and M >= self.tcgen05_min_rows and K % 8 == 0 and x.data_ptr() % 16 == 0
                and w.data_ptr() % 16 == 0):
            return self.gemm_tcgen05(x, w, bias, out_dtype)
        if K % 8 == 0 and N % 8 == 0:
            # Library GEMM on the tensor cores (fp32 accumulation inside).
            if out_dtype == torch.bfloat16:
                if bias is not None and bias.dtype == torch.bfloat16:
                    y = torch.addmm(bias, x, w.t())
                else:
                    y = torch.mm(x, w.t())
                    if bias is not None:
                        y += bias.to(torch.bfloat16)
            else:
                y = torch.mm(x, w.t(), out_dtype=torch.float32)
                if bias is not None:
                    y += bias.float()
            self._mark("library_gemm")
            return y
        return self.gemm_simt(x, w, bias, out_dtype)

    def gemm_tcgen05(self, x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out_dtype: torch.dtype,
                     swiglu: bool = False, pairs: Optional[bool] = None, wait_limit: int = 0, tx_extra: int = 0
                     ) -> torch.Tensor:
        """bf16 product on tcgen05 tensor cores with TMA-fed operands and the accumulator in TMEM.
        ``swiglu``: w is [2I, K] (gate rows first) and the result is silu(x Wg^T) * (x Wu^T), [M, I].
        ``pairs``: two CTAs per 256-row tile (cta_group::2); None: from ``tcgen05_pair_min_rows``.
        ``wait_limit`` / ``tx_extra``: only for the test that makes a wait inside the one-CTA kernel run out."""
        _cuda_contig("x", x, torch.bfloat16)
        _cuda_contig("w", w, torch.bfloat16)
        M, K = x.shape
        N = w.shape[0]
        _check(w.shape[1] == K, "gemm_tcgen05: x [M,K], w [N,K]")
        y = torch.empty((M, N // 2 if swiglu else N), dtype=out_dtype, device=x.device)
        if pairs is None:
            pairs = M >= (self.tcgen05_pair_min_rows_swiglu if swiglu else self.tcgen05_pair_min_rows)
        if wait_limit or tx_extra:
            _check(not pairs, "gemm_tcgen05: the wait test runs the one-CTA kernel")
            rc = self.lib.osb_gemm_tcgen05_bf16_ex(_p(y), _dt(y), _p(x), _p(w), _p(bias), _dt(bias) if bias is not None else 0,
                                                   M, N, K, 1 if swiglu else 0, _p(self.err_flag(x.device)),
                                                   int(wait_limit), int(tx_extra), self._stream())
            self._ok(rc, "gemm_tcgen05_bf16")
            return y
        fn = self.lib.osb_gemm_tcgen05_2cta_bf16 if pairs else self.lib.osb_gemm_tcgen05_bf16
        rc = fn(_p(y), _dt(y), _p(x), _p(w), _p(bias), _dt(bias) if bias is not None else 0,
                M, N, K, 1 if swiglu else 0, _p(self.err_flag(x.device)), self._stream())
        self._ok(rc, "gemm_tcgen05_2cta_bf16" if pairs else "gemm_tcgen05_bf16")
        return y

    def gemm_fewrows(self, x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, swiglu: bool = False,
                     splits: int = 0, form: int = 0, wait_limit: int = 0, tx_extra: int = 0) -> torch.Tensor:
        """bf16 product for up to 128 rows of x on tcgen05 with W on the M side of the MMA (128 rows of W per CTA, the
        rows of x as 32, 64 or 128 accumulator columns), K cut into ``splits`` parts (1 to 8) that are the CTAs of a
        cluster (0: from the shape). ``swiglu``: w is [2I, K] (gate rows first) and the result is
        silu(x Wg^T) * (x Wu^T); ``form`` 1: a CTA has 128 gate and 128 up rows in two accumulators, 2: 64 and 64 in
        one, 0: from the shape. ``wait_limit`` / ``tx_extra``: only for the test that makes a wait inside the kernel
        run out."""
        _cuda_contig("x", x, torch.bfloat16)
        _cuda_contig("w", w, torch.bfloat16)
        M, K = x.shape
        N = w.shape[0]
        _check(w.dim() == 2 and w.shape[1] == K and 0 < M <= self.FEWROWS_MAX_ROWS_KERNEL,
               "gemm_fewrows: x [M<=128,K], w [N,K]")
        if bias is not None:
            _cuda_contig("bias", bias)
            _check(bias.shape == (N,) and not swiglu, "gemm_fewrows: bias [N], none with the activation")
        y = torch.empty((M, N // 2 if swiglu else N), dtype=torch.bfloat16, device=x.device)
        rc = self.lib.osb_gemm_fewrows_tc(_p(y), _p(x), _p(w), _p(bias), _dt(bias) if bias is not None else 0, M, N, K,
                                          1 if swiglu else 0, int(splits), int(form), _p(self.err_flag(x.device)),
                                          int(wait_limit), int(tx_extra), self._stream())
        self._ok(rc, "gemm_fewrows_tc")
        return y

    def can_gemm_fewrows(self, x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype) -> bool:
        """Whether these operands may go to ``gemm_fewrows``: bf16, few enough rows that a 128-row tile of x would
        be mostly padding, and what TMA asks of the addresses."""
        M, K = x.shape
        return (self.fewrows_tc and x.dtype == w.dtype == torch.bfloat16 and out_dtype == torch.bfloat16
                and 0 < M <= self.fewrows_max_rows and K % 8 == 0
                and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)

    def prefer_gemm_fewrows(self, M: int, N: int, K: int) -> bool:
        """Whether a plain product of these sizes is faster in ``gemm_fewrows`` than in the streaming kernels (up to
        16 rows) or the library (more). Measured on a B200, us: at 24 to 64 rows a long K over few features (the
        down projections) 11 to 12 / 27 to 28 / 76 to 79 at the three model sizes against the library's 14 / 30 to
        31 / 73 to 81, squarer matrices of a few MB 6 to 7 against 5 (the floor of a kernel that depends on the one
        in front); at 1 to 16 rows matrices from 64 MB on (7B down; 72B qkv, o, down) 26 / 29 to 31, 24 to 26, 74
        to 75 against the streaming kernel's 26 to 27 / 31 to 32, 26 to 27, 79 to 82, smaller ones (2B down) 10.8
        against 7.6."""
        if M > self.SKINNY_MAX_ROWS:
            return K >= 2 * N
        return N * K >= self.LARGE_MATRIX_ELEMS and N <= self.STREAM_LINEAR_MAX_N

    def gate_up_silu(self, x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
        """silu(x Wg^T) * (x Wu^T) for w = [Wg; Wu] of shape [2I, K]: y [M, I].

        For few bf16 rows one kernel streams W once and applies the activation in its epilogue;
        otherwise the product and the activation are two kernels.
        """
        _cuda_contig("x", x)
        _cuda_contig("w", w)
        _check(x.dim() == 2 and w.dim() == 2 and x.shape[1] == w.shape[1] and w.shape[0] % 2 == 0,
               "gate_up_silu: x [M,K], w [2I,K]")
        M, K = x.shape
        N = w.shape[0]
        if (self.can_gemm_fewrows(x, w, out_dtype) and M < self.tcgen05_min_rows_swiglu
                and (M > self.SKINNY_MAX_ROWS
                     or (M >= self.FEWROWS_GATED_MIN_ROWS and N * K >= self.LARGE_MATRIX_ELEMS))):
            # (measured, us at the three model sizes: 24 to 48 rows 12.4 to 13.7 / 46 / 153 against 14.2 to 15.1 /
            # 51 / 169 of the library and the activation kernel; from 64 rows the kernel with 128-row tiles of x is
            # as fast and then faster; up to 16 rows 12.1 / 45 / 151 against the streaming kernel's 12.2 / 50 to 53 /
            # 151 to 155, but inside a step the 2B size lost 3 % there, so only matrices from 64 MB on)
            return self.gemm_fewrows(x, w, None, swiglu=True)
        if self.stream_linear_decode and out_dtype == torch.bfloat16 and self.can_stream_linear(x, w, None):
            # a few rows: the weight-streaming kernel (as fast as the skinny one at 8 rows, ahead of it from 9)
            return self.stream_linear(x, w, None, gated=True)
        if (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and M <= self.SKINNY_MAX_ROWS and K % 8 == 0
                and out_dtype in (torch.bfloat16, torch.float32)):
            y = torch.empty((M, N // 2), dtype=out_dtype, device=x.device)
            rc = self.lib.osb_gemm_skinny_bf16(_p(y), _dt(y), _p(x), _p(w), _p(None), 0, M, N, K, 1, self.skinny_warps,
                                               self._stream())
            self._ok(rc, "gemm_skinny_bf16(swiglu)")
            return y
        if (self.use_tcgen05 and M >= self.tcgen05_min_rows_swiglu and x.dtype == torch.bfloat16
                and w.dtype == torch.bfloat16 and out_dtype == torch.bfloat16
                and K % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0):
            return self.gemm_tcgen05(x, w, None, out_dtype, swiglu=True)
        return self.silu_mul(self.linear(x, w, None, x.dtype if x.dtype == w.dtype else torch.float32), out_dtype)

    # ------------------------------------------------------------------ rotary + cache write
    def rope_tables(self, positions: torch.Tensor, pos_mode: torch.Tensor, tok_seq: torch.Tensor,
                    cu_q: torch.Tensor, state_slot: torch.Tensor, cursor: torch.Tensor, inv_freq: torch.Tensor,
                    axis_of: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        for n, t in (("positions", positions), ("pos_mode", pos_mode), ("tok_seq", tok_seq), ("cu_q", cu_q),
                     ("state_slot", state_slot), ("cursor", cursor), ("axis_of", axis_of)):
            _cuda_contig(n, t, torch.int32)
        _cuda_contig("inv_freq", inv_freq, torch.float32)
        T = tok_seq.shape[0]
        half = inv_freq.shape[0]
        _check(positions.shape == (3, T) and axis_of.shape == (half,), "rope_tables: positions [3,T], axis_of [half]")
        cos = torch.empty((T, half), dtype=torch.float32, device=tok_seq.device)
        sin = torch.empty_like(cos)
        rc = self.lib.osb_rope_tables(_p(cos), _p(sin), _p(positions), _p(pos_mode), _p(tok_seq), _p(cu_q),
                                      _p(state_slot), _p(cursor), _p(inv_freq), _p(axis_of), T, half, self._stream())
        self._ok(rc, "rope_tables")
        return cos, sin

    def advance_cursor(self, cursor: torch.Tensor, state_slot: torch.Tensor, cu_q: torch.Tensor) -> None:
        _cuda_contig("cursor", cursor, torch.int32)
        rc = self.lib.osb_advance_cursor(_p(cursor), _p(state_slot), _p(cu_q), state_slot.shape[0], self._stream())
        self._ok(rc, "advance_cursor")

    def rope_kv_write(self, qkv: torch.Tensor, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
                      k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor],
                      slot_map: Optional[torch.Tensor], nh: int, nkv: int, hd: int, rot: int) -> None:
        """Rotate q (in place in ``qkv``) and k, write k/v into their pages. slot_map None: no write."""
        _cuda_contig("qkv", qkv)
        T = qkv.shape[0]
        _check(qkv.dim() == 2 and qkv.shape[1] == (nh + 2 * nkv) * hd, "rope_kv_write: qkv [T,(nh+2nkv)*hd]")
        if rot > 0:
            _cuda_contig("cos", cos, torch.float32)
            _cuda_contig("sin", sin, torch.float32)
            _check(cos.shape == (T, rot // 2) and sin.shape == (T, rot // 2), "rope_kv_write: cos/sin [T, rot/2]")
        page_size = num_slots = 0
        cache_dt = _dt(qkv)
        if slot_map is not None:
            _cuda_contig("slot_map", slot_map, torch.int32)
            _cuda_contig("k_cache", k_cache)
            _cuda_contig("v_cache", v_cache)
            _check(k_cache.dim() == 4 and k_cache.shape[1] == nkv and k_cache.shape[3] == hd
                   and v_cache.shape == k_cache.shape and v_cache.dtype == k_cache.dtype,
                   "rope_kv_write: caches [pages, nkv, page_size, hd]")
            page_size = k_cache.shape[2]
            num_slots = k_cache.shape[0] * page_size
            cache_dt = _dt(k_cache)
        rc = self.lib.osb_rope_kv_write(_p(qkv), _dt(qkv), _p(cos), _p(sin), _p(k_cache), _p(v_cache), cache_dt,
                                        _p(slot_map), T, nh, nkv, hd, rot, page_size, num_slots,
                                        _p(self.err_flag(qkv.device)), self._stream())
        self._ok(rc, "rope_kv_write")

    # ------------------------------------------------------------------ attention
    def paged_attention(self, qkv: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                        block_table: torch.Tensor, cu_q: torch.Tensor, seq_lens: torch.Tensor, tok_seq: torch.Tensor,
                        nh: int, nkv: int, hd: int, scale: float, window: Optional[int],
                        max_q_len: int, max_kv_len: int, out_dtype: torch.dtype,
                        decode_index: Optional[torch.Tensor] = None, n_decode: int = 0, n_multi: int = 0,
                        exact: bool = False, scratch: Optional[dict] = None,
                        rope: Optional[Tuple[torch.Tensor, torch.Tensor, torch.Tensor, int]] = None,
                        order: Optional[torch.Tensor] = None, uneven: bool = False,
                        units: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Attention of the step's queries (the first nh*hd columns of ``qkv``) over the paged cache.

        bfloat16 operands run on the tensor cores (one kernel for requests bringing several tokens,
        a split-key kernel for requests bringing one: ``decode_index`` [S] numbers those, -1 for the
        others). float32 operands, ``exact=True`` and head sizes that are no multiple of 16 run
        through the kernel whose sums have a fixed order.

        ``rope`` = (cos, sin, slot_map, rot_dim): only for steps of single-token requests for which
        ``can_fuse_rope_decode`` holds; the decode kernel then rotates q and k itself and stores the new
        key and value, and the caller must not have called ``rope_kv_write``.

        ``order`` [S] int32: the requests by falling length. The decode kernel starts their CTAs in that order, so
        that with more CTAs than SMs the short ones fill the gaps at the end (64 requests of 256 to 4,352 keys on 4
        kv heads: 79 us in the order given, 53 us longest first; 47 us would be the copy rate).
        ``units`` [n, 2] int32 (``prefill_units``): the (request, 128-row tile) pairs of the requests that bring
        several tokens, most keys first; the tcgen05 kernel then works through exactly these (beside 60 decoding
        requests a 2,048-token portion otherwise cost 3.95 instead of 1.60 ms over 28 layers: every CTA looked at
        every (tile, request, head) of the batch).
        ``uneven``: the single-token requests' lengths differ much (the longest is 1.5 times the mean or more): the
        keys may then be cut into more splits than fill the SMs once (see ``decode_splits``).
        """
        _cuda_contig("qkv", qkv)
        _cuda_contig("k_cache", k_cache)
        _cuda_contig("v_cache", v_cache)
        for n, t in (("block_table", block_table), ("cu_q", cu_q), ("seq_lens", seq_lens), ("tok_seq", tok_seq)):
            _cuda_contig(n, t, torch.int32)
        T = qkv.shape[0]
        S = seq_lens.shape[0]
        if units is not None:
            _cuda_contig("units", units, torch.int32)
            _check(units.dim() == 2 and units.shape[1] == 2, "paged_attention: units [n, 2]")
        if order is not None:
            _cuda_contig("order", order, torch.int32)
            _check(order.shape == (S,), "paged_attention: order [S]")
        _check(qkv.shape[1] >= nh * hd, "paged_attention: q columns missing")
        _check(k_cache.dim() == 4 and k_cache.shape[1] == nkv and k_cache.shape[3] == hd
               and v_cache.shape == k_cache.shape, "paged_attention: caches [pages, nkv, page_size, hd]")
        _check(block_table.dim() == 2 and block_table.shape[0] == S, "paged_attention: block_table [S,*]")
        _check(nh % nkv == 0, "paged_attention: heads must be a multiple of kv heads")
        out = torch.empty((T, nh * hd), dtype=out_dtype, device=qkv.device)
        win = int(window) if window else 0
        _check(rope is None or self.can_fuse_rope_decode(qkv, k_cache, nh, nkv, hd, n_decode, n_multi, exact),
               "paged_attention: this step cannot fuse the rotary encoding into the decode kernel")
        fast = (not exact and qkv.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16
                and out_dtype == torch.bfloat16 and hd % 16 == 0 and hd <= 256 and decode_index is not None
                and k_cache.shape[2] >= 2 and (k_cache.shape[2] & (k_cache.shape[2] - 1)) == 0)
        if fast:
            _cuda_contig("decode_index", decode_index, torch.int32)
            if (self.tc_prefill and (n_multi > 0 or n_decode == 0) and hd in (64, 128) and k_cache.shape[2] >= 8
                    and qkv.shape[1] % 8 == 0 and scale > 0):
                # requests bringing several tokens: tcgen05 kernel; the others follow in the decode kernel
                rc = self.lib.osb_attn_prefill_tc(
                    _p(out), _p(qkv), qkv.shape[1], T, _p(k_cache), _p(v_cache), _p(block_table),
                    block_table.shape[1], _p(cu_q), _p(seq_lens), S, nh, nkv, hd, k_cache.shape[2],
                    k_cache.shape[0], ctypes.c_float(scale), win, max_q_len, 1 if n_decode > 0 else 0,
                    _p(units), 0 if units is None else units.shape[0], _p(self.err_flag(qkv.device)), self._stream())
                self._ok(rc, "attn_prefill_tc")
                if n_decode == 0:
                    return out
                n_multi = 0
            if (self.decode_stream and n_decode > 0 and n_multi == 0 and hd in (64, 128) and qkv.shape[1] % 8 == 0
                    and nh // nkv <= 8):
                # single-token requests, head size 64 / 128: keys and values go from the pages straight into
                # MMA registers; one CTA of eight warps per SM, so the (request, kv head) pairs get as many
                # splits (at most 8, merged inside a cluster) as fill the SMs once
                # up to stream_max_splits splits; 2 or 4 of them are merged inside a thread-block cluster, other counts through
                # scratch memory by the CTA that finishes last: a cluster of CTAs that each fill an SM has to wait
                # until that many SMs of one GPC are free at once, which for 3 or 8 cost more than it saved
                # (measured in full decode steps at batch 8 and 24)
                # (one request of 32,768 / 131,072 keys: 16.4 / 48.4 us with 32 splits, 15.1 / 32.2 us with 47 / 64;
                # of 8,192 keys: 8.4 us with 32, 9.2 with 43: a split should keep some 640 keys)
                most = max(self.stream_max_splits, min(self.stream_max_splits_long, max_kv_len // 640))
                chunk, nsplits = self.decode_splits(n_decode, nkv, nh // nkv, max_kv_len, self.stream_target_ctas,
                                                    max_splits=most, uneven=uneven)
                use_cluster = 1 if self.decode_clusters and nsplits in self.stream_cluster_sizes else 0
                if nsplits > 1 and not use_cluster and nsplits * n_decode * nkv > self.stream_target_ctas:
                    # the CTA that merges waits for the others: the grid must fit on the GPU at once
                    nsplits = max(1, self.stream_target_ctas // (n_decode * nkv))
                    chunk = -(-max(1, max_kv_len) // nsplits)
                    chunk = -(-chunk // 64) * 64
                    nsplits = -(-max_kv_len // chunk)
                    use_cluster = 1 if self.decode_clusters and nsplits in self.stream_cluster_sizes else 0
                part_o = part_ml = counters = None
                if nsplits > 1 and not use_cluster:
                    part_o = self._scratch(scratch, "attn_part_o", n_decode * nh * nsplits * hd, qkv.device)
                    part_ml = self._scratch(scratch, "attn_part_ml", n_decode * nh * nsplits * 2, qkv.device)
                    counters = self._scratch(scratch, "attn_counters", n_decode * nkv, qkv.device, zero_int=True)
                if order is not None and nsplits * n_decode * nkv * ((nh // nkv + 7) // 8) <= self.stream_target_ctas:
                    order = None      # all CTAs start at once: no order to choose (and one round trip less in the kernel)
                rc = self.lib.osb_attn_decode_stream(
                    _p(out), _p(qkv), qkv.shape[1], _p(k_cache), _p(v_cache), _p(block_table), block_table.shape[1],
                    _p(cu_q), _p(seq_lens), _p(decode_index), _p(order), S, nh, nkv, hd, k_cache.shape[2], k_cache.shape[0],
                    ctypes.c_float(scale), win, _p(part_o), _p(part_ml), _p(counters), chunk, nsplits,
                    _p(rope[0] if rope else None), _p(rope[1] if rope else None), _p(rope[2] if rope else None),
                    int(rope[3]) if rope else 0, 1 if (use_cluster and nsplits > 1) else 0, n_decode, _p(self.err_flag(qkv.device)),
                    self._stream())
                self._ok(rc, "attn_decode_stream")
                return out
            part_o = part_ml = counters = None
            chunk, nsplits = 64, 1
            use_cluster = 0
            if n_decode > 0:
                # (request, kv head) pairs to spread over the SMs. Few of them: eight splits each, merged inside
                # a thread-block cluster, one CTA per SM. More: as many splits as fill three CTAs per SM (the
                # kernel then keeps two tiles in flight instead of three), merged inside a cluster when there
                # are at most eight of them, else through scratch memory by the last CTA. Measured in full decode
                # steps at batch 8 / 16 / 32 / 64.
                units = n_decode * nkv * ((nh // nkv + 15) // 16)
                if self.decode_clusters and units * self.CLUSTER_MAX_SPLITS <= 148:
                    chunk, nsplits = self.decode_splits(n_decode, nkv, nh // nkv, max_kv_len,
                                                        max_splits=self.CLUSTER_MAX_SPLITS)
                    use_cluster = 1 if nsplits > 1 else 0
                else:
                    chunk, nsplits = self.decode_splits(n_decode, nkv, nh // nkv, max_kv_len,
                                                        444 if units >= 24 else 296)
                    use_cluster = 1 if self.decode_clusters and 1 < nsplits <= self.CLUSTER_MAX_SPLITS else 0
                if nsplits > 1 and not use_cluster:
                    n_o, n_ml = n_decode * nh * nsplits * hd, n_decode * nh * nsplits * 2
                    part_o = self._scratch(scratch, "attn_part_o", n_o, qkv.device)
                    part_ml = self._scratch(scratch, "attn_part_ml", n_ml, qkv.device)
                    counters = self._scratch(scratch, "attn_counters", n_decode * nkv * ((nh // nkv + 15) // 16),
                                             qkv.device, zero_int=True)
            rc = self.lib.osb_paged_attn_bf16(
                _p(out), _p(qkv), qkv.shape[1], _p(k_cache), _p(v_cache), _p(block_table), block_table.shape[1],
                _p(cu_q), _p(seq_lens), _p(decode_index), S, nh, nkv, hd, k_cache.shape[2], k_cache.shape[0],
                ctypes.c_float(scale), win, max_q_len, n_decode, n_multi, _p(part_o), _p(part_ml), _p(counters), chunk,
                nsplits, _p(rope[0] if rope else None), _p(rope[1] if rope else None),
                _p(rope[2] if rope else None), int(rope[3]) if rope else 0, use_cluster, self._stream())
            self._ok(rc, "paged_attn_bf16")
            self.launches += (1 if n_multi > 0 or n_decode == 0 else 0) + (1 if n_decode > 0 else 0) - 1
            return out
        rc = self.lib.osb_paged_attn_generic(
            _p(out), _dt(out), _p(qkv), _dt(qkv), qkv.shape[1], _p(k_cache), _p(v_cache), _dt(k_cache),
            _p(block_table), block_table.shape[1], _p(cu_q), _p(seq_lens), _p(tok_seq), T, nh, nkv, hd,
            k_cache.shape[2], k_cache.shape[0], ctypes.c_float(scale), win, _p(self.err_flag(qkv.device)),
            self._stream())
        self._ok(rc, "paged_attn_generic")
        return out

    @staticmethod
    def can_fuse_rope_decode(qkv: torch.Tensor, k_cache: torch.Tensor, nh: int, nkv: int, hd: int, n_decode: int,
                             n_multi: int, exact: bool = False) -> bool:
        """Whether a step's attention may take the rotary encoding and the cache write into the
        decode kernel: every request brings one token, bf16 tensor-core path, groups of at most 16 heads."""
        ps = k_cache.shape[2]
        return (not exact and n_multi == 0 and n_decode > 0 and qkv.dtype == torch.bfloat16
                and k_cache.dtype == torch.bfloat16 and hd % 16 == 0 and hd <= 256 and nh // nkv <= 16
                and ps >= 2 and (ps & (ps - 1)) == 0)

    PREFILL_ROW_TILE = 128     # query rows of one unit of work of the tcgen05 prefill attention

    @staticmethod
    def prefill_units(q_lens, kv_lens) -> np.ndarray:
        """[n, 2] int32 (request, row tile) for every 128-row tile of the requests that bring more than one token,
        ordered by the number of keys the tile's last row sees, most first (host-side plan of a step)."""
        tile = CudaKernels.PREFILL_ROW_TILE
        ql, kv = np.asarray(q_lens, dtype=np.int64), np.asarray(kv_lens, dtype=np.int64)
        req = np.nonzero(ql > 1)[0]
        if req.size == 0:
            return np.zeros((0, 2), dtype=np.int32)
        n_tiles = -(-ql[req] // tile)
        s = np.repeat(req, n_tiles)
        m = np.concatenate([np.arange(n) for n in n_tiles])
        keys = kv[s] - ql[s] + np.minimum((m + 1) * tile, ql[s])
        order = np.argsort(-keys, kind="stable")
        return np.stack([s[order], m[order]], axis=1).astype(np.int32)

    @staticmethod
    def decode_splits(n_decode: int, nkv: int, group: int, max_kv_len: int, target_ctas: int = 296,
                      max_splits: int = 128, uneven: bool = False):
        """(chunk, nsplits) of the split-key decode kernel. ``target_ctas`` is the number of CTAs the
        GPU holds at once (148 SMs x 2); the keys are cut so that the grid fills them but does not
        spill into a second wave. Splits end at multiples of ``chunk`` keys (a multiple of 64).

        ``uneven``: the requests' lengths differ much. With one CTA per (request, kv head) the longest request then
        sets the time; twice the splits are taken if this estimate says so: a CTA costs its keys plus a fixed part
        worth about 600 keys, the step takes the longer of the longest CTA and of all CTAs' costs over the SMs, the
        mean length taken as half the longest (64 requests of 256 to 4,352 keys on 2 kv heads: 48 us with one split,
        34 us with two, 50 us with four; equal lengths of 2,048: 29 us with one, 35 us with two)."""
        per_split = max(1, n_decode * nkv * ((group + 15) // 16))
        want = max(1, target_ctas // per_split)
        chunk = -(-max(1, max_kv_len) // want)
        chunk = max(128, -(-chunk // 64) * 64)
        while -(-max_kv_len // chunk) > max_splits:   # the kernel merges at most 128 splits (8 in a cluster)
            chunk += 64
        nsplits = max(1, -(-max_kv_len // chunk))
        if uneven and 2 * nsplits <= max_splits and max_kv_len >= 256 * nsplits:
            fixed, sms = 600.0, max(1, min(target_ctas, 148))

            def cost(s: int) -> float:
                return max(max_kv_len / s + fixed, per_split * s * (0.5 * max_kv_len / s + fixed) / sms)
            if cost(2 * nsplits) < 0.9 * cost(nsplits):
                chunk2 = max(128, -(-(-(-max_kv_len // (2 * nsplits))) // 64) * 64)
                return chunk2, max(1, -(-max_kv_len // chunk2))
        return chunk, nsplits

    @staticmethod
    def _scratch(pool: Optional[dict], name: str, numel: int, device, zero_int: bool = False) -> torch.Tensor:
        """A scratch buffer kept in ``pool`` across calls. ``zero_int``: int32 counters that start at
        zero (the kernels that use them leave them zero)."""
        def make(n):
            with torch.inference_mode(False):
                if zero_int:
                    return torch.zeros(n, dtype=torch.int32, device=device)
                return torch.empty(n, dtype=torch.float32, device=device)
        if pool is None:
            return make(numel)
        t = pool.get(name)
        if t is None or t.numel() < numel:
            if t is not None:
                pool.setdefault("_retired", []).append(t)   # a captured graph may still point at it
            t = make(max(numel, 2 * t.numel() if t is not None else numel))
            pool[name] = t
        return t

    # ------------------------------------------------------------------ activation
    def silu_mul(self, gu: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
        _cuda_contig("gu", gu)
        _check(gu.dim() == 2 and gu.shape[1] % 2 == 0, "silu_mul: gu [T, 2I]")
        T, I2 = gu.shape
        out = torch.empty((T, I2 // 2), dtype=out_dtype, device=gu.device)
        rc = self.lib.osb_silu_mul(_p(out), _dt(out), _p(gu), _dt(gu), T, I2 // 2, self._stream())
        self._ok(rc, "silu_mul")
        return out

    # ------------------------------------------------------------------ sampling
    def sample(self, logits: torch.Tensor, temperature: Optional[torch.Tensor], uniform: Optional[torch.Tensor],
               keep: Optional[torch.Tensor] = None, keep_at: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Token ids [R] int32: argmax where temperature <= 0, else inverse-CDF draw with the given uniforms.
        With ``keep`` (int32 [N]) and ``keep_at`` (int32 [R], values in [0, N)) row r's token is also stored
        at ``keep[keep_at[r]]``."""
        _cuda_contig("logits", logits, torch.float32)
        R, V = logits.shape
        if keep is not None:
            _cuda_contig("keep", keep, torch.int32)
            _cuda_contig("keep_at", keep_at, torch.int32)
            _check(keep_at.shape == (R,), "sample: keep_at [R]")
        else:
            keep_at = None
        if temperature is not None:
            _cuda_contig("temperature", temperature, torch.float32)
            _cuda_contig("uniform", uniform, torch.float32)
            _check(temperature.shape == (R,) and uniform.shape == (R,), "sample: temperature/uniform [R]")
        out = torch.empty((R,), dtype=torch.int32, device=logits.device)
        if temperature is None and V >= 4096:
            sv = torch.empty((R, 32), dtype=torch.float32, device=logits.device)
            si = torch.empty((R, 32), dtype=torch.int32, device=logits.device)
            rc = self.lib.osb_argmax(_p(out), _p(logits), _p(sv), _p(si), R, V, _p(keep), _p(keep_at), self._stream())
            self._ok(rc, "argmax")
            self.launches += 1
            return out
        rc = self.lib.osb_sample(_p(out), _p(logits), _p(temperature), _p(uniform), R, V, _p(keep), _p(keep_at),
                                 self._stream())
        self._ok(rc, "sample")
        return out


_KERNELS = None


def kernels():
    """The process-wide kernel object; builds and loads the CUDA library at first use."""
    global _KERNELS
    if _KERNELS is None:
        if not torch.cuda.is_available():
            raise KernelLibraryError(
                "omniserver_b200 runs on a CUDA device (sm_100a) only; no GPU is visible to this process")
        _KERNELS = CudaKernels()
    return _KERNELS


def profile_mark(what: str) -> None:
    """While a profile is being taken (``CudaKernels.start_profile``), what ran since the event before is counted
    under ``what``; otherwise nothing happens."""
    k = _KERNELS
    if k is not None and getattr(k, "_prof", None) is not None:
        k._mark(what)


__all__ = ["kernels", "CudaKernels", "KernelError", "KernelLibraryError", "library", "profile_mark"]
