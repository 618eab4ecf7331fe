"""What every module of ``ops`` shares: the error type, status and device error texts, argument checks."""

from __future__ import annotations

import ctypes
from typing import Optional

import torch

_DT = {torch.float32: 0, torch.bfloat16: 1}


class KernelError(RuntimeError):
    pass


_STATUS = {
    10001: "unsupported dtype",
    10002: "bad shape",
    10003: "size not supported by this kernel",
    10004: "size too large for this kernel",
}

_DEVICE_ERR = {
    1: "a token id outside the vocabulary reached the embedding lookup",
    2: "an embedding-override row outside the step's tokens",
    3: "a cache slot outside the page pool in the key/value write",
    4: "a page index outside the page pool in attention",
    101: "tcgen05 GEMM: the TMA producer waited too long for a free stage",
    102: "tcgen05 GEMM: the MMA issuer waited too long for operands",
    103: "tcgen05 GEMM: the epilogue waited too long for the accumulator",
    104: "tcgen05 GEMM: the MMA issuer waited too long for a drained accumulator",
    121: "tcgen05 GEMM (CTA pairs): the TMA producer waited too long for a free stage",
    122: "tcgen05 GEMM (CTA pairs): the MMA issuer waited too long for operands",
    123: "tcgen05 GEMM (CTA pairs): the epilogue waited too long for the accumulator",
    124: "tcgen05 GEMM (CTA pairs): the MMA issuer waited too long for a drained accumulator",
    151: "tcgen05 GEMM (few rows): the TMA producer waited too long for a free stage",
    152: "tcgen05 GEMM (few rows): the MMA issuer waited too long for operands",
    153: "tcgen05 GEMM (few rows): the epilogue waited too long for the accumulator",
    111: "tcgen05 attention: the TMA producer waited too long for a free key/value stage",
    112: "tcgen05 attention: the MMA issuer waited too long for operands",
    113: "tcgen05 attention: the softmax warps waited too long for scores or the output",
    141: "decode attention: the CTA that merges a request's splits waited too long for the others",
    131: "weight-streaming decode kernel: the consumer warps waited too long for a weight tile",
    132: "weight-streaming decode kernel: the weight stream waited too long for a free tile",
    133: "weight-streaming decode kernel: a CTA waited too long for the others at the grid barrier",
    134: "weight-streaming decode kernel: copies were still in flight when the kernel gave up",
}


def _dt(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise KernelError(f"kernels take float32 or bfloat16 tensors, got {t.dtype}") from None


def _p(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _check(cond: bool, msg: str) -> None:
    if not cond:
        raise KernelError(msg)


def _cuda_contig(name: str, t: torch.Tensor, dtype: Optional[torch.dtype] = None) -> None:
    if t.is_cuda and t.is_contiguous() and (dtype is None or t.dtype == dtype):
        return
    _check(t.is_cuda, f"{name} must be a CUDA tensor (there is no CPU path)")
    _check(t.is_contiguous(), f"{name} must be contiguous")
    _check(t.dtype == dtype, f"{name} must be {dtype}, got {t.dtype}")
