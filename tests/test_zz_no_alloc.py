"""The decode-attention entry point that allocates nothing, called through its exported C symbol.

Some users of the kernel library cannot call cudaMalloc where they call it: a runtime that hands
out all device memory at start-up, a plug-in inside another process's allocator, a loop in which an
allocator call is not allowed. ``osb_attn_decode_noalloc`` keeps the scratch memory of the split-key
decode kernel in a fixed array inside the library instead of taking it from the caller. This test
calls it twice in a row (the array keeps the first call's contents) and checks both results against
the regular entry point, which gets its scratch from the caller, and against the plain fp32 attention
of tests/plain/kernels.py, which shares nothing with either. It runs last so that a failure here
leaves every other test already run; it passes alone in a fresh process as well.
"""

import ctypes

import pytest
import torch

from plain.kernels import PlainKernels

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _case(kv_lens, nh, nkv, hd, ps, seed):
    g = torch.Generator().manual_seed(seed)
    S = len(kv_lens)
    n_pages = sum(-(-kv // ps) for kv in kv_lens) + 2
    perm = torch.randperm(n_pages, generator=g).tolist()
    width = max(-(-kv // ps) for kv in kv_lens)
    bt = torch.full((S, width), -1, dtype=torch.int32)
    for s, kv in enumerate(kv_lens):
        for i in range(-(-kv // ps)):
            bt[s, i] = perm.pop()
    kc = torch.randn(n_pages, nkv, ps, hd, generator=g).to(torch.bfloat16)
    vc = torch.randn(n_pages, nkv, ps, hd, generator=g).to(torch.bfloat16)
    qkv = torch.randn(S, (nh + 2 * nkv) * hd, generator=g).to(torch.bfloat16)
    cu_q = torch.arange(S + 1, dtype=torch.int32)
    seq_lens = torch.tensor(kv_lens, dtype=torch.int32)
    tok_seq = torch.arange(S, dtype=torch.int32)
    didx = torch.arange(S, dtype=torch.int32)
    return [t.to(DEV) for t in (qkv, kc, vc, bt, cu_q, seq_lens, tok_seq, didx)]


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


@pytest.mark.parametrize("nh,nkv,hd,ps,window", [(12, 2, 128, 16, None), (6, 3, 48, 8, 200)])
def test_no_alloc_entry_point_matches_the_regular_one_twice(nh, nkv, hd, ps, window):
    from omniserver_b200 import ops
    K = ops.kernels()
    lib = K.lib
    lib.osb_attn_decode_noalloc_capacity.restype = ctypes.c_longlong
    capacity = lib.osb_attn_decode_noalloc_capacity()
    assert capacity == 1 << 20
    scale = hd ** -0.5
    for trial, kv_lens in enumerate([[2048, 1, 777, 64, 65, 1500, 128, 129], [900, 901, 3, 1100]]):
        qkv, kc, vc, bt, cu_q, seq_lens, tok_seq, didx = _case(kv_lens, nh, nkv, hd, ps, seed=trial)
        S, max_kv = len(kv_lens), max(kv_lens)
        want = K.paged_attention(qkv, kc, vc, bt, cu_q, seq_lens, tok_seq, nh, nkv, hd, scale, window, 1, max_kv,
                                 torch.bfloat16, decode_index=didx, n_decode=S, n_multi=0)
        chunk, nsplits = K.decode_splits(S, nkv, nh // nkv, max_kv)
        assert nsplits > 1, "the case must use the scratch"
        assert S * nh * nsplits * (hd + 2) < capacity
        out = torch.full_like(want, float("nan"))
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        rc = lib.osb_attn_decode_noalloc(_ptr(out), _ptr(qkv), qkv.shape[1], _ptr(kc), _ptr(vc), _ptr(bt), bt.shape[1],
                                         _ptr(cu_q), _ptr(seq_lens), _ptr(didx), S, nh, nkv, hd, ps, kc.shape[0],
                                         ctypes.c_float(scale), int(window or 0), S, chunk, nsplits, stream)
        assert rc == 0
        torch.cuda.synchronize()
        # same kernels, same split boundaries, same merge order: within the tolerance of the bf16 kernel tests
        assert torch.allclose(out.float(), want.float(), rtol=1.6e-2, atol=2e-3), f"call {trial}"
        assert torch.isfinite(out.float()).all()
        # and the plain attention in fp32 on the CPU: a fault of the kernel itself would show here
        cpu = [t.cpu() for t in (qkv, kc, vc, bt, cu_q, seq_lens, tok_seq)]
        plain = PlainKernels().paged_attention(cpu[0].float(), cpu[1].float(), cpu[2].float(), cpu[3], cpu[4], cpu[5],
                                               cpu[6], nh, nkv, hd, scale, window, 1, max_kv, torch.float32)
        assert torch.allclose(out.float().cpu(), plain, rtol=1.6e-2, atol=4e-3), f"call {trial} against plain"


def test_no_alloc_entry_point_with_one_split_uses_no_scratch():
    """Short contexts: one split, nothing is merged, the array is not touched."""
    from omniserver_b200 import ops
    lib = ops.kernels().lib
    nh, nkv, hd, ps = 8, 2, 64, 16
    kv_lens = [5, 64, 33, 1]
    qkv, kc, vc, bt, cu_q, seq_lens, tok_seq, didx = _case(kv_lens, nh, nkv, hd, ps, seed=4)
    S = len(kv_lens)
    out = torch.full((S, nh * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = lib.osb_attn_decode_noalloc(_ptr(out), _ptr(qkv), qkv.shape[1], _ptr(kc), _ptr(vc), _ptr(bt), bt.shape[1],
                                     _ptr(cu_q), _ptr(seq_lens), _ptr(didx), S, nh, nkv, hd, ps, kc.shape[0],
                                     ctypes.c_float(hd ** -0.5), 0, S, 64, 1, stream)
    assert rc == 0
    torch.cuda.synchronize()
    cpu = [t.cpu() for t in (qkv, kc, vc, bt, cu_q, seq_lens, tok_seq)]
    plain = PlainKernels().paged_attention(cpu[0].float(), cpu[1].float(), cpu[2].float(), cpu[3], cpu[4], cpu[5], cpu[6],
                                           nh, nkv, hd, hd ** -0.5, None, 1, max(kv_lens), torch.float32)
    assert torch.allclose(out.float().cpu(), plain, rtol=1.6e-2, atol=4e-3)


def test_no_alloc_entry_point_refuses_bad_shapes():
    """A chunk that is no multiple of 64, more splits than the kernel merges, a head size it has no form for:
    a status, nothing launched, the output untouched."""
    from omniserver_b200 import ops
    lib = ops.kernels().lib
    nh, nkv, hd, ps = 8, 2, 64, 16
    qkv, kc, vc, bt, cu_q, seq_lens, tok_seq, didx = _case([300, 200], nh, nkv, hd, ps, seed=5)
    out = torch.zeros(2, nh * hd, dtype=torch.bfloat16, device=DEV)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    def call(hd_, chunk, nsplits):
        return lib.osb_attn_decode_noalloc(_ptr(out), _ptr(qkv), qkv.shape[1], _ptr(kc), _ptr(vc), _ptr(bt), bt.shape[1],
                                           _ptr(cu_q), _ptr(seq_lens), _ptr(didx), 2, nh, nkv, hd_, ps, kc.shape[0],
                                           ctypes.c_float(0.125), 0, 2, chunk, nsplits, stream)
    assert call(hd, 100, 3) == 10002          # chunk % 64 != 0
    assert call(hd, 64, 129) == 10002         # more than 128 splits
    assert call(40, 64, 5) == 10003           # a head size that is no multiple of 16
    torch.cuda.synchronize()
    assert not out.any()


def test_no_alloc_entry_point_refuses_what_does_not_fit():
    from omniserver_b200 import ops
    lib = ops.kernels().lib
    nh, nkv, hd, ps = 32, 8, 128, 16
    S = 64
    qkv, kc, vc, bt, cu_q, seq_lens, tok_seq, didx = _case([40] * S, nh, nkv, hd, ps, seed=9)
    out = torch.zeros(S, nh * hd, dtype=torch.bfloat16, device=DEV)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    # 64 requests x 32 heads x 8 splits x 130 floats is more than the array holds
    rc = lib.osb_attn_decode_noalloc(_ptr(out), _ptr(qkv), qkv.shape[1], _ptr(kc), _ptr(vc), _ptr(bt), bt.shape[1],
                                     _ptr(cu_q), _ptr(seq_lens), _ptr(didx), S, nh, nkv, hd, ps, kc.shape[0],
                                     ctypes.c_float(hd ** -0.5), 0, S, 64, 8, stream)
    assert rc == 10004
    torch.cuda.synchronize()
    assert not out.any()
