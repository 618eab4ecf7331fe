"""Each CUDA kernel alone against its plain reference (tests/plain/kernels.py), at sizes other
than the engine's tiny models: widths and vocabularies that are no power of two, head sizes in
steps of 16, odd head counts and groups, in float32 and bfloat16."""

import math

import pytest
import torch

from plain.kernels import PlainKernels

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
REF = PlainKernels()
DTYPES = [torch.float32, torch.bfloat16]


def K():
    from omniserver_b200 import ops
    return ops.kernels()


def tol(dtype):
    # one rounding of the output: 2^-24 vs 2^-9 relative, plus accumulation-order noise
    return dict(rtol=2e-5, atol=2e-6) if dtype == torch.float32 else dict(rtol=1.6e-2, atol=2e-3)


def rnd(*shape, dtype=torch.float32, scale=1.0, seed=0):
    g = torch.Generator().manual_seed(seed + sum(shape))
    return (torch.randn(*shape, generator=g) * scale).to(dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("V,H,T", [(1000, 96, 7), (777, 1536, 33), (50, 20, 1)])
def test_embed_lookup_and_scatter(dtype, V, H, T):
    table = rnd(V, H, dtype=dtype)
    ids = torch.randint(0, V, (T,), dtype=torch.int32)
    got = K().embed_lookup(table.to(DEV), ids.to(DEV), dtype)
    assert torch.equal(got.cpu(), REF.embed_lookup(table, ids, dtype))
    rows = torch.tensor(sorted(set([0, T - 1, T // 2])), dtype=torch.int32)
    vals = rnd(len(rows), H, seed=5)
    K().scatter_rows(got, rows.to(DEV), vals.to(DEV))
    want = REF.embed_lookup(table, ids, dtype)
    REF.scatter_rows(want, rows, vals)
    assert torch.equal(got.cpu(), want)
    K().check_device_errors()


def test_embed_lookup_takes_ids_kept_on_the_device():
    table = rnd(50, 24)
    ids = torch.tensor([3, 7, 0, 49, 5], dtype=torch.int32)
    src = torch.tensor([-1, 2, -1, 0, 5], dtype=torch.int32)
    last = torch.tensor([11, 0, 13, 0, 0, 48], dtype=torch.int32)
    got = K().embed_lookup(table.to(DEV), ids.to(DEV), torch.float32, src.to(DEV), last.to(DEV))
    assert torch.equal(got.cpu(), table[torch.tensor([3, 13, 0, 11, 48])])
    assert torch.equal(got.cpu(), REF.embed_lookup(table, ids, torch.float32, src, last))
    K().check_device_errors()


def test_embed_lookup_reports_bad_id():
    from omniserver_b200.ops import KernelError
    table = rnd(10, 8)
    ids = torch.tensor([1, 10], dtype=torch.int32)
    K().embed_lookup(table.to(DEV), ids.to(DEV), torch.float32)
    with pytest.raises(KernelError, match="outside the vocabulary"):
        K().check_device_errors()


def test_device_errors_are_also_reported_without_waiting():
    """The check that the engine makes after every step does not wait for the device: it queues a copy of the
    flag and raises what an earlier copy has brought back."""
    from omniserver_b200.ops import KernelError
    k = K()
    k.check_device_errors()
    table = rnd(50, 32, dtype=torch.bfloat16).to(DEV)
    k.embed_lookup(table, torch.tensor([3, 50], dtype=torch.int32, device=DEV), torch.bfloat16)
    k.check_device_errors_async()          # the copy is on its way; nothing to report yet, or already there
    torch.cuda.synchronize()
    with pytest.raises(KernelError, match="outside the vocabulary"):
        k.check_device_errors_async()
    k.check_device_errors_async()          # the flag was cleared
    torch.cuda.synchronize()
    k.check_device_errors_async()
    k.check_device_errors()


@pytest.mark.parametrize("xdt", DTYPES)
@pytest.mark.parametrize("wdt", DTYPES)
@pytest.mark.parametrize("T,H,eps", [(5, 96, 1e-5), (3, 1536, 1e-6), (2, 5000, 1e-6), (1, 17, 1e-3), (300, 1536, 1e-6), (67, 2048, 1e-5),
                                     (100, 256, 1e-6), (64, 1280, 1e-6)])
def test_add_rmsnorm(xdt, wdt, T, H, eps):
    x = rnd(T, H, dtype=xdt, scale=3.0)
    res = rnd(T, H, seed=1, scale=5.0)
    w = (1 + 0.1 * rnd(H, seed=2)).to(wdt)
    for residual in (None, res):
        r_dev = residual.clone().to(DEV) if residual is not None else None
        y, r_out = K().add_rmsnorm(x.to(DEV), r_dev, w.to(DEV), eps, xdt)
        r_ref = residual.clone() if residual is not None else None
        y_ref, r_ref_out = REF.add_rmsnorm(x, r_ref, w, eps, xdt)
        assert torch.allclose(r_out.cpu(), r_ref_out, rtol=0, atol=0)
        assert torch.allclose(y.float().cpu(), y_ref.float(), **tol(xdt))
    rows = torch.tensor([T - 1, 0], dtype=torch.int32)
    y = K().add_rmsnorm_rows(x.to(DEV), res.to(DEV), w.to(DEV), eps, rows.to(DEV), xdt)
    y_ref = REF.add_rmsnorm_rows(x, res, w, eps, rows, xdt)
    assert torch.allclose(y.float().cpu(), y_ref.float(), **tol(xdt))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M,N,K_", [(1, 200, 96), (7, 1000, 96), (33, 130, 200), (70, 64, 1536), (128, 257, 77)])
def test_gemm_simt(dtype, M, N, K_):
    x, w, b = rnd(M, K_, dtype=dtype), rnd(N, K_, dtype=dtype, seed=1, scale=0.05), rnd(N, dtype=dtype, seed=2)
    for bias in (None, b):
        got = K().gemm_simt(x.to(DEV), w.to(DEV), bias.to(DEV) if bias is not None else None, torch.float32)
        want = REF.linear(x.double(), w.double(), bias.double() if bias is not None else None, torch.float64)
        assert torch.allclose(got.cpu().double(), want, rtol=1e-5, atol=1e-5)


def test_gemm_simt_rows_do_not_depend_on_the_batch():
    x, w = rnd(70, 200), rnd(130, 200, seed=1)
    whole = K().gemm_simt(x.to(DEV), w.to(DEV), None, torch.float32)
    for a, b in [(0, 1), (5, 7), (63, 70)]:
        part = K().gemm_simt(x[a:b].contiguous().to(DEV), w.to(DEV), None, torch.float32)
        assert torch.equal(part, whole[a:b])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M,N,K_", [(1, 200, 96), (8, 1536, 1536), (13, 1536, 1536), (16, 300, 256), (64, 1000, 256), (200, 264, 1536),
                                    (3, 17920, 64)])
def test_linear_bf16_and_f32(dtype, M, N, K_):
    x, w, b = rnd(M, K_, dtype=dtype), rnd(N, K_, dtype=dtype, seed=1, scale=0.05), rnd(N, dtype=dtype, seed=2)
    for bias in (None, b):
        for out_dtype in (dtype, torch.float32):
            got = K().linear(x.to(DEV), w.to(DEV), bias.to(DEV) if bias is not None else None, out_dtype)
            want = REF.linear(x.double(), w.double(), bias.double() if bias is not None else None, torch.float64)
            assert got.dtype == out_dtype
            # against a float64 reference: fp32 accumulation over K in another order, then one rounding of the output
            t = dict(rtol=1e-5, atol=1e-5) if dtype == torch.float32 else tol(dtype)
            assert torch.allclose(got.double().cpu(), want, **t)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M,I,K_", [(1, 200, 96), (8, 8960, 1536), (33, 176, 80), (64, 128, 64), (100, 200, 96)])
def test_gate_up_silu(dtype, M, I, K_):
    x, w = rnd(M, K_, dtype=dtype), rnd(2 * I, K_, dtype=dtype, seed=1, scale=0.1)
    got = K().gate_up_silu(x.to(DEV), w.to(DEV), dtype)
    assert got.shape == (M, I)
    if dtype == torch.bfloat16:   # the product is rounded to bf16 before the activation, as in the two-kernel path
        assert_swiglu_close(got, x, w, I)
        return
    want = REF.silu_mul(REF.linear(x.double(), w.double(), None, torch.float64), torch.float64)
    # a product of two sums: its absolute error is the sums' error (~1e-6 after K fp32 additions)
    # times the other factor, which reaches a few tens here
    scale = float(want.abs().max())
    t = dict(rtol=1e-5, atol=3e-6 * max(1.0, scale)) if dtype == torch.float32 else dict(rtol=2e-2, atol=4e-3)
    assert torch.allclose(got.double().cpu(), want, **t)


@pytest.mark.parametrize("M,N,K_", [(1, 1536, 1536), (8, 2048, 1536), (8, 1536, 8960), (64, 17920, 1536), (5, 151936, 1536),
                                    (17, 40, 72), (64, 1000, 200)])
def test_skinny_gemm_bf16(M, N, K_):
    """The weight-streaming product at the decode step's shapes and at ragged ones (N not a multiple
    of 16, K not a multiple of 64)."""
    x, w = rnd(M, K_, dtype=torch.bfloat16), rnd(N, K_, dtype=torch.bfloat16, seed=1, scale=0.05)
    b = rnd(N, dtype=torch.bfloat16, seed=2)
    for bias in (None, b, b.float()):
        for out_dtype in (torch.bfloat16, torch.float32):
            got = K().gemm_skinny(x.to(DEV), w.to(DEV), bias.to(DEV) if bias is not None else None, out_dtype)
            want = REF.linear(x.double(), w.double(), bias.double() if bias is not None else None, torch.float64)
            t = dict(rtol=1e-4, atol=2.5e-8 * K_ * float(want.abs().max()) + 1e-5) if out_dtype == torch.float32 \
                else tol(torch.bfloat16)
            assert torch.allclose(got.double().cpu(), want, **t)


# Layer widths of the 2B, 7B and 72B checkpoints of the architecture beside small and odd ones: the streaming
# kernels take any multiple of 128 (a norm in front: as long as the rows fit in shared memory beside the tiles).
@pytest.mark.parametrize("H,N", [(256, 100), (384, 1000), (2048, 300), (1536, 2048), (1536, 17), (3584, 4608),
                                 (8192, 1280), (2176, 333)])
@pytest.mark.parametrize("B", [1, 5, 8, 9, 13, 16])
def test_stream_linear_with_the_norm_inside(H, N, B):
    """The projection of a few rows that normalises them itself while its weights stream in. The new residual
    stream is the fp32 sum bit for bit; the product matches the norm's output (rounded to bf16 as the separate
    kernel rounds it) times W. The norm's statistics are summed in another order than in the norm kernel, so a
    value of the normalised row may fall on the other side of a bf16 rounding tie: the bound allows for one such
    step (2^-8) on every term, and for the output's own rounding to bf16."""
    x = rnd(B, H, dtype=torch.bfloat16)
    res = rnd(B, H, seed=3, scale=2.0)
    gm = (1.0 + 0.2 * rnd(H, seed=4)).to(torch.bfloat16)
    w = rnd(N, H, dtype=torch.bfloat16, seed=1, scale=H ** -0.5)
    b = rnd(N, dtype=torch.bfloat16, seed=2)
    k = K()
    if H == 8192 and B > 8:
        # sixteen rows of 8,192 elements do not fit beside the tiles: refused by rule, not computed wrongly
        assert not k.can_stream_linear(x.to(DEV), w.to(DEV), None, gm.to(DEV))
        with pytest.raises(Exception):
            k.stream_linear(x.to(DEV), w.to(DEV), None, norm=(None, gm.to(DEV), 1e-6))
        return
    for bias in (None, b):
        for with_res in (True, False):
            res_dev = res.to(DEV) if with_res else None
            bd = bias.to(DEV) if bias is not None else None
            assert k.can_stream_linear(x.to(DEV), w.to(DEV), bd, gm.to(DEV))
            y, new_res = k.stream_linear(x.to(DEV), w.to(DEV), bd, norm=(res_dev, gm.to(DEV), 1e-6))
            if with_res:
                assert torch.equal(res_dev.cpu(), res), "the old residual stream must stay as it was"
            r = x.float() + res if with_res else x.float()
            assert torch.equal(new_res.cpu(), r)
            h, _ = REF.add_rmsnorm(x, res.clone() if with_res else None, gm, 1e-6, torch.bfloat16)
            want = REF.linear(h.double(), w.double(), bias.double() if bias is not None else None, torch.float64)
            slack = 2.0 ** -8 * (h.double().abs() @ w.double().abs().t()) + 2.0 ** -8 * want.abs() + 1e-5
            over = (y.double().cpu() - want).abs() - slack
            assert not (over > 0).any(), f"worst excess {float(over.max())}"
    k.check_device_errors()


@pytest.mark.parametrize("K_,N", [(1536, 1536), (256, 40), (3584, 3584), (8192, 8192), (8960, 1536), (18944, 1000),
                                  (29568, 700), (640, 129)])
@pytest.mark.parametrize("B", [1, 8, 11, 16])
def test_stream_linear_plain_and_gated(K_, N, B):
    """The streaming projection without a norm: rows kept whole in shared memory where they fit, else streamed in
    tiles beside the weights (any K that is a multiple of 128: the inputs of the down projections of the 7B and
    72B sizes). Plain with bias, and gated: silu(x Wg^T) * (x Wu^T) in the epilogue."""
    x = rnd(B, K_, dtype=torch.bfloat16)
    w = rnd(N, K_, dtype=torch.bfloat16, seed=1, scale=K_ ** -0.5)
    b = rnd(N, dtype=torch.bfloat16, seed=2)
    k = K()
    assert k.can_stream_linear(x.to(DEV), w.to(DEV), b.to(DEV))
    for bias in (None, b):
        y = k.stream_linear(x.to(DEV), w.to(DEV), bias.to(DEV) if bias is not None else None)
        want = REF.linear(x.double(), w.double(), bias.double() if bias is not None else None, torch.float64)
        assert torch.allclose(y.double().cpu(), want, rtol=2.0 ** -7, atol=1e-4 + 2e-8 * K_)
    half = (N // 2)
    if half >= 1:
        wg = w[:2 * half]
        y = k.stream_linear(x.to(DEV), wg.contiguous().to(DEV), None, gated=True)
        g, u = x.double() @ wg[:half].double().t(), x.double() @ wg[half:].double().t()
        want = g / (1 + torch.exp(-g)) * u
        assert y.shape == (B, half)
        assert torch.allclose(y.double().cpu(), want, rtol=2.0 ** -7, atol=1e-4 + 2e-8 * K_)
    k.check_device_errors()


@pytest.mark.parametrize("H,I", [(256, 512), (384, 1920), (2048, 256), (1536, 8960), (3584, 18944), (8192, 3712), (640, 1152)])
@pytest.mark.parametrize("B", [1, 3, 8, 9, 12, 16])
def test_stream_ffn(H, I, B):
    """The feed-forward half as one kernel (norm, gate/up with the activation, all CTAs meet, down) against the
    plain parts in float64 from the same bf16-rounded intermediates, at the widths of the 2B and 7B sizes, at the
    72B hidden size and at small and odd ones. The new residual stream is the fp32 sum bit for bit. The bound: the
    normalised row may differ by one bf16 step where a rounding tie falls the other way (2^-8 on every term of
    gate and up), the activation and the output are rounded to bf16 once each. Launched several times over: the
    barrier's counter stays a multiple of the grid size."""
    x = rnd(B, H, dtype=torch.bfloat16)
    res = rnd(B, H, seed=3, scale=2.0)
    gm = (1.0 + 0.2 * rnd(H, seed=4)).to(torch.bfloat16)
    wgu = rnd(2 * I, H, dtype=torch.bfloat16, seed=1, scale=H ** -0.5)
    wd = rnd(H, I, dtype=torch.bfloat16, seed=2, scale=I ** -0.5)
    k = K()
    if H == 8192 and B > 8:
        assert not k.can_stream_ffn(x.to(DEV), gm.to(DEV), wgu.to(DEV), wd.to(DEV))   # refused by rule
        return
    assert k.can_stream_ffn(x.to(DEV), gm.to(DEV), wgu.to(DEV), wd.to(DEV))
    h, _ = REF.add_rmsnorm(x, res.clone(), gm, 1e-6, torch.bfloat16)
    hd, wg, wu, wdd = h.double(), wgu[:I].double(), wgu[I:].double(), wd.double()
    g, u = hd @ wg.t(), hd @ wu.t()
    act = (g / (1 + torch.exp(-g)) * u)
    act_b = act.to(torch.bfloat16).double()
    want = act_b @ wdd.t()
    dg, du = 2.0 ** -8 * (hd.abs() @ wg.abs().t()), 2.0 ** -8 * (hd.abs() @ wu.abs().t())
    slack_act = 1.1 * u.abs() * dg + g.abs() * du + 2.0 ** -8 * act.abs()
    slack = slack_act @ wdd.abs().t() + 2.0 ** -8 * want.abs() + 1e-5
    xd, wgud, wdn, gmd = x.to(DEV), wgu.to(DEV), wd.to(DEV), gm.to(DEV)
    for with_res in (True, False, True):
        res_dev = res.to(DEV) if with_res else None
        y, new_res = k.stream_ffn(xd, res_dev, gmd, 1e-6, wgud, wdn)
        if with_res:
            assert torch.equal(res_dev.cpu(), res), "the old residual stream must stay as it was"
            assert torch.equal(new_res.cpu(), x.float() + res)
            over = (y.double().cpu() - want).abs() - slack
            assert not (over > 0).any(), f"worst excess {float(over.max())}"
            # the separate kernels give the same to that bound
            h2, _ = k.add_rmsnorm(xd, res.to(DEV), gmd, 1e-6, torch.bfloat16)
            y2 = k.linear(k.gate_up_silu(h2, wgud, torch.bfloat16), wdn, None, torch.bfloat16)
            assert not ((y.double() - y2.double()).cpu().abs() - 2 * slack > 0).any()
        else:
            assert torch.equal(new_res.cpu(), x.float())
            assert torch.isfinite(y.float()).all()
    k.check_device_errors()
    bar, _ = k._stream_state(torch.device(DEV), I)
    n_sm = torch.cuda.get_device_properties(0).multi_processor_count
    assert int(bar.view(torch.int64)[0]) % n_sm == 0, "every CTA arrived at every grid barrier"


def test_a_wait_of_all_ctas_for_one_another_runs_out_and_reports():
    """The CTAs of the feed-forward kernel meet at a counter in global memory; every CTA polls it a bounded number
    of times. Here the barrier is told to expect one arrival more than there are CTAs, and to give up after 2,000
    polls: every CTA runs out of patience, records error 133, keeps its control flow and the kernel returns. The
    host's check raises that error and puts the counter back; the next launch is right."""
    from omniserver_b200.ops import KernelError
    H, I, B = 1536, 8960, 4
    x = rnd(B, H, dtype=torch.bfloat16)
    res = rnd(B, H, seed=3, scale=2.0)
    gm = (1.0 + 0.2 * rnd(H, seed=4)).to(torch.bfloat16)
    wgu = rnd(2 * I, H, dtype=torch.bfloat16, seed=1, scale=H ** -0.5)
    wd = rnd(H, I, dtype=torch.bfloat16, seed=2, scale=I ** -0.5)
    k = K()
    xd, rd, gmd, wgud, wdn = x.to(DEV), res.to(DEV), gm.to(DEV), wgu.to(DEV), wd.to(DEV)
    good, _ = k.stream_ffn(xd, rd, gmd, 1e-6, wgud, wdn)
    k.check_device_errors()
    bar, _ = k._stream_state(torch.device(DEV), I)
    bar.zero_()                       # the count starts at a multiple of (CTAs + 1) too
    torch.cuda.synchronize()
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    k.stream_ffn(xd, rd, gmd, 1e-6, wgud, wdn, wait_limit=2000, bar_extra=1)
    t1.record()
    torch.cuda.synchronize()          # the kernel returned
    assert t0.elapsed_time(t1) < 1000.0
    with pytest.raises(KernelError, match="waited too long for the others"):
        k.check_device_errors()
    assert int(bar.view(torch.int64)[0]) == 0, "the host puts the counter back"
    again, _ = k.stream_ffn(xd, rd, gmd, 1e-6, wgud, wdn)
    k.check_device_errors()
    assert torch.equal(again, good)


def test_a_wait_inside_the_tcgen05_gemm_runs_out_and_reports():
    """Every mbarrier wait of the tcgen05 kernels is bounded. Here the TMA producer announces 16 bytes more to every
    stage's barrier than it copies, so no stage ever becomes full, and the waits give up after 4,096 polls: the MMA
    issuer (or the epilogue waiting for it) records its error, the CTA waits for its copies in flight, frees its
    tensor memory and returns. The host's check raises the error, and the same product launched normally is right."""
    from omniserver_b200.ops import KernelError
    x, w = rnd(256, 128, dtype=torch.bfloat16), rnd(384, 128, dtype=torch.bfloat16, seed=1, scale=0.05)
    k = K()
    k.check_device_errors()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    k.gemm_tcgen05(x.to(DEV), w.to(DEV), None, torch.float32, pairs=False, wait_limit=4096, tx_extra=16)
    t1.record()
    torch.cuda.synchronize()          # the kernel returned
    assert t0.elapsed_time(t1) < 2000.0
    with pytest.raises(KernelError, match="tcgen05 GEMM: the (MMA issuer|epilogue) waited too long"):
        k.check_device_errors()
    got = k.gemm_tcgen05(x.to(DEV), w.to(DEV), None, torch.float32, pairs=False)
    k.check_device_errors()
    want = REF.linear(x.double(), w.double(), None, torch.float64)
    assert torch.allclose(got.double().cpu(), want, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("M,N,K_", [(128, 128, 64), (17, 128, 64), (128, 128, 128), (2048, 2048, 1536), (200, 264, 1536), (130, 1000, 200),
                                    (300, 1536, 8960), (33, 151936, 96), (129, 8, 72)])
@pytest.mark.parametrize("pairs", [False, True])
def test_gemm_tcgen05(M, N, K_, pairs):
    """The TMA/tcgen05/TMEM product at tile-aligned shapes and at ragged ones (rows, columns and K
    that are no multiples of the tile); with one CTA per 128-row tile and with two CTAs sharing a
    256-row tile (cta_group::2)."""
    x, w = rnd(M, K_, dtype=torch.bfloat16), rnd(N, K_, dtype=torch.bfloat16, seed=1, scale=0.05)
    b = rnd(N, dtype=torch.bfloat16, seed=2)
    want0 = REF.linear(x.double(), w.double(), None, torch.float64)
    for bias in (None, b, b.float()):
        for out_dtype in (torch.bfloat16, torch.float32):
            got = K().gemm_tcgen05(x.to(DEV), w.to(DEV), bias.to(DEV) if bias is not None else None, out_dtype,
                                   pairs=pairs)
            K().check_device_errors()
            want = want0 if bias is None else want0 + bias.double()
            # fp32 accumulation in the tensor core over K products: error grows with K and with the
            # size of the partial sums, far below one bf16 rounding of the result
            t = dict(rtol=1e-4, atol=2.5e-8 * K_ * float(want.abs().max()) + 1e-5) if out_dtype == torch.float32 \
                else tol(torch.bfloat16)
            assert torch.allclose(got.double().cpu(), want, **t)


@pytest.mark.parametrize("M,I,K_", [(128, 64, 64), (2048, 8960, 1536), (100, 200, 96), (33, 176, 80), (700, 1000, 264)])
@pytest.mark.parametrize("pairs", [False, True])
def test_gemm_tcgen05_swiglu(M, I, K_, pairs):
    x, w = rnd(M, K_, dtype=torch.bfloat16), rnd(2 * I, K_, dtype=torch.bfloat16, seed=1, scale=0.1)
    got = K().gemm_tcgen05(x.to(DEV), w.to(DEV), None, torch.bfloat16, swiglu=True, pairs=pairs)
    K().check_device_errors()
    assert got.shape == (M, I)
    assert_swiglu_close(got, x, w, I)


@pytest.mark.parametrize("M,N,K_", [(64, 128, 64), (17, 2048, 1536), (64, 1536, 8960), (33, 264, 200), (40, 1000, 72), (128, 1536, 1536),
                                    (100, 24, 520), (1, 130, 64), (64, 19072, 128)])
@pytest.mark.parametrize("splits", [0, 1, 2, 3, 4, 5, 7, 8])
def test_gemm_fewrows(M, N, K_, splits):
    """The product with W on the M side of the MMA: tile-aligned and ragged shapes (rows of x below and at the
    tile's 32, 64 and 128, features and K that are no multiples of the tile, more tiles than SMs), K whole and cut
    into parts that a cluster adds up (more parts than K has blocks are cut back by the launcher)."""
    x, w = rnd(M, K_, dtype=torch.bfloat16), rnd(N, K_, dtype=torch.bfloat16, seed=1, scale=0.05)
    b = rnd(N, dtype=torch.bfloat16, seed=2)
    want0 = REF.linear(x.double(), w.double(), None, torch.float64)
    for bias in (None, b, b.float()):
        got = K().gemm_fewrows(x.to(DEV), w.to(DEV), bias.to(DEV) if bias is not None else None, splits=splits)
        K().check_device_errors()
        want = want0 if bias is None else want0 + bias.double()
        assert got.shape == (M, N) and got.dtype == torch.bfloat16
        assert torch.allclose(got.double().cpu(), want, **tol(torch.bfloat16))


@pytest.mark.parametrize("M,I,K_", [(64, 128, 64), (64, 8960, 1536), (24, 200, 96), (33, 176, 80), (128, 1000, 264), (50, 19000, 64)])
@pytest.mark.parametrize("splits", [0, 1, 2, 6, 8])
@pytest.mark.parametrize("form", [0, 1, 2])
def test_gemm_fewrows_swiglu(M, I, K_, splits, form):
    """With the activation, in both forms: 128 gate and 128 up rows per CTA in two accumulators, and 64 and 64 in the
    two halves of one (gate and up of a feature then lie in different warps' lanes)."""
    x, w = rnd(M, K_, dtype=torch.bfloat16), rnd(2 * I, K_, dtype=torch.bfloat16, seed=1, scale=0.1)
    got = K().gemm_fewrows(x.to(DEV), w.to(DEV), None, swiglu=True, splits=splits, form=form)
    K().check_device_errors()
    assert got.shape == (M, I)
    assert_swiglu_close(got, x, w, I)


def test_gemm_fewrows_does_not_depend_on_the_other_rows():
    """A row's result is the same bits whatever the other rows of the step are, and whichever of the tile's columns it
    occupies: the parts of K are added in a fixed order."""
    k = K()
    x, w = rnd(64, 1536, dtype=torch.bfloat16), rnd(2048, 1536, dtype=torch.bfloat16, seed=1, scale=0.05)
    full = k.gemm_fewrows(x.to(DEV), w.to(DEV))
    part = k.gemm_fewrows(x[20:45].contiguous().to(DEV), w.to(DEV))
    assert torch.equal(full[20:45], part)
    x2 = x.clone()
    x2[:20] = 7.0
    assert torch.equal(k.gemm_fewrows(x2.to(DEV), w.to(DEV))[20:], full[20:])


def test_products_of_few_rows_take_the_fewrows_kernel_where_it_was_measured_faster():
    """``linear`` sends 17 to 64 rows over a long K and few features (a down projection) to the few-rows kernel and a
    squarer matrix to the library, and up to 16 rows only over a large matrix; ``gate_up_silu`` sends 17 to 63 rows
    to it, and up to 16 over a large matrix; the results agree with the plain product."""
    k = K()
    x = rnd(40, 1024, dtype=torch.bfloat16)
    w_down, w_sq = rnd(256, 1024, dtype=torch.bfloat16, seed=1, scale=0.05), rnd(1024, 1024, dtype=torch.bfloat16, seed=2, scale=0.05)
    before = k.counts["gemm_fewrows_tc"]
    got = k.linear(x.to(DEV), w_down.to(DEV), None, torch.bfloat16)
    assert k.counts["gemm_fewrows_tc"] == before + 1
    assert torch.allclose(got.double().cpu(), REF.linear(x.double(), w_down.double(), None, torch.float64), **tol(torch.bfloat16))
    got = k.linear(x.to(DEV), w_sq.to(DEV), None, torch.bfloat16)
    assert k.counts["gemm_fewrows_tc"] == before + 1
    assert torch.allclose(got.double().cpu(), REF.linear(x.double(), w_sq.double(), None, torch.float64), **tol(torch.bfloat16))
    w_gu = rnd(2 * 320, 1024, dtype=torch.bfloat16, seed=3, scale=0.05)
    got = k.gate_up_silu(x.to(DEV), w_gu.to(DEV), torch.bfloat16)
    assert k.counts["gemm_fewrows_tc"] == before + 2
    assert_swiglu_close(got, x, w_gu, 320)
    # up to 16 rows: only over matrices of 64 MB and more
    n0 = k.counts["gemm_fewrows_tc"]
    got = k.gate_up_silu(x[:12].contiguous().to(DEV), w_gu.to(DEV), torch.bfloat16)
    assert k.counts["gemm_fewrows_tc"] == n0
    assert_swiglu_close(got, x[:12], w_gu, 320)
    xg, w_gu_big = rnd(12, 4096, dtype=torch.bfloat16, seed=6), rnd(2 * 4096, 4096, dtype=torch.bfloat16, seed=7, scale=0.03)
    for rows, expect in ((12, 1), (8, 1), (1, 1)):
        n0 = k.counts["gemm_fewrows_tc"]
        got = k.gate_up_silu(xg[:rows].contiguous().to(DEV), w_gu_big.to(DEV), torch.bfloat16)
        assert k.counts["gemm_fewrows_tc"] == n0 + expect
        assert_swiglu_close(got, xg[:rows], w_gu_big, 4096)
    xb, w_big = rnd(12, 8192, dtype=torch.bfloat16, seed=4), rnd(4096, 8192, dtype=torch.bfloat16, seed=5, scale=0.02)
    n0 = k.counts["gemm_fewrows_tc"]
    got = k.linear(xb.to(DEV), w_big.to(DEV), None, torch.bfloat16)
    assert k.counts["gemm_fewrows_tc"] == n0 + 1
    assert torch.allclose(got.double().cpu(), REF.linear(xb.double(), w_big.double(), None, torch.float64), **tol(torch.bfloat16))
    got = k.linear(x[:12].contiguous().to(DEV), w_down.to(DEV), None, torch.bfloat16)
    assert k.counts["gemm_fewrows_tc"] == n0 + 1
    assert torch.allclose(got.double().cpu(), REF.linear(x[:12].double(), w_down.double(), None, torch.float64), **tol(torch.bfloat16))
    k.check_device_errors()


def test_a_wait_inside_the_fewrows_gemm_runs_out_and_reports():
    """As for the other tcgen05 kernels: the producer announces 16 bytes more to every stage than it copies, so no
    stage becomes full and the waits give up after 4,096 polls; the CTAs still meet their cluster at its barriers,
    free their tensor memory and return, the host's check raises, and the same product launched normally is right."""
    from omniserver_b200.ops import KernelError
    x, w = rnd(48, 512, dtype=torch.bfloat16), rnd(384, 512, dtype=torch.bfloat16, seed=1, scale=0.05)
    k = K()
    k.check_device_errors()
    for splits in (1, 4):
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        k.gemm_fewrows(x.to(DEV), w.to(DEV), splits=splits, wait_limit=4096, tx_extra=16)
        t1.record()
        torch.cuda.synchronize()          # the kernel returned
        assert t0.elapsed_time(t1) < 2000.0
        with pytest.raises(KernelError, match=r"tcgen05 GEMM \(few rows\): the (MMA issuer|epilogue) waited too long"):
            k.check_device_errors()
        got = k.gemm_fewrows(x.to(DEV), w.to(DEV), splits=splits)
        k.check_device_errors()
        want = REF.linear(x.double(), w.double(), None, torch.float64)
        assert torch.allclose(got.double().cpu(), want, **tol(torch.bfloat16))


@pytest.mark.parametrize("dtype", DTYPES)
def test_silu_mul(dtype):
    gu = rnd(5, 2 * 200, dtype=dtype, scale=3.0)
    got = K().silu_mul(gu.to(DEV), dtype)
    assert torch.allclose(got.float().cpu(), REF.silu_mul(gu, dtype).float(), **tol(dtype))


def assert_swiglu_close(got, x, w, I):
    """silu(g) * u with g and u rounded to bf16 before the activation and the result rounded to
    bf16: the error allowed is one bf16 ulp (2^-8 relative) on g, on u and on the result, carried
    through the derivative of silu (in its negative tail a relative error of g is amplified by ~|g|)."""
    g = x.double() @ w[:I].double().T
    u = x.double() @ w[I:].double().T
    sig = torch.sigmoid(g)
    silu = g * sig
    dsilu = sig + g * sig * (1 - sig)
    want = silu * u
    ulp = 2.0 ** -8
    bound = ulp * ((g * dsilu * u).abs() + 2 * want.abs()) + 1e-3
    err = (got.double().cpu() - want).abs()
    assert bool((err <= bound).all()), f"max excess {(err - bound).max().item():.3e}"


def _rope_inputs(T, S, half, seed=0):
    g = torch.Generator().manual_seed(seed)
    q_lens = [T // S] * S
    q_lens[-1] += T - sum(q_lens)
    cu_q = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32)
    tok_seq = torch.cat([torch.full((n,), i, dtype=torch.int32) for i, n in enumerate(q_lens)])
    positions = torch.randint(0, 5000, (3, T), generator=g, dtype=torch.int32)
    pos_mode = torch.tensor([i % 2 for i in range(S)], dtype=torch.int32)
    state_slot = torch.tensor([(3 * i + 1) % 8 for i in range(S)], dtype=torch.int32)
    cursor = torch.randint(0, 3000, (8, 2), generator=g, dtype=torch.int32)
    cursor[:, 1] -= 1500
    cursor[:, 0] += 1500
    return positions, pos_mode, tok_seq, cu_q, state_slot, cursor


@pytest.mark.parametrize("hd,theta,sections", [(16, 1e4, (2, 3, 3)), (128, 1e6, (16, 24, 24)), (48, 5e4, (10, 7, 7))])
def test_rope_tables(hd, theta, sections):
    from omniserver_b200.parts import MRope
    T, S = 37, 4
    mr = MRope(hd, theta, sections)
    inv, axis = mr._inv_freq_cpu, mr._axis_cpu
    args = _rope_inputs(T, S, hd // 2)
    cos, sin = K().rope_tables(*[a.to(DEV) for a in args], inv.to(DEV), axis.to(DEV))
    cos_r, sin_r = REF.rope_tables(*args, inv, axis)
    assert torch.allclose(cos.cpu(), cos_r, rtol=0, atol=3e-7)
    assert torch.allclose(sin.cpu(), sin_r, rtol=0, atol=3e-7)
    cur = args[5].clone().to(DEV)
    K().advance_cursor(cur, args[4].to(DEV), args[3].to(DEV))
    cur_r = args[5].clone()
    REF.advance_cursor(cur_r, args[4], args[3])
    assert torch.equal(cur.cpu(), cur_r)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,hd,rot,ps", [(4, 2, 16, 16, 16), (3, 1, 32, 32, 8), (6, 3, 48, 48, 16), (12, 2, 128, 128, 16),
                                              (2, 2, 64, 32, 4)])
def test_rope_kv_write(dtype, nh, nkv, hd, rot, ps):
    T, pages = 21, 9
    qkv = rnd(T, (nh + 2 * nkv) * hd, dtype=dtype)
    ang = rnd(T, rot // 2, seed=3, scale=3.0)
    cos, sin = ang.cos(), ang.sin()
    slot_map = torch.randperm(pages * ps)[:T].to(torch.int32)
    kc, vc = torch.zeros(pages, nkv, ps, hd, dtype=dtype), torch.zeros(pages, nkv, ps, hd, dtype=dtype)
    q_dev, kc_dev, vc_dev = qkv.clone().to(DEV), kc.clone().to(DEV), vc.clone().to(DEV)
    K().rope_kv_write(q_dev, cos.to(DEV), sin.to(DEV), kc_dev, vc_dev, slot_map.to(DEV), nh, nkv, hd, rot)
    q_ref = qkv.clone()
    REF.rope_kv_write(q_ref, cos, sin, kc, vc, slot_map, nh, nkv, hd, rot)
    t = tol(dtype)
    assert torch.allclose(q_dev[:, :nh * hd].float().cpu(), q_ref[:, :nh * hd].float(), **t)
    assert torch.allclose(kc_dev.float().cpu(), kc.float(), **t)
    assert torch.equal(vc_dev.cpu(), vc)
    # an entry that borrows a cache writes nothing
    q2, kc2 = qkv.clone().to(DEV), torch.zeros_like(kc_dev)
    K().rope_kv_write(q2, cos.to(DEV), sin.to(DEV), None, None, None, nh, nkv, hd, rot)
    assert torch.equal(q2[:, :nh * hd], q_dev[:, :nh * hd]) and not kc2.any()
    K().check_device_errors()


def _paged_case(q_lens, kv_lens, nh, nkv, hd, ps, dtype, seed=0, pages_extra=3):
    """Random q and a paged cache with shuffled pages for the given requests."""
    g = torch.Generator().manual_seed(seed)
    S, T = len(q_lens), sum(q_lens)
    n_pages = sum(-(-kv // ps) for kv in kv_lens) + pages_extra
    perm = torch.randperm(n_pages, generator=g).tolist()
    width = max(-(-kv // ps) for kv in kv_lens)
    bt = torch.full((S, width), -1, dtype=torch.int32)
    for s, kv in enumerate(kv_lens):
        for i in range(-(-kv // ps)):
            bt[s, i] = perm.pop()
    kc = (torch.randn(n_pages, nkv, ps, hd, generator=g)).to(dtype)
    vc = (torch.randn(n_pages, nkv, ps, hd, generator=g)).to(dtype)
    qkv = (torch.randn(T, (nh + 2 * nkv) * hd, generator=g)).to(dtype)
    cu_q = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32)
    tok_seq = torch.cat([torch.full((n,), i, dtype=torch.int32) for i, n in enumerate(q_lens)])
    seq_lens = torch.tensor(kv_lens, dtype=torch.int32)
    return qkv, kc, vc, bt, cu_q, seq_lens, tok_seq


def _run_attn(case, nh, nkv, hd, window, dtype, exact=False, units=None):
    qkv, kc, vc, bt, cu_q, seq_lens, tok_seq = case
    scale = hd ** -0.5
    mq, mk = int((cu_q[1:] - cu_q[:-1]).max()), int(seq_lens.max())
    ql = (cu_q[1:] - cu_q[:-1])
    single = ql == 1
    decode_index = torch.where(single, torch.cumsum(single.int(), 0) - 1, torch.full_like(ql, -1)).to(torch.int32)
    got = K().paged_attention(qkv.to(DEV), kc.to(DEV), vc.to(DEV), bt.to(DEV), cu_q.to(DEV), seq_lens.to(DEV),
                              tok_seq.to(DEV), nh, nkv, hd, scale, window, mq, mk, dtype,
                              decode_index=decode_index.to(DEV), n_decode=int(single.sum()),
                              n_multi=int((~single).sum()), exact=exact, units=None if units is None else units.to(DEV))
    want = REF.paged_attention(qkv, kc, vc, bt, cu_q, seq_lens, tok_seq, nh, nkv, hd, scale, window, mq, mk,
                               torch.float32)
    K().check_device_errors()
    return got.float().cpu(), want


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,hd,ps", [(4, 2, 16, 16), (3, 1, 32, 16), (6, 3, 48, 8), (12, 2, 128, 16), (5, 5, 80, 32)])
@pytest.mark.parametrize("window", [None, 20])
def test_paged_attention_mixed_batch(dtype, nh, nkv, hd, ps, window):
    # a whole prompt, a decode token deep into a long context, a 2-token portion, a portion ending on a page edge
    q_lens, kv_lens = [33, 1, 2, 16, 1], [33, 300, 47, 64, 1]
    got, want = _run_attn(_paged_case(q_lens, kv_lens, nh, nkv, hd, ps, dtype), nh, nkv, hd, window, dtype)
    assert torch.allclose(got, want, **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hd", list(range(16, 257, 16)))
def test_paged_attention_every_head_size(dtype, hd):
    """Head sizes in steps of 16 up to 256, prompt portions beside decode tokens with long contexts: each size is
    either computed right by whichever kernel takes it, or refused with an error that says so."""
    nh, nkv, ps = 6, 2, 16
    q_lens, kv_lens = [150, 1, 2, 1, 130], [150, 700, 260, 129, 400]
    case = _paged_case(q_lens, kv_lens, nh, nkv, hd, ps, dtype, seed=hd)
    try:
        got, want = _run_attn(case, nh, nkv, hd, None, dtype)
    except Exception as e:      # a refusal names the size
        assert "head" in str(e).lower() or "unsupported" in str(e).lower(), e
        return
    if dtype == torch.bfloat16:   # the bound that follows from rounding P and the output to bf16 (one or two of
        _assert_attn_close(got, want, case, nh, nkv, hd, None, f"head size {hd}")   # 10^5 values pass the flat one by a hair)
    else:
        assert torch.allclose(got, want, **tol(dtype))


@pytest.mark.parametrize("nh,nkv,hd,ps", [(12, 2, 128, 16), (28, 4, 128, 16), (6, 3, 48, 8), (4, 4, 64, 64), (40, 2, 32, 16),
                                          (8, 1, 256, 16), (16, 2, 128, 16), (7, 1, 128, 32), (8, 2, 64, 4), (12, 2, 128, 8),
                                          (6, 6, 64, 2), (24, 2, 128, 16)])
@pytest.mark.parametrize("window", [None, 300])
def test_decode_attention_long_contexts_split_keys(nh, nkv, hd, ps, window):
    """Single-token requests with long and uneven contexts: the keys are split over CTAs and merged. Head
    sizes 64 and 128 with at most 8 query heads per kv head run in the kernel that streams K and V into
    registers (pages down to 2 tokens, groups of 6, 7 and 8 heads), the others in the shared-memory kernel."""
    kv_lens = [2048, 1, 777, 64, 65, 3000, 128, 129]
    case = _paged_case([1] * len(kv_lens), kv_lens, nh, nkv, hd, ps, torch.bfloat16, seed=3)
    got, want = _run_attn(case, nh, nkv, hd, window, torch.bfloat16)
    assert torch.allclose(got, want, **tol(torch.bfloat16))


@pytest.mark.parametrize("nh,nkv,batch", [(12, 2, 40), (28, 4, 64), (12, 2, 7)])
def test_decode_attention_in_a_given_order_of_requests(nh, nkv, batch):
    """The order in which the requests' CTAs start (longest first, as the engine asks for; any permutation) changes
    nothing of the result: bitwise the same output as without it, more CTAs than SMs or fewer."""
    hd, ps = 128, 16
    g = torch.Generator().manual_seed(batch)
    kv_lens = [int(x) for x in torch.randint(1, 1200, (batch,), generator=g)]
    case = _paged_case([1] * batch, kv_lens, nh, nkv, hd, ps, torch.bfloat16, seed=batch + 1)
    qkv, kc, vc, bt, cu_q, seq_lens, tok_seq = [t.to(DEV) for t in case]
    ts = torch.arange(batch, device=DEV, dtype=torch.int32)
    outs = []
    for order in (None, torch.argsort(-seq_lens.cpu(), stable=True).to(torch.int32), torch.randperm(batch, generator=g).to(torch.int32)):
        outs.append(K().paged_attention(qkv, kc, vc, bt, cu_q, seq_lens, tok_seq, nh, nkv, hd, hd ** -0.5, None, 1, max(kv_lens),
                                        torch.bfloat16, decode_index=ts, n_decode=batch, n_multi=0, scratch={},
                                        order=None if order is None else order.to(DEV)).cpu())
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    want = REF.paged_attention(*case, nh, nkv, hd, hd ** -0.5, None, 1, max(kv_lens), torch.float32)
    assert torch.allclose(outs[1].float(), want, **tol(torch.bfloat16))
    # told that the lengths are uneven the kernel may cut the keys into more parts: the same result up to rounding
    more = K().paged_attention(qkv, kc, vc, bt, cu_q, seq_lens, tok_seq, nh, nkv, hd, hd ** -0.5, None, 1, max(kv_lens),
                               torch.bfloat16, decode_index=ts, n_decode=batch, n_multi=0, scratch={},
                               order=torch.argsort(-seq_lens.cpu(), stable=True).to(torch.int32).to(DEV), uneven=True).cpu()
    assert torch.allclose(more.float(), want, **tol(torch.bfloat16))
    K().check_device_errors()


@pytest.mark.parametrize("batch", [1, 3, 20, 40, 150])
@pytest.mark.parametrize("stream", [True, False])
def test_decode_attention_split_and_merge_paths(batch, stream):
    """The number of requests decides how many splits a request gets and how they are merged (one split,
    a cluster, scratch memory and the last CTA); every path of both decode kernels against the reference."""
    nh, nkv, hd, ps = 12, 2, 128, 16
    g = torch.Generator().manual_seed(batch)
    kv_lens = [int(x) for x in torch.randint(1, 1400, (batch,), generator=g)]
    kv_lens[0] = 1399
    case = _paged_case([1] * batch, kv_lens, nh, nkv, hd, ps, torch.bfloat16, seed=batch)
    K().decode_stream = stream
    try:
        got, want = _run_attn(case, nh, nkv, hd, None, torch.bfloat16)
    finally:
        K().decode_stream = True
    assert torch.allclose(got, want, **tol(torch.bfloat16))


@pytest.mark.parametrize("nh,nkv,hd,ps,rot", [(12, 2, 128, 16, 128), (6, 3, 48, 8, 48), (16, 1, 64, 16, 32)])
def test_decode_attention_with_fused_rotary_and_cache_write(nh, nkv, hd, ps, rot):
    """The decode kernel rotating q and k and storing the new key/value itself must give what the
    rotary kernel followed by the plain decode kernel gives, and leave the same cache behind."""
    kv_lens = [2048, 1, 777, 64, 65, 129]
    S = len(kv_lens)
    qkv, kc, vc, bt, cu_q, seq_lens, tok_seq = [t.to(DEV) for t in _paged_case([1] * S, kv_lens, nh, nkv, hd, ps, torch.bfloat16, seed=5)]
    ang = rnd(S, rot // 2, seed=3, scale=3.0)
    cos, sin = ang.cos().to(DEV), ang.sin().to(DEV)
    slot_map = torch.stack([bt[s, (kv - 1) // ps] * ps + (kv - 1) % ps for s, kv in enumerate(kv_lens)]).to(torch.int32)
    didx = torch.arange(S, dtype=torch.int32, device=DEV)
    args = dict(decode_index=didx, n_decode=S, n_multi=0)
    q1, k1, v1 = qkv.clone(), kc.clone(), vc.clone()
    K().rope_kv_write(q1, cos, sin, k1, v1, slot_map, nh, nkv, hd, rot)
    want = K().paged_attention(q1, k1, v1, bt, cu_q, seq_lens, tok_seq, nh, nkv, hd, hd ** -0.5, None, 1, max(kv_lens),
                               torch.bfloat16, **args)
    q2, k2, v2 = qkv.clone(), kc.clone(), vc.clone()
    got = K().paged_attention(q2, k2, v2, bt, cu_q, seq_lens, tok_seq, nh, nkv, hd, hd ** -0.5, None, 1, max(kv_lens),
                              torch.bfloat16, rope=(cos, sin, slot_map, rot), **args)
    K().check_device_errors()
    assert torch.equal(k2, k1) and torch.equal(v2, v1)
    assert torch.equal(got, want)


@pytest.mark.parametrize("window", [None, 100])
def test_decode_attention_finds_one_key_that_matters(window):
    """As below, for the split-key decode kernel: one key dominates, placed at tile, split and window edges."""
    nh, nkv, hd, ps, dtype = 12, 2, 128, 16, torch.bfloat16
    kv_len = 1500
    p = kv_len - 1
    spots = [0, 15, 16, 17, 63, 64, 93, 94, 95, 96, 127, 128, 255, 256, 1023, 1024, p - 1, p]
    if window:
        spots = [p - window, p - window + 1, p - window + 2, 1407, 1408, p]
    for j in spots:
        case = list(_paged_case([1, 1], [kv_len, 900], nh, nkv, hd, ps, dtype, seed=j + 1))
        qkv, kc, vc, bt = case[0], case[1], case[2], case[3]
        g = nh // nkv
        for kvh in range(nkv):
            qh = qkv[0, kvh * g * hd:(kvh * g + 1) * hd].float()
            for h in range(kvh * g, (kvh + 1) * g):
                qkv[0, h * hd:(h + 1) * hd] = qh.to(dtype)
            kvec = qh / qh.norm() ** 2 * 30.0 * math.sqrt(hd)
            page = int(bt[0, j // ps])
            kc[page, kvh, j % ps] = kvec.to(dtype)
            vc[page, kvh, j % ps] = 7.0
        got, want = _run_attn(tuple(case), nh, nkv, hd, window, dtype)
        assert torch.allclose(got, want, **tol(dtype)), f"key {j}"
        visible = not window or j > p - window
        if visible:
            assert got[0].mean() > 6.5, f"key {j} should dominate"
        else:
            assert got[0].abs().mean() < 2.0, f"key {j} must be invisible"


def test_decode_attention_of_one_very_long_request_takes_more_splits():
    """One request of 40,000 keys: its keys are cut into more than 32 splits (62 of 704 keys here), merged by the
    CTA that finishes last. One key dominates, placed in the first, a middle and the last split and at split edges."""
    nh, nkv, hd, ps, dtype = 12, 2, 128, 32, torch.bfloat16
    kv_len = 40000
    chunk, nsplits = K().decode_splits(1, nkv, nh // nkv, kv_len, K().stream_target_ctas,
                                       max_splits=max(K().stream_max_splits, min(K().stream_max_splits_long, kv_len // 640)))
    assert 32 < nsplits <= 64 and nsplits * nkv <= 148
    for j in (0, chunk - 1, chunk, 20 * chunk + 5, (nsplits - 1) * chunk, kv_len - 1):
        case = list(_paged_case([1], [kv_len], nh, nkv, hd, ps, dtype, seed=j + 1))
        qkv, kc, vc, bt = case[0], case[1], case[2], case[3]
        g = nh // nkv
        for kvh in range(nkv):
            qh = qkv[0, kvh * g * hd:(kvh * g + 1) * hd].float()
            for h in range(kvh * g, (kvh + 1) * g):
                qkv[0, h * hd:(h + 1) * hd] = qh.to(dtype)
            kvec = qh / qh.norm() ** 2 * 40.0 * math.sqrt(hd)
            page = int(bt[0, j // ps])
            kc[page, kvh, j % ps] = kvec.to(dtype)
            vc[page, kvh, j % ps] = 7.0
        got, want = _run_attn(tuple(case), nh, nkv, hd, None, dtype)
        assert torch.allclose(got, want, **tol(dtype)), f"key {j}"
        assert got[0].mean() > 6.5, f"key {j} should dominate"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [None, 24])
def test_paged_attention_finds_one_key_that_matters(dtype, window):
    """Random keys give near-uniform softmax, which hides a missed key among hundreds. Here one key
    is made to dominate: its score is ~25 above the rest, its value is distinctive. Placed at the
    first key, at both sides of page edges, at the window's edge and just outside it, and at the
    query itself, the output must be that value or, when the key is not visible, must not change."""
    nh, nkv, hd, ps = 4, 2, 32, 16
    kv_len, q_len = 200, 3
    for qi in range(q_len):
        p = kv_len - q_len + qi
        spots = [0, 15, 16, 17, p - 1, p, p + 1 if p + 1 < kv_len else p]
        if window:
            spots += [p - window + 1, p - window, p - window + 2]
        for j in spots:
            case = list(_paged_case([q_len], [kv_len], nh, nkv, hd, ps, dtype, seed=j + 7))
            qkv, kc, vc, bt = case[0], case[1], case[2], case[3]
            t = qi
            for kvh in range(nkv):
                # the key at j is aligned with the queries of the heads of this group
                qh = qkv[t, (kvh * (nh // nkv)) * hd:(kvh * (nh // nkv) + 1) * hd].float()
                for h in range(kvh * (nh // nkv), (kvh + 1) * (nh // nkv)):
                    qkv[t, h * hd:(h + 1) * hd] = qh.to(dtype)
                kvec = qh / qh.norm() ** 2 * 25.0 * math.sqrt(hd)
                page = int(bt[0, j // ps])
                kc[page, kvh, j % ps] = kvec.to(dtype)
                vc[page, kvh, j % ps] = 7.0
            got, want = _run_attn(tuple(case), nh, nkv, hd, window, dtype)
            visible = j <= p and (not window or j > p - window)
            assert torch.allclose(got, want, **tol(dtype)), f"key {j}, query at {p}"
            if visible:
                assert got[t].mean() > 6.5, f"key {j} should dominate the query at {p}"
            else:
                assert got[t].abs().mean() < 2.0, f"key {j} must be invisible to the query at {p}"


def _attn_bf16_bound(case, nh, nkv, hd, window, want):
    """What bf16 tensor-core attention may differ by: the probabilities are rounded to bf16 (2^-9
    relative each) before they meet the values, so the numerator is off by at most 2^-9 sum_j p_j |v_j|,
    and the output is rounded once more; a factor of two covers the fp32 sums' order."""
    qkv, kc, vc, bt, cu_q, seq_lens, tok_seq = case
    mq, mk = int((cu_q[1:] - cu_q[:-1]).max()), int(seq_lens.max())
    mag = REF.paged_attention(qkv, kc, vc.abs(), bt, cu_q, seq_lens, tok_seq, nh, nkv, hd, hd ** -0.5, window, mq, mk,
                              torch.float32)
    return 2.0 ** -8 * (mag + want.abs()) + 1e-6


def _assert_attn_close(got, want, case, nh, nkv, hd, window, what=""):
    bound = _attn_bf16_bound(case, nh, nkv, hd, window, want)
    over = (got - want).abs() - bound
    assert not (over > 0).any(), f"{what}: {int((over > 0).sum())} values beyond the bf16 bound, worst by {float(over.max()):.3g}"


def _poison_unused(case, ps):
    """NaN wherever no live key lies: pages of nobody, and the rest of each request's last page."""
    qkv, kc, vc, bt, cu_q, seq_lens, tok_seq = case
    live = torch.zeros(kc.shape[0], ps, dtype=torch.bool)
    for s, kv in enumerate(seq_lens.tolist()):
        for j in range(kv):
            live[int(bt[s, j // ps]), j % ps] = True
    dead = ~live
    for c in (kc, vc):
        c.permute(0, 2, 1, 3)[dead] = float("nan")
    return case


@pytest.mark.parametrize("nh,nkv,hd,ps", [(12, 2, 128, 16), (4, 4, 64, 8), (6, 2, 64, 32), (2, 1, 128, 128), (3, 1, 128, 256),
                                          (2, 2, 64, 64)])
@pytest.mark.parametrize("window", [None, 100, 200])
def test_prefill_attention_tcgen05(nh, nkv, hd, ps, window):
    """Prompt portions on the tcgen05 kernel: several 128-key tiles, portions that start and end inside
    tiles and pages, a request shorter than a tile, single tokens beside them; what lies in the pages
    beyond a request's length is NaN and must not reach the output."""
    assert K().tc_prefill
    q_lens, kv_lens = [300, 1, 130, 128, 2, 257], [300, 500, 700, 128, 259, 1000]
    case = _poison_unused(_paged_case(q_lens, kv_lens, nh, nkv, hd, ps, torch.bfloat16, seed=11), ps)
    before = K().launches
    got, want = _run_attn(case, nh, nkv, hd, window, torch.bfloat16)
    assert K().launches - before == 2  # the tcgen05 kernel and the decode kernel
    assert torch.isfinite(got).all()
    _assert_attn_close(got, want, case, nh, nkv, hd, window, "tcgen05")
    # the mma.sync kernel stays within the same bound
    K().tc_prefill = False
    try:
        other, _ = _run_attn(case, nh, nkv, hd, window, torch.bfloat16)
    finally:
        K().tc_prefill = True
    _assert_attn_close(other, want, case, nh, nkv, hd, window, "mma.sync")


@pytest.mark.parametrize("nh,nkv,hd,ps,window", [(12, 2, 128, 16, None), (14, 2, 64, 32, 150), (16, 4, 128, 64, None)])
def test_prefill_attention_tcgen05_many_units_per_cta(nh, nkv, hd, ps, window):
    """More units of work (128 rows of a request and head) than SMs, several times over: a CTA takes one
    after another (a long one, then short ones, empty ones between them) with its barriers, tensor memory and
    K/V stages running on; requests of very different lengths, with and without earlier context."""
    q_lens = [600, 129, 1, 384, 77, 512, 2, 640, 300]
    kv_lens = [600, 1200, 333, 384, 900, 513, 130, 1500, 301]
    case = _poison_unused(_paged_case(q_lens, kv_lens, nh, nkv, hd, ps, torch.bfloat16, seed=23), ps)
    assert -(-max(q_lens) // 128) * nh * len(q_lens) > 3 * 148
    got, want = _run_attn(case, nh, nkv, hd, window, torch.bfloat16)
    assert torch.isfinite(got).all()
    _assert_attn_close(got, want, case, nh, nkv, hd, window, "tcgen05, several units per CTA")
    # given the list of (request, row tile) pairs that have work, as the engine's plan gives it: the same output
    from omniserver_b200.ops import CudaKernels
    units = torch.from_numpy(CudaKernels.prefill_units(q_lens, kv_lens))
    assert units.shape[0] == sum(-(-q // 128) for q in q_lens if q > 1)
    listed, _ = _run_attn(case, nh, nkv, hd, window, torch.bfloat16, units=units)
    assert torch.equal(listed, got)


@pytest.mark.parametrize("window", [None, 130])
def test_prefill_attention_tcgen05_finds_one_key_that_matters(window):
    """One dominating key at the edges of the 128-key tiles, of pages, of the window and at the query
    itself, for queries in the first and in a later 128-row tile of the portion."""
    nh, nkv, hd, ps = 4, 2, 64, 16
    kv_len, q_len = 700, 300
    dtype = torch.bfloat16
    for qi in (0, 127, 128, 299):
        p = kv_len - q_len + qi
        spots = [0, 127, 128, 255, 256, 511, 512, p - 1, p, min(p + 1, kv_len - 1)]
        if window:
            spots += [p - window + 1, p - window, p - window + 2]
        for j in spots:
            case = list(_paged_case([q_len], [kv_len], nh, nkv, hd, ps, dtype, seed=j + 7))
            qkv, kc, vc, bt = case[0], case[1], case[2], case[3]
            for kvh in range(nkv):
                qh = qkv[qi, (kvh * (nh // nkv)) * hd:(kvh * (nh // nkv) + 1) * hd].float()
                for h in range(kvh * (nh // nkv), (kvh + 1) * (nh // nkv)):
                    qkv[qi, h * hd:(h + 1) * hd] = qh.to(dtype)
                kvec = qh / qh.norm() ** 2 * 25.0 * math.sqrt(hd)
                page = int(bt[0, j // ps])
                kc[page, kvh, j % ps] = kvec.to(dtype)
                vc[page, kvh, j % ps] = 7.0
            got, want = _run_attn(tuple(case), nh, nkv, hd, window, dtype)
            visible = j <= p and (not window or j > p - window)
            _assert_attn_close(got, want, tuple(case), nh, nkv, hd, window, f"key {j}, query at {p}")
            if visible:
                assert got[qi].mean() > 6.5, f"key {j} should dominate the query at {p}"
            else:
                assert got[qi].abs().mean() < 2.0, f"key {j} must be invisible to the query at {p}"


def test_prefill_attention_tcgen05_rescales_when_the_maximum_grows():
    """Scores that grow along the keys: the running offset has to move several times and the
    accumulated output has to be rescaled in tensor memory each time."""
    nh, nkv, hd, ps = 2, 1, 128, 16
    kv_len = q_len = 640
    case = list(_paged_case([q_len], [kv_len], nh, nkv, hd, ps, torch.bfloat16, seed=5))
    qkv, kc, bt = case[0], case[1], case[3]
    qkv[:, :nh * hd] = 0
    qkv[:, 0] = 4.0
    qkv[:, hd] = 4.0
    for j in range(kv_len):
        kc[int(bt[0, j // ps]), 0, j % ps, 0] = 0.25 * j   # score of key j: j / sqrt(hd) * ... grows by tiles
    got, want = _run_attn(tuple(case), nh, nkv, hd, None, torch.bfloat16)
    _assert_attn_close(got, want, tuple(case), nh, nkv, hd, None)


def test_paged_attention_fp32_is_independent_of_the_batch():
    """In 32-bit the kernel's sums run in an order fixed by absolute key positions: a request's
    output is bitwise the same alone, cut into portions, or beside other requests."""
    nh, nkv, hd, ps = 6, 3, 48, 16
    full = _paged_case([70], [70], nh, nkv, hd, ps, torch.float32, seed=11)
    qkv, kc, vc, bt, cu_q, seq_lens, tok_seq = full
    whole, _ = _run_attn(full, nh, nkv, hd, None, torch.float32)
    # last 5 tokens as a portion beside another request's decode token
    other = _paged_case([1], [40], nh, nkv, hd, ps, torch.float32, seed=12)
    n_pages = kc.shape[0]
    kc2, vc2 = torch.cat([kc, other[1]]), torch.cat([vc, other[2]])
    bt2 = torch.full((2, bt.shape[1]), -1, dtype=torch.int32)
    bt2[1] = bt[0]
    bt2[0, :other[3].shape[1]] = other[3][0] + n_pages
    qkv2 = torch.cat([other[0], qkv[65:70]])
    case = (qkv2, kc2, vc2, bt2, torch.tensor([0, 1, 6], dtype=torch.int32), torch.tensor([40, 70], dtype=torch.int32),
            torch.tensor([0, 1, 1, 1, 1, 1], dtype=torch.int32))
    part, _ = _run_attn(case, nh, nkv, hd, None, torch.float32)
    assert torch.equal(part[1:], whole[65:70])


@pytest.mark.parametrize("V", [512, 1000, 151936])
def test_sample_greedy_and_temperature(V):
    R = 5
    logits = rnd(R, V, scale=2.0)
    logits[1, 7] = logits[1, 900 % V] = logits[1].max() + 1   # a tie: the lowest index wins
    got = K().sample(logits.to(DEV), None, None).cpu()
    assert torch.equal(got, REF.sample(logits, None, None))
    # the tokens can be kept on the device at given places as well
    keep, at = torch.full((9,), -7, dtype=torch.int32, device=DEV), torch.tensor([4, 0, 8, 1, 6], dtype=torch.int32)
    temps = torch.tensor([0.8, 0.0, 1.5, 0.3, 1.0])
    for tp, u in ((None, None), (temps.to(DEV), torch.full((R,), 0.37, device=DEV))):
        ids = K().sample(logits.to(DEV), tp, u, keep, at.to(DEV)).cpu()
        assert torch.equal(keep.cpu()[at.long()], ids) and (keep.cpu()[[2, 3, 5, 7]] == -7).all()
    for trial in range(8):
        u = torch.rand(R, generator=torch.Generator().manual_seed(trial))
        got = K().sample(logits.to(DEV), temps.to(DEV), u.to(DEV)).cpu()
        for r in range(R):
            if temps[r] == 0:
                assert got[r] == logits[r].argmax() or logits[r, got[r]] == logits[r].max()
                continue
            # the chosen index's CDF interval must hold u up to float32 rounding of the running sum
            p = torch.softmax(logits[r].double() / float(temps[r]), -1)
            cdf = torch.cumsum(p, 0)
            i = int(got[r])
            lo = float(cdf[i - 1]) if i > 0 else 0.0
            assert lo - 1e-4 <= float(u[r]) <= float(cdf[i]) + 1e-4, f"row {r}: u={float(u[r])} not in [{lo}, {float(cdf[i])}]"
