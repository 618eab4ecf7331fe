"""Times single kernels at the shapes of a decode or prefill step and prints achieved bandwidth.

    python -m omniserver_b200.ops.microbench [--what gemm|gemm_prefill|attn_decode|attn_prefill|ffn_fused|norm|all]
        [--batch 1,8,64] [--ctx 2048] [--hidden 1536 --heads 12 --kv-heads 2 --head-dim 128 --inter 8960 --vocab 151936]
        [--peak-gbs 6544]

Every timed call runs on its own copy of the weights or cache pages (enough copies to exceed the
L2), and the calls are replayed from a CUDA graph so that host launch time is not measured.
Times are CUDA-event times per call; GB/s counts the bytes the kernel has to read once.
"""

from __future__ import annotations

import argparse
from typing import Callable, List

import torch

from .. import ops


def graph_time_us(fn: Callable[[int], None], n_rot: int, iters: int = 5) -> float:
    """Mean time of fn(i) over i in range(n_rot), replayed from a CUDA graph."""
    for i in range(n_rot):
        fn(i)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(n_rot):
            fn(i)
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / (iters * n_rot)


def bench_gemm(args, K, dev, peak) -> None:
    H, I, V = args.hidden, args.inter, args.vocab
    qkv = (args.heads + 2 * args.kv_heads) * args.head_dim
    shapes = [("qkv", qkv, H, 0), ("o", H, args.heads * args.head_dim, 0), ("gate_up+silu", 2 * I, H, 1), ("down", H, I, 0),
              ("head", V, H, 0)]
    print("== projections: y[M,N] = x[M,K] W[N,K]^T  (us | GB/s of W | fraction of %.0f GB/s)" % peak)
    for name, N, Kd, mode in shapes:
        if args.only and name not in args.only:
            continue
        n_rot = max(3, int(300e6 // (N * Kd * 2)) + 1)
        ws = [torch.randn(N, Kd, device=dev, dtype=torch.bfloat16) * 0.02 for _ in range(n_rot)]
        for M in args.batch:
            x = torch.randn(M, Kd, device=dev, dtype=torch.bfloat16)
            out_dt = torch.float32 if name == "head" else torch.bfloat16
            cols = []
            for warps in args.warps if M <= (16 if mode else 64) else []:
                K.skinny_warps = warps
                if mode:
                    us = graph_time_us(lambda i: K.gate_up_silu(x, ws[i], out_dt), n_rot)
                else:
                    us = graph_time_us(lambda i: K.gemm_skinny(x, ws[i], None, out_dt), n_rot)
                gbs = N * Kd * 2 / us / 1e3
                cols.append(f"skinny warps={warps}: {us:7.1f} us {gbs:6.0f} GB/s {gbs / peak:4.2f}")
            K.skinny_warps = 0
            if name != "head" and K.can_stream_linear(x, ws[0], None):
                us = graph_time_us(lambda i: K.stream_linear(x, ws[i], None, gated=bool(mode)), n_rot)
                gbs = N * Kd * 2 / us / 1e3
                cols.append(f"streaming: {us:7.1f} us {gbs:6.0f} GB/s {gbs / peak:4.2f}")
            if name == "qkv" and K.can_stream_linear(x, ws[0], None):
                # with the add + norm in front of it: inside the kernel, or as a kernel of its own
                res = torch.randn(M, Kd, device=dev)
                gm = torch.ones(Kd, device=dev, dtype=torch.bfloat16)

                def apart(i):
                    h, _ = K.add_rmsnorm(x, res, gm, 1e-6, torch.bfloat16)
                    K.stream_linear(h, ws[i], None)
                us2 = graph_time_us(apart, n_rot)
                txt = f"norm + streaming: {us2:7.1f} us"
                if K.can_stream_linear(x, ws[0], None, gm):
                    us1 = graph_time_us(lambda i: K.stream_linear(x, ws[i], None, norm=(res, gm, 1e-6)), n_rot)
                    txt = f"norm inside: {us1:7.1f} us | " + txt
                cols.append(txt)
            if name != "head" and M <= K.FEWROWS_MAX_ROWS_KERNEL:
                for sp in args.splits:
                    for form in ((1, 2) if mode and sp else (0,)):
                        us = graph_time_us(lambda i: K.gemm_fewrows(x, ws[i], None, swiglu=bool(mode), splits=sp, form=form), n_rot)
                        gbs = N * Kd * 2 / us / 1e3
                        plan = K.lib.osb_gemm_fewrows_tc_plan(M, N, Kd, mode)
                        what = f"K in {sp}" + (", 64 + 64 rows" if form == 2 else "") if sp else \
                            f"its choice (K in {plan % 100}" + (", 64 + 64 rows)" if plan >= 100 else ")")
                        cols.append(f"few rows, {what}: {us:7.1f} us {gbs:6.0f} GB/s {gbs / peak:4.2f}")
            if not mode:
                us = graph_time_us(lambda i: torch.mm(x, ws[i].t()), n_rot)
                cols.append(f"library: {us:7.1f} us {N * Kd * 2 / us / 1e3:6.0f} GB/s")
            elif M > 16:
                us = graph_time_us(lambda i: K.silu_mul(torch.mm(x, ws[i].t()), torch.bfloat16), n_rot)
                cols.append(f"library + activation: {us:7.1f} us {N * Kd * 2 / us / 1e3:6.0f} GB/s")
                us = graph_time_us(lambda i: K.gemm_tcgen05(x, ws[i], None, torch.bfloat16, swiglu=True, pairs=False), n_rot)
                cols.append(f"128-row tiles of x: {us:7.1f} us {N * Kd * 2 / us / 1e3:6.0f} GB/s")
            print(f"{name:13s} M={M:3d} N={N:6d} K={Kd:5d} | " + " | ".join(cols), flush=True)


def bench_gemm_prefill(args, K, dev, peak) -> None:
    H, I = args.hidden, args.inter
    qkv = (args.heads + 2 * args.kv_heads) * args.head_dim
    shapes = [("qkv", qkv, H, 0), ("o", H, args.heads * args.head_dim, 0), ("gate_up", 2 * I, H, 0), ("gate_up+silu", 2 * I, H, 1),
              ("down", H, I, 0)]
    print("== projections with many rows: tcgen05 kernel vs the vendor library (us | TFLOP/s)")
    for M in args.rows:
        for name, N, Kd, mode in shapes:
            if args.only and name not in args.only:
                continue
            x = torch.randn(M, Kd, device=dev, dtype=torch.bfloat16)
            ws = [torch.randn(N, Kd, device=dev, dtype=torch.bfloat16) * 0.02 for _ in range(3)]
            fl = 2.0 * M * N * Kd
            us1 = graph_time_us(lambda i: K.gemm_tcgen05(x, ws[i], None, torch.bfloat16, swiglu=bool(mode), pairs=False), 3)
            us = graph_time_us(lambda i: K.gemm_tcgen05(x, ws[i], None, torch.bfloat16, swiglu=bool(mode), pairs=True), 3)
            if mode:
                lib = graph_time_us(lambda i: K.silu_mul(torch.mm(x, ws[i].t()), torch.bfloat16), 3)
            else:
                lib = graph_time_us(lambda i: torch.mm(x, ws[i].t()), 3)
            print(f"M={M:5d} {name:13s} N={N:6d} K={Kd:5d} | tcgen05 one CTA per tile {us1:8.1f} us {fl / us1 / 1e6:7.1f} TF | "
                  f"CTA pairs {us:8.1f} us {fl / us / 1e6:7.1f} TF | library {lib:8.1f} us {fl / lib / 1e6:7.1f} TF", flush=True)


def bench_attn_decode(args, K, dev, peak) -> None:
    nh, nkv, hd, ps, ctx = args.heads, args.kv_heads, args.head_dim, args.page_size, args.ctx
    print("== decode attention: one token per request over %d cached keys (us | GB/s of K,V | fraction)" % ctx)
    for B in args.batch:
        pages = B * (-(-ctx // ps))
        n_rot = max(3, int(300e6 // (pages * nkv * ps * hd * 4)) + 1)
        kc = [torch.randn(pages, nkv, ps, hd, device=dev, dtype=torch.bfloat16) for _ in range(n_rot)]
        vc = [torch.randn(pages, nkv, ps, hd, device=dev, dtype=torch.bfloat16) for _ in range(n_rot)]
        qkv = torch.randn(B, (nh + 2 * nkv) * hd, device=dev, dtype=torch.bfloat16)
        bt = torch.randperm(pages, device=dev).to(torch.int32).view(B, -1)
        cu_q = torch.arange(B + 1, device=dev, dtype=torch.int32)
        sl = torch.full((B,), ctx, device=dev, dtype=torch.int32)
        ts = torch.arange(B, device=dev, dtype=torch.int32)
        pool = {}
        for target, K.stream_max_splits, K.stream_max_splits_long in [(t, m, max(m, 64)) for t in args.target_ctas for m in args.max_splits]:
            keep = K.stream_target_ctas
            K.stream_target_ctas = target
            try:
                us = graph_time_us(lambda i: K.paged_attention(
                    qkv, kc[i], vc[i], bt, cu_q, sl, ts, nh, nkv, hd, hd ** -0.5, None, 1, ctx, torch.bfloat16,
                    decode_index=ts, n_decode=B, n_multi=0, scratch=pool), n_rot)
            finally:
                K.stream_target_ctas = keep
            orig = ops.CudaKernels.decode_splits
            gbs = B * ctx * nkv * hd * 2 * 2 / us / 1e3
            stream = K.decode_stream and hd in (64, 128) and nh // nkv <= 8
            if stream:
                chunk, nsp = orig(B, nkv, nh // nkv, ctx, target, max_splits=max(K.stream_max_splits, min(K.stream_max_splits_long, ctx // 640)))
                how = "streaming kernel, " + ("cluster merge" if nsp in K.stream_cluster_sizes else
                                              "one split" if nsp == 1 else "merge by the last CTA")
            else:
                chunk, nsp = orig(B, nkv, nh // nkv, ctx, target)
                how = "shared-memory kernel"
            print(f"B={B:3d} splits={nsp:3d} {how:40s} | {us:7.1f} us {gbs:6.0f} GB/s {gbs / peak:4.2f}", flush=True)


def bench_attn_prefill(args, K, dev, peak) -> None:
    nh, nkv, hd, ps, ctx = args.heads, args.kv_heads, args.head_dim, args.page_size, args.ctx
    pages = -(-ctx // ps)
    kc = torch.randn(pages, nkv, ps, hd, device=dev, dtype=torch.bfloat16)
    vc = torch.randn(pages, nkv, ps, hd, device=dev, dtype=torch.bfloat16)
    qkv = torch.randn(ctx, (nh + 2 * nkv) * hd, device=dev, dtype=torch.bfloat16)
    bt = torch.randperm(pages, device=dev).to(torch.int32).view(1, -1)
    cu_q = torch.tensor([0, ctx], device=dev, dtype=torch.int32)
    sl = torch.tensor([ctx], device=dev, dtype=torch.int32)
    ts = torch.zeros(ctx, device=dev, dtype=torch.int32)
    di = torch.full((1,), -1, device=dev, dtype=torch.int32)
    us = graph_time_us(lambda i: K.paged_attention(qkv, kc, vc, bt, cu_q, sl, ts, nh, nkv, hd, hd ** -0.5, None, ctx, ctx,
                                                   torch.bfloat16, decode_index=di, n_decode=0, n_multi=1), 3)
    flops = 4 * nh * hd * (ctx * (ctx + 1) // 2)
    print(f"== prefill attention: {ctx} tokens, causal: {us:8.1f} us  {flops / us / 1e6:7.1f} TFLOP/s", flush=True)


def bench_ffn_fused(args, K, dev, peak) -> None:
    """The feed-forward half of a layer for a decode step: the persistent kernel against the three kernels it
    replaces (add + norm, gate/up with the activation, down), each layer on weights of its own."""
    H, I = args.hidden, args.inter
    n_rot = max(3, int(300e6 // (3 * I * H * 2)) + 1)
    wgu = [torch.randn(2 * I, H, device=dev, dtype=torch.bfloat16) * H ** -0.5 for _ in range(n_rot)]
    wd = [torch.randn(H, I, device=dev, dtype=torch.bfloat16) * I ** -0.5 for _ in range(n_rot)]
    gm = torch.ones(H, device=dev, dtype=torch.bfloat16)
    print("== feed-forward half, decode: norm + gate/up + silu*up + down  (us | GB/s of both weights | fraction of %.0f GB/s)" % peak)
    for B in args.batch:
        x = torch.randn(B, H, device=dev, dtype=torch.bfloat16)
        res = torch.randn(B, H, device=dev)
        cols = []
        if K.can_stream_ffn(x, gm, wgu[0], wd[0]):
            us = graph_time_us(lambda i: K.stream_ffn(x, res, gm, 1e-6, wgu[i], wd[i]), n_rot)
            gbs = 3 * I * H * 2 / us / 1e3
            cols.append(f"persistent: {us:6.1f} us {gbs:6.0f} GB/s {gbs / peak:4.2f}")

        if K.can_stream_linear(x, wgu[0], None, gm):
            def two(i):
                h, _ = K.stream_linear(x, wgu[i], None, norm=(res, gm, 1e-6), gated=True)
                K.linear(h, wd[i], None, torch.bfloat16)
            us = graph_time_us(two, n_rot)
            gbs = 3 * I * H * 2 / us / 1e3
            cols.append(f"norm inside gate/up, down: {us:6.1f} us {gbs:6.0f} GB/s {gbs / peak:4.2f}")

        def separate(i):
            h, _ = K.add_rmsnorm(x, res, gm, 1e-6, torch.bfloat16)
            K.linear(K.gate_up_silu(h, wgu[i], torch.bfloat16), wd[i], None, torch.bfloat16)
        us = graph_time_us(separate, n_rot)
        gbs = 3 * I * H * 2 / us / 1e3
        cols.append(f"three kernels: {us:6.1f} us {gbs:6.0f} GB/s {gbs / peak:4.2f}")

        def separate_lib(i):
            h, _ = K.add_rmsnorm(x, res, gm, 1e-6, torch.bfloat16)
            torch.mm(K.gate_up_silu(h, wgu[i], torch.bfloat16), wd[i].t())
        us = graph_time_us(separate_lib, n_rot)
        gbs = 3 * I * H * 2 / us / 1e3
        cols.append(f"with the library's down: {us:6.1f} us {gbs:6.0f} GB/s {gbs / peak:4.2f}")
        print(f"ffn half B={B:3d} H={H} I={I} | " + " | ".join(cols), flush=True)


def bench_norm(args, K, dev, peak) -> None:
    H = args.hidden
    print("== add + RMSNorm, rotary + cache write")
    for T in args.batch:
        x = torch.randn(T, H, device=dev, dtype=torch.bfloat16)
        r = torch.randn(T, H, device=dev)
        w = torch.ones(H, device=dev, dtype=torch.bfloat16)
        us = graph_time_us(lambda i: K.add_rmsnorm(x, r, w, 1e-6, torch.bfloat16), 20)
        print(f"add_rmsnorm T={T:3d} H={H}: {us:6.2f} us", flush=True)


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--what", default="all", choices=["all", "gemm", "gemm_prefill", "attn_decode", "attn_prefill", "ffn_fused", "norm"])
    ap.add_argument("--only", default="", help="comma-separated projection names to restrict --what gemm / gemm_prefill to")
    ap.add_argument("--rows", default="2048", help="row counts for --what gemm_prefill")
    ap.add_argument("--batch", default="1,8,64")
    ap.add_argument("--ctx", type=int, default=2048)
    ap.add_argument("--hidden", type=int, default=1536)
    ap.add_argument("--heads", type=int, default=12)
    ap.add_argument("--kv-heads", type=int, default=2)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--inter", type=int, default=8960)
    ap.add_argument("--vocab", type=int, default=151936)
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--splits", default="0", help="parts of K of the few-rows GEMM to try (0 = its own choice)")
    ap.add_argument("--warps", default="0", help="K splits of the skinny GEMM to try (0 = its own choice)")
    ap.add_argument("--no-stream", action="store_true", help="decode attention: the shared-memory kernel instead of the streaming one")
    ap.add_argument("--no-clusters", action="store_true", help="decode attention: merge splits through global memory")
    ap.add_argument("--peak-gbs", type=float, default=6650.0, help="the copy bandwidth the fractions are taken of")
    ap.add_argument("--target-ctas", default="148", help="CTA targets of the decode attention's key split to try")
    ap.add_argument("--max-splits", default="32", help="most splits of a request's keys to try")
    args = ap.parse_args()
    args.batch = [int(b) for b in args.batch.split(",")]
    args.rows = [int(b) for b in args.rows.split(",")]
    args.only = [x for x in args.only.split(",") if x]
    args.warps = [int(b) for b in args.warps.split(",")]
    args.splits = [int(b) for b in args.splits.split(",")]
    args.target_ctas = [int(b) for b in args.target_ctas.split(",")]
    args.max_splits = [int(b) for b in args.max_splits.split(",")]
    dev = torch.device("cuda:0")
    K = ops.kernels()
    K.decode_clusters = not args.no_clusters
    K.decode_stream = not args.no_stream
    peak = args.peak_gbs
    with torch.inference_mode():
        if args.what in ("all", "gemm"):
            bench_gemm(args, K, dev, peak)
        if args.what in ("all", "gemm_prefill"):
            bench_gemm_prefill(args, K, dev, peak)
        if args.what in ("all", "attn_decode"):
            bench_attn_decode(args, K, dev, peak)
        if args.what in ("all", "attn_prefill"):
            bench_attn_prefill(args, K, dev, peak)
        if args.what in ("all", "ffn_fused"):
            bench_ffn_fused(args, K, dev, peak)
        if args.what in ("all", "norm"):
            bench_norm(args, K, dev, peak)


if __name__ == "__main__":
    main()
