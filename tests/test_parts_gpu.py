"""Each part of a layer alone against the plain implementation's function for it, at sizes other
than the tiny models': norm, position encoding, attention mixer (with and without a window),
feed-forward, block, embedding and head."""

import pytest
import torch

from plain import model as pm

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


class Ctx:
    """The slice of a step context the parts read: one request, whole, from an empty cache."""

    def __init__(self, T, dtype, nkv, hd, ps=16, window=None, extra_pages=3):
        from omniserver_b200.engine.step import StepContext
        c = StepContext()
        i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
        pages = -(-T // ps)
        perm = torch.randperm(pages + extra_pages, generator=torch.Generator().manual_seed(T))[:pages]
        c.device, c.act_dtype, c.T, c.S = torch.device(DEV), dtype, T, 1
        c.cu_q, c.seq_lens, c.tok_seq, c.state_slot = i32([0, T]), i32([T]), i32([0] * T), i32([0])
        c.positions = torch.arange(T, dtype=torch.int32, device=DEV).repeat(3, 1).contiguous()
        c.pos_mode = i32([0])
        c.block_tables = [perm.to(torch.int32).view(1, -1).to(DEV)]
        c.slot_maps = [(perm[torch.arange(T) // ps] * ps + torch.arange(T) % ps).to(torch.int32).to(DEV)]
        c.q_lens, c.kv_lens, c.max_q_len, c.max_kv_len, c.page_size = [T], [T], T, T, ps
        c.decode_index, c.n_decode, c.n_multi = i32([-1 if T > 1 else 0]), int(T == 1), int(T > 1)
        c.token_ids = None
        self.ctx = c
        self.k_cache = torch.zeros(pages + extra_pages, nkv, ps, hd, dtype=dtype, device=DEV)
        self.v_cache = torch.zeros_like(self.k_cache)


def rnd(*shape, scale=1.0, seed=0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed + sum(shape))) * scale


def close(got, want, dtype):
    if dtype == torch.float32:
        return torch.allclose(got.float().cpu(), want, rtol=2e-4, atol=2e-5)
    return ((got.float().cpu() - want).norm() / want.norm()).item() < 1.5e-2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm_part(dtype):
    from omniserver_b200.parts import RMSNorm
    n = RMSNorm(200, 1e-5, "x.")
    w = 1 + 0.1 * rnd(200)
    n.bind({"weight": w.to(dtype).to(DEV)})
    x, res = rnd(9, 200, seed=1).to(dtype), rnd(9, 200, seed=2)
    y, r = n.forward_add(x.to(DEV), res.clone().to(DEV), dtype)
    r_want = pm.add_residual(res, x.float())
    assert torch.equal(r.cpu(), r_want)
    assert close(y, pm.rms_norm(r_want, w.to(dtype).float(), 1e-5), dtype)
    y0, r0 = n.forward_add(x.to(DEV), None, dtype)
    assert torch.equal(r0.cpu(), x.float())


def test_mrope_part_tables_match_plain_cos_sin():
    from omniserver_b200.parts import MRope
    T, hd, sec = 40, 48, (10, 7, 7)
    mr = MRope(hd, 5e4, sec)
    c = Ctx(T, torch.float32, 1, hd).ctx
    pos, _ = pm.image_span_positions(T, 5, 1, 4, 6)
    c.positions = pos.to(torch.int32).to(DEV).contiguous()
    tables = mr.prepare(c, {"rope_cursor": torch.zeros(4, 2, dtype=torch.int32, device=DEV)})
    cos, sin = pm.mrope_cos_sin(pos, 5e4, hd, sec)
    assert torch.allclose(tables.cos.cpu(), cos[:, :hd // 2], atol=3e-7) and torch.allclose(tables.sin.cpu(), sin[:, :hd // 2], atol=3e-7)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,window", [(6, 3, 48, None), (5, 1, 64, 24), (8, 8, 32, None)])
def test_attention_mixer_part(dtype, nh, nkv, hd, window):
    from omniserver_b200.parts import GQAAttention, MRope
    from omniserver_b200.parts.base import CacheBinding
    Hs, T = 72, 75
    sec = (hd // 2 - 2 * (hd // 6), hd // 6, hd // 6)
    mr = MRope(hd, 1e4, sec)
    att = GQAAttention(Hs, nh, nkv, hd, "a.", position=mr, window=window)
    wq, wk, wv = rnd(nh * hd, Hs, scale=0.1, seed=1), rnd(nkv * hd, Hs, scale=0.1, seed=2), rnd(nkv * hd, Hs, scale=0.1, seed=3)
    bq, bk, bv = rnd(nh * hd, seed=4), rnd(nkv * hd, seed=5), rnd(nkv * hd, seed=6)
    wo = rnd(Hs, nh * hd, scale=0.1, seed=7)
    cast = lambda t: t.to(dtype).to(DEV)
    att.bind({"qkv_weight": cast(torch.cat([wq, wk, wv])), "qkv_bias": cast(torch.cat([bq, bk, bv])), "o_weight": cast(wo)})
    cc = Ctx(T, dtype, nkv, hd)
    ctx = cc.ctx
    from omniserver_b200.models import DecoderModel  # noqa: F401  (context needs a model only for shared state)

    class M:
        shared_state = {"rope_cursor": torch.zeros(4, 2, dtype=torch.int32, device=DEV)}
    ctx.bind_model(M())
    x = rnd(T, Hs, seed=8).to(dtype)
    y = att.forward(ctx, x.to(DEV), CacheBinding(group=0, k_cache=cc.k_cache, v_cache=cc.v_cache, writes=True))
    f = lambda t: t.to(dtype).float()
    q, k, v = pm.qkv_proj(f(x), f(wq), f(bq), f(wk), f(bk), f(wv), f(bv), nh, nkv, hd)
    cos, sin = pm.mrope_cos_sin(pm.text_positions(T), 1e4, hd, sec)
    want = pm.o_proj(pm.attention(pm.apply_rotary(q, cos, sin), pm.apply_rotary(k, cos, sin), v, window), f(wo))
    assert close(y, want, dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T", [3, 100])
def test_swiglu_part(dtype, T):
    from omniserver_b200.parts import SwiGLU
    Hs, I = 72, 200
    ff = SwiGLU(Hs, I, "m.")
    wg, wu, wd = rnd(I, Hs, scale=0.2, seed=1), rnd(I, Hs, scale=0.2, seed=2), rnd(Hs, I, scale=0.2, seed=3)
    cast = lambda t: t.to(dtype).to(DEV)
    ff.bind({"gate_up_weight": cast(torch.cat([wg, wu])), "down_weight": cast(wd)})
    x = rnd(T, Hs, seed=4).to(dtype)
    y = ff.forward(Ctx(T, dtype, 1, 16).ctx, x.to(DEV))
    f = lambda t: t.to(dtype).float()
    assert close(y, pm.swiglu(f(x), f(wg), f(wu), f(wd)), dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding_and_head_parts(dtype):
    from omniserver_b200.parts import LMHead, TokenEmbedding
    Vv, Hs, T = 1000, 72, 11
    emb = TokenEmbedding(Vv, Hs)
    table = rnd(Vv, Hs, seed=1)
    emb.bind({"weight": table.to(dtype).to(DEV)})
    ctx = Ctx(T, dtype, 1, 16).ctx
    ids = torch.randint(0, Vv, (T,), generator=torch.Generator().manual_seed(3))
    ctx.token_ids = ids.to(torch.int32).to(DEV)
    ctx.override_rows = torch.tensor([2, 7], dtype=torch.int32, device=DEV)
    ov = rnd(2, Hs, seed=5)
    ctx.override_vals = ov.to(DEV)
    x = emb.forward(ctx)
    want = pm.embed(ids, table.to(dtype).float(), torch.tensor([2, 7]), ov)
    assert close(x, want.to(dtype).float(), dtype)
    for tied in (True, False):
        head = LMHead(Vv, Hs, tied_to=emb if tied else None)
        w2 = rnd(Vv, Hs, seed=9)
        if not tied:
            head.bind({"weight": w2.to(dtype).to(DEV)})
        h = rnd(4, Hs, seed=6).to(dtype)
        lg = head.forward(h.to(DEV))
        assert lg.dtype == torch.float32
        assert close(lg, pm.lm_head(h.float(), (table if tied else w2).to(dtype).float()), dtype)
