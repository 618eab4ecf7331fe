"""Plain references of the CUDA kernels, one function per kernel, in torch on any device.

Used two ways by the tests: each CUDA kernel is compared with its function here at several sizes,
and, with ``install()``, the engine's host logic (step function, cache manager, scheduler) can be
exercised on a machine without a GPU.  It is test code: the product has no CPU path.  Everything
is computed in float32 (or the dtype given) from the formulas cited in tests/plain/model.py.
"""

from __future__ import annotations

import contextlib
from typing import Optional, Tuple

import torch


class PlainKernels:
    SKINNY_MAX_ROWS = 0
    launches = 0

    fuse_norm_linear_decode = False

    def can_stream_linear(self, x, w, bias, norm_weight=None):
        return False

    def can_stream_ffn(self, x, norm_weight, w_gate_up, w_down):
        return False

    @contextlib.contextmanager
    def pinned_stream(self):
        yield

    def check_device_errors_async(self) -> None:
        pass

    def check_device_errors(self) -> None:
        pass

    # -- embedding
    def embed_lookup(self, table, ids, out_dtype, src_slots=None, last_token=None):
        ids = ids.long()
        if src_slots is not None:
            from_slot = src_slots >= 0
            ids = torch.where(from_slot, last_token[src_slots.clamp(min=0).long()].long(), ids)
        return table[ids].to(out_dtype)

    def scatter_rows(self, x, rows, vals):
        x[rows.long()] = vals.to(x.dtype)

    # -- norm
    def add_rmsnorm(self, x, residual, weight, eps, out_dtype):
        r = x.float() if residual is None else residual + x.float()
        if residual is not None:
            residual.copy_(r)
            r = residual
        rstd = 1.0 / torch.sqrt((r * r).sum(-1, keepdim=True) / r.shape[-1] + eps)
        return (r * rstd * weight.float()).to(out_dtype), r

    def add_rmsnorm_rows(self, x, residual, weight, eps, rows, out_dtype):
        r = x.float()[rows.long()]
        if residual is not None:
            r = residual[rows.long()] + r
        rstd = 1.0 / torch.sqrt((r * r).sum(-1, keepdim=True) / r.shape[-1] + eps)
        return (r * rstd * weight.float()).to(out_dtype)

    # -- matrix product
    def linear(self, x, w, bias, out_dtype):
        acc = torch.float64 if x.dtype == torch.float64 else torch.float32
        y = x.to(acc) @ w.to(acc).T
        if bias is not None:
            y = y + bias.to(acc)
        return y.to(out_dtype)

    gemm_simt = linear

    def gate_up_silu(self, x, w, out_dtype):
        mid = x.dtype if x.dtype == w.dtype else torch.float32
        return self.silu_mul(self.linear(x, w, None, mid), out_dtype)

    # -- rotary
    def rope_tables(self, positions, pos_mode, tok_seq, cu_q, state_slot, cursor, inv_freq, axis_of):
        T = tok_seq.shape[0]
        s = tok_seq.long()
        off = torch.arange(T, device=tok_seq.device) - cu_q.long()[s]
        slot = state_slot.long()[s]
        from_state = cursor[slot, 0].long() + cursor[slot, 1].long() + off          # [T]
        explicit = positions.long()[axis_of.long()]                                  # [half, T]
        use_state = (pos_mode.long()[s] == 1)[None, :]
        p = torch.where(use_state, from_state[None, :].expand_as(explicit), explicit)  # [half, T]
        ang = p.T.float() * inv_freq[None, :]
        return ang.cos(), ang.sin()

    def advance_cursor(self, cursor, state_slot, cu_q):
        q = (cu_q[1:] - cu_q[:-1]).to(cursor.dtype)
        cursor[state_slot.long(), 0] += q

    def rope_kv_write(self, qkv, cos, sin, k_cache, v_cache, slot_map, nh, nkv, hd, rot):
        T = qkv.shape[0]
        x = qkv.view(T, nh + 2 * nkv, hd)
        qk = x[:, :nh + nkv, :].float()
        if rot > 0:
            half = rot // 2
            x1, x2 = qk[..., :half], qk[..., half:rot]
            c, s = cos[:, None, :], sin[:, None, :]
            qk = torch.cat([x1 * c - x2 * s, x2 * c + x1 * s, qk[..., rot:]], dim=-1)
        x[:, :nh, :] = qk[:, :nh].to(qkv.dtype)
        if slot_map is None:
            return
        ps = k_cache.shape[2]
        page, off = slot_map.long() // ps, slot_map.long() % ps
        k_cache[page, :, off, :] = qk[:, nh:].to(k_cache.dtype)
        v_cache[page, :, off, :] = x[:, nh + nkv:, :].to(v_cache.dtype)

    @staticmethod
    def can_fuse_rope_decode(*args, **kw):
        return False

    # -- attention
    def paged_attention(self, qkv, k_cache, v_cache, block_table, cu_q, seq_lens, tok_seq, nh, nkv, hd, scale,
                        window, max_q_len, max_kv_len, out_dtype, decode_index=None, n_decode=0, n_multi=0, exact=False,
                        scratch=None, rope=None, order=None, uneven=False, units=None):
        T = qkv.shape[0]
        ps = k_cache.shape[2]
        g = nh // nkv
        q = qkv[:, :nh * hd].view(T, nh, hd).float()
        out = torch.zeros(T, nh, hd, dtype=torch.float32, device=qkv.device)
        for s in range(seq_lens.shape[0]):
            a, b = int(cu_q[s]), int(cu_q[s + 1])
            kv_len = int(seq_lens[s])
            n = b - a
            if n == 0:
                continue
            lo_all = 0
            first_q = kv_len - n
            if window:
                lo_all = max(0, first_q - window + 1)
            idx = torch.arange(lo_all, kv_len, device=qkv.device)
            pages = block_table[s].long()[idx // ps]
            assert (pages >= 0).all(), "attention reaches a page that was given back"
            K = k_cache[pages, :, idx % ps, :].float()       # [n_keys, nkv, hd]
            Vv = v_cache[pages, :, idx % ps, :].float()
            qpos = first_q + torch.arange(n, device=qkv.device)
            allowed = idx[None, :] <= qpos[:, None]
            if window:
                allowed &= idx[None, :] > (qpos[:, None] - window)
            for h in range(nh):
                sc = (q[a:b, h, :] @ K[:, h // g, :].T) * scale
                sc = sc.masked_fill(~allowed, float("-inf"))
                out[a:b, h, :] = torch.softmax(sc, dim=-1) @ Vv[:, h // g, :]
        return out.reshape(T, nh * hd).to(out_dtype)

    # -- activation
    def silu_mul(self, gu, out_dtype):
        n = gu.shape[1] // 2
        acc = torch.float64 if gu.dtype == torch.float64 else torch.float32
        g, u = gu[:, :n].to(acc), gu[:, n:].to(acc)
        return ((g * torch.sigmoid(g)) * u).to(out_dtype)

    # -- sampling
    def sample(self, logits, temperature, uniform, keep=None, keep_at=None):
        out = self._sample(logits, temperature, uniform)
        if keep is not None:
            keep[keep_at.long()] = out
        return out

    def _sample(self, logits, temperature, uniform):
        R = logits.shape[0]
        out = torch.empty(R, dtype=torch.int32, device=logits.device)
        for r in range(R):
            row = logits[r]
            t = float(temperature[r]) if temperature is not None else 0.0
            if t <= 0:
                m = row.max()
                out[r] = int((row == m).nonzero()[0])
            else:
                p = torch.exp((row - row.max()) / t).double()
                cdf = torch.cumsum(p, 0)
                target = float(uniform[r]) * float(cdf[-1])
                i = int(torch.searchsorted(cdf, torch.tensor(target, dtype=cdf.dtype), right=True))
                out[r] = min(i, row.numel() - 1)
        return out


def install():
    """Routes the engine's kernel calls to the plain references (tests without a GPU)."""
    from omniserver_b200 import ops
    k = PlainKernels()
    ops._KERNELS = k
    return k


def uninstall():
    from omniserver_b200 import ops
    ops._KERNELS = None
