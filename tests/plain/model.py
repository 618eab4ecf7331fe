"""Plain, slow implementation of the Qwen2 text decoder of Qwen2-VL.

Whole sequences, no cache, no batching: one request at a time, one function
per part, CPU tensors in one dtype (float32 by default, float64 for a tighter
oracle).  It shares no code with ``omniserver_b200``; it is written from the
reference's formulas and each function cites the file and lines it restates
(paths are relative to the reference project's root).

Where the reference rounds to half precision (residual add, cos/sin) this
implementation does not: those roundings are properties of its fp16 storage,
not of the architecture (omniserve/kernels/fused_ops.py:43-57 rounds the new
residual to the tensor's dtype, which in one dtype is the identity).

The window is not in the reference (it has no sliding window at all); its
meaning here is: a query at position p sees keys p-window+1 .. p.
"""

from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence, Tuple

import torch


# --------------------------------------------------------------------------- config
class PlainConfig:
    """The numbers the formulas need, read from a config.json dictionary."""

    def __init__(self, d: dict):
        t = d.get("text_config", {}) if isinstance(d.get("text_config"), dict) else {}
        g = lambda k, default=None: t.get(k, d.get(k, default))  # noqa: E731
        self.H = g("hidden_size")
        self.L = g("num_hidden_layers")
        self.nh = g("num_attention_heads")
        self.nkv = g("num_key_value_heads")
        self.hd = g("head_dim") or self.H // self.nh
        self.I = g("intermediate_size")
        self.V = g("vocab_size")
        self.eps = float(g("rms_norm_eps"))
        self.theta = float(g("rope_theta"))
        rs = g("rope_scaling") or {}
        self.section = list(rs.get("mrope_section", [self.hd // 2, 0, 0]))
        self.tied = bool(g("tie_word_embeddings", False))
        self.use_window = bool(g("use_sliding_window", False))
        self.window = g("sliding_window")
        self.first_window_layer = g("max_window_layers") or 0

    def window_of(self, layer: int) -> Optional[int]:
        if self.use_window and self.window is not None and layer >= self.first_window_layer:
            return int(self.window)
        return None

    @classmethod
    def from_dir(cls, model_dir: str) -> "PlainConfig":
        with open(os.path.join(model_dir, "config.json")) as f:
            return cls(json.load(f))


# --------------------------------------------------------------------------- parts
def embed(ids: torch.Tensor, table: torch.Tensor,
          override_rows: Optional[torch.Tensor] = None,
          override_vals: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Token lookup; rows flagged as vision tokens are overwritten by given embeddings.

    omniserve/model/qwen2_llm.py:164 (lookup), omniserve/runners/multimodal.py:123-126 (overwrite).
    """
    x = table[ids.long()].clone()
    if override_rows is not None and len(override_rows):
        x[override_rows.long()] = override_vals.to(x.dtype)
    return x


def rms_norm(r: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """y = r * (1/sqrt(mean(r^2) + eps)) * w.  omniserve/kernels/fused_ops.py:21-29."""
    rstd = 1.0 / torch.sqrt((r * r).sum(dim=-1, keepdim=True) / r.shape[-1] + eps)
    return r * rstd * w


def add_residual(res: Optional[torch.Tensor], x: torch.Tensor) -> torch.Tensor:
    """The residual stream: first layer res = x, later res = res + x.

    omniserve/model/qwen2_llm.py:145-151, omniserve/kernels/fused_ops.py:43-49.
    """
    return x.clone() if res is None else res + x


def qkv_proj(y: torch.Tensor, wq, bq, wk, bk, wv, bv, nh: int, nkv: int, hd: int):
    """q/k/v = y W^T + b, all three biased; heads are contiguous bands of the row.

    omniserve/model/qwen2_llm.py:78-92 and 207-212 (concatenation order q,k,v).
    """
    T = y.shape[0]
    q = (y @ wq.T + bq).view(T, nh, hd)
    k = (y @ wk.T + bk).view(T, nkv, hd)
    v = (y @ wv.T + bv).view(T, nkv, hd)
    return q, k, v


def inv_freq(theta: float, hd: int, dtype=torch.float32) -> torch.Tensor:
    """inv_freq[j] = theta^(-2j/hd), computed in float32.  omniserve/model/qwen2_llm.py:169."""
    f = 1.0 / (theta ** (torch.arange(0, hd, 2).float() / hd))
    return f.to(dtype)


def mrope_cos_sin(pos: torch.Tensor, theta: float, hd: int, section: Sequence[int],
                  dtype=torch.float32) -> Tuple[torch.Tensor, torch.Tensor]:
    """cos/sin tables [T, hd] for 3-axis positions ``pos`` [3, T].

    Angles: omniserve/model/qwen2_llm.py:172-177 (pos * inv_freq, duplicated to hd).
    Axis choice per frequency band: omniserve/model/qwen2_llm.py:64-69 (the section list
    doubled; band i is driven by axis i mod 3).
    """
    inv = inv_freq(theta, hd, dtype)
    freqs = pos.to(dtype)[..., None] * inv                  # [3, T, hd/2]
    emb = torch.cat([freqs, freqs], dim=-1)                 # [3, T, hd]
    cos, sin = emb.cos(), emb.sin()
    sec = list(section) * 2
    cos = torch.cat([m[i % 3] for i, m in enumerate(cos.split(sec, dim=-1))], dim=-1)
    sin = torch.cat([m[i % 3] for i, m in enumerate(sin.split(sec, dim=-1))], dim=-1)
    return cos, sin                                          # [T, hd]


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    """omniserve/model/qwen2_llm.py:59-61."""
    h = x.shape[-1] // 2
    return torch.cat((-x[..., h:], x[..., :h]), dim=-1)


def apply_rotary(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x [T, heads, hd] -> x*cos + rotate_half(x)*sin.  omniserve/model/qwen2_llm.py:70-72."""
    return x * cos[:, None, :] + rotate_half(x) * sin[:, None, :]


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
              window: Optional[int] = None) -> torch.Tensor:
    """Causal GQA attention of one whole sequence; q [T,nh,hd], k/v [T,nkv,hd] -> [T, nh*hd].

    scale hd^-1/2 (omniserve/model/qwen2_llm.py:98,103); q head h reads kv head h // (nh/nkv)
    (repeat_interleave, omniserve/model/qwen2_llm.py:108-110); causal within the sequence
    (omniserve/cache/kv_prealloc.py:138-142).  ``window``: keys p-window+1..p (not in the reference).
    """
    T, nh, hd = q.shape
    nkv = k.shape[1]
    g = nh // nkv
    scale = hd ** -0.5
    out = torch.empty(T, nh, hd, dtype=q.dtype)
    idx = torch.arange(T)
    allowed = idx[None, :] <= idx[:, None]
    if window is not None:
        allowed &= idx[None, :] > (idx[:, None] - window)
    for h in range(nh):
        kh = k[:, h // g, :]
        vh = v[:, h // g, :]
        s = (q[:, h, :] @ kh.T) * scale
        s = s.masked_fill(~allowed, float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[:, h, :] = p @ vh
    return out.reshape(T, nh * hd)


def o_proj(a: torch.Tensor, wo: torch.Tensor) -> torch.Tensor:
    """No bias.  omniserve/model/qwen2_llm.py:83."""
    return a @ wo.T


def swiglu(y: torch.Tensor, wg: torch.Tensor, wu: torch.Tensor, wd: torch.Tensor) -> torch.Tensor:
    """down( silu(gate(y)) * up(y) ), no biases.  omniserve/model/qwen2_llm.py:116-134,
    omniserve/kernels/fused_ops.py:111-119 (silu(z) = z * sigmoid(z))."""
    gte = y @ wg.T
    up = y @ wu.T
    return ((gte * torch.sigmoid(gte)) * up) @ wd.T


def lm_head(h: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """logits = h W^T, no bias; W is the embedding table when tied.  omniserve/model/qwen2_llm.py:167-168,190."""
    return h @ w.T


# --------------------------------------------------------------------------- positions
def text_positions(n: int, start: int = 0) -> torch.Tensor:
    """Text-only prompt: the token index on all three axes.  omniserve/models/qwen2_vl.py:100-104."""
    return (torch.arange(n) + start).view(1, -1).expand(3, -1).contiguous()


def image_span_positions(L: int, span_start: int, grid_t: int, grid_h: int, grid_w: int
                         ) -> Tuple[torch.Tensor, int]:
    """Positions [3, L] of a prompt with one image span of grid_t*grid_h*grid_w tokens at span_start.

    omniserve/model/positions.py:17-58: text counts up on all axes; the span gets
    (t, h, w) grid indices offset by the text length before it; text after resumes at max+1;
    rope_delta = max + 1 - L.  (grid_h, grid_w are the merged grid sizes.)
    """
    pieces = [torch.arange(span_start).view(1, -1).expand(3, -1)]
    ti = torch.arange(grid_t).view(-1, 1).expand(-1, grid_h * grid_w).flatten()
    hi = torch.arange(grid_h).view(1, -1, 1).expand(grid_t, -1, grid_w).flatten()
    wi = torch.arange(grid_w).view(1, 1, -1).expand(grid_t, grid_h, -1).flatten()
    pieces.append(torch.stack([ti, hi, wi]) + span_start)
    n_img = grid_t * grid_h * grid_w
    rest = L - span_start - n_img
    if rest > 0:
        st = int(torch.cat(pieces, dim=1).max()) + 1
        pieces.append(torch.arange(rest).view(1, -1).expand(3, -1) + st)
    pos = torch.cat(pieces, dim=1).long()
    return pos, int(pos.max()) + 1 - L


def decode_position(index: int, rope_delta: int) -> torch.Tensor:
    """A generated token at cache index c sits at c + rope_delta on all axes.  omniserve/models/qwen2_vl.py:108-112."""
    return torch.full((3, 1), index + rope_delta, dtype=torch.long)


def extend_positions(prompt_pos: torch.Tensor, rope_delta: int, total: int) -> torch.Tensor:
    """Positions of prompt + generated tokens up to ``total`` tokens."""
    L = prompt_pos.shape[1]
    if total <= L:
        return prompt_pos[:, :total]
    tail = (torch.arange(L, total) + rope_delta).view(1, -1).expand(3, -1)
    return torch.cat([prompt_pos, tail], dim=1)


# --------------------------------------------------------------------------- sampling
def greedy(logits_row: torch.Tensor) -> int:
    """argmax; ties go to the lowest index.  omniserve/runners/multimodal.py:376-377."""
    m = logits_row.max()
    return int((logits_row == m).nonzero()[0])


def temperature_cdf(logits_row: torch.Tensor, temperature: float) -> torch.Tensor:
    """Cumulative distribution of softmax(logits / T) in float64.  omniserve/runners/multimodal.py:378."""
    p = torch.softmax(logits_row.double() / temperature, dim=-1)
    return torch.cumsum(p, dim=-1)


def sample_inverse_cdf(logits_row: torch.Tensor, temperature: float, u: float) -> int:
    """The smallest index whose cumulative probability reaches u (u uniform in [0,1)).

    The reference draws with torch.multinomial from an unseeded generator
    (omniserve/runners/multimodal.py:379); a given uniform makes the draw repeatable.
    """
    cdf = temperature_cdf(logits_row, temperature)
    i = int(torch.searchsorted(cdf, torch.tensor(u, dtype=cdf.dtype), right=False))
    return min(i, logits_row.numel() - 1)


# --------------------------------------------------------------------------- weights
def load_weights(model_dir: str, dtype=torch.float32) -> Dict[str, torch.Tensor]:
    """All tensors of model*.safetensors as ``dtype`` CPU tensors, prefix stripped.

    omniserve/models/qwen2_vl.py:42-44 (files), omniserve/model/qwen2_llm.py:196-199 (prefix).
    """
    from safetensors import safe_open
    sd: Dict[str, torch.Tensor] = {}
    for fn in sorted(os.listdir(model_dir)):
        if fn.startswith("model") and fn.endswith(".safetensors"):
            with safe_open(os.path.join(model_dir, fn), framework="pt") as f:
                for k in f.keys():
                    sd[k] = f.get_tensor(k)
    pfx = "model.language_model." if "model.language_model.embed_tokens.weight" in sd else "model."
    out = {}
    for k, v in sd.items():
        name = k[len(pfx):] if k.startswith(pfx) else k
        out[name] = v.to(dtype) if v.is_floating_point() else v
    return out


# --------------------------------------------------------------------------- whole model
def forward(cfg: PlainConfig, w: Dict[str, torch.Tensor], ids: torch.Tensor,
            pos: Optional[torch.Tensor] = None,
            override_rows: Optional[torch.Tensor] = None,
            override_vals: Optional[torch.Tensor] = None,
            return_hidden: bool = False, rows: Optional[Sequence[int]] = None):
    """Logits [T, V] of one whole sequence (of the given rows only when ``rows`` is set, as the
    reference's logits_indices, omniserve/model/qwen2_llm.py:187-189).
    Layer order: omniserve/model/qwen2_llm.py:145-157,179-190."""
    T = ids.shape[0]
    dtype = w["embed_tokens.weight"].dtype
    if pos is None:
        pos = text_positions(T)
    x = embed(ids, w["embed_tokens.weight"], override_rows, override_vals)
    cos, sin = mrope_cos_sin(pos, cfg.theta, cfg.hd, cfg.section, dtype)
    res = None
    for i in range(cfg.L):
        p = f"layers.{i}."
        res = add_residual(res, x)
        y = rms_norm(res, w[p + "input_layernorm.weight"], cfg.eps)
        q, k, v = qkv_proj(y, w[p + "self_attn.q_proj.weight"], w[p + "self_attn.q_proj.bias"],
                           w[p + "self_attn.k_proj.weight"], w[p + "self_attn.k_proj.bias"],
                           w[p + "self_attn.v_proj.weight"], w[p + "self_attn.v_proj.bias"],
                           cfg.nh, cfg.nkv, cfg.hd)
        q = apply_rotary(q, cos, sin)
        k = apply_rotary(k, cos, sin)
        a = attention(q, k, v, cfg.window_of(i))
        x = o_proj(a, w[p + "self_attn.o_proj.weight"])
        res = add_residual(res, x)
        y = rms_norm(res, w[p + "post_attention_layernorm.weight"], cfg.eps)
        x = swiglu(y, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
    res = add_residual(res, x)
    h = rms_norm(res, w["norm.weight"], cfg.eps)
    head = w["embed_tokens.weight"] if cfg.tied else w["lm_head.weight"]
    hs = h if rows is None else h[torch.as_tensor(list(rows), dtype=torch.long)]
    logits = lm_head(hs, head)
    return (logits, h) if return_hidden else logits


def generate(cfg: PlainConfig, w: Dict[str, torch.Tensor], prompt: Sequence[int], max_new_tokens: int,
             prompt_pos: Optional[torch.Tensor] = None, rope_delta: int = 0,
             override_rows=None, override_vals=None,
             temperature: float = 0.0, uniforms: Optional[Sequence[float]] = None,
             stop_token_ids: Sequence[int] = ()) -> List[int]:
    """Generation by re-running the whole sequence for every new token (no cache).

    Stop rules: omniserve/request.py:103-111 (a stop id ends it, the stop token is kept;
    max_new_tokens counts the first token).
    """
    toks = list(prompt)
    out: List[int] = []
    if prompt_pos is None:
        prompt_pos = text_positions(len(prompt))
    for step in range(max_new_tokens):
        pos = extend_positions(prompt_pos, rope_delta, len(toks))
        logits = forward(cfg, w, torch.tensor(toks), pos, override_rows, override_vals)[-1]
        if temperature == 0.0:
            t = greedy(logits)
        else:
            t = sample_inverse_cdf(logits, temperature, uniforms[step])
        out.append(t)
        toks.append(t)
        if t in stop_token_ids:
            break
    return out
