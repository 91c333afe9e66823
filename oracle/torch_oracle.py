"""Restatement of the reference's torch-eager path (its ``backend="torch"`` branch).

Each function names the reference lines it follows. Everything runs on CPU tensors with
plain torch ops, so the rounding sequence is the one the reference's torch path has.
"""
from __future__ import annotations

import math
from typing import Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

__all__ = [
    "kv_paged_append", "kv_paged_scatter", "kv_paged_lookup", "kv_paged_lookup_as_written",
    "build_rope_tables", "apply_rope", "online_softmax", "attention", "naive_attention_f64",
    "paged_attention_composed", "bottom_right_mask", "merge_partials", "fused_linear_norm",
    "kv_quantize_rows", "kv_paged_append_q8", "kv_dequantize",
]


# ---- kv_cache -------------------------------------------------------------------------

def kv_paged_append(k_in, v_in, k_cache, v_cache, slot_mapping) -> None:
    """``cache[slot // bs, :, slot % bs, :] = in`` for K and V, in place.

    Follows torch_reference_kv_paged_append, kernels/kv_cache/triton_kv_paged.py:279-292
    (floor division and Python-style modulo on the int64 slots, one advanced-index store).
    """
    block_size = k_cache.shape[2]
    page = torch.div(slot_mapping, block_size, rounding_mode="floor")
    pos = torch.remainder(slot_mapping, block_size)
    k_cache[page, :, pos, :] = k_in
    v_cache[page, :, pos, :] = v_in


def kv_paged_scatter(k_updates, v_updates, k_cache, v_cache, slot_mapping) -> None:
    """Same operation as append: kernels/kv_cache/__init__.py:74-90, triton_kv_paged.py:263-276."""
    kv_paged_append(k_updates, v_updates, k_cache, v_cache, slot_mapping)


def kv_paged_lookup(k_cache, v_cache, block_table, context_lens, max_ctx: int):
    """Dense gather with zero tail, vectorised: out[b,h,t] = cache[bt[b,t//bs], h, t%bs].

    Same result as torch_reference_kv_paged_lookup, kernels/kv_cache/triton_kv_paged.py:295-317
    (checked against the per-token form below in the tests), without its Python loop.
    """
    B = context_lens.shape[0]
    _, H, bs, D = k_cache.shape
    k_out = torch.zeros((B, H, max_ctx, D), dtype=k_cache.dtype)
    v_out = torch.zeros_like(k_out)
    if max_ctx == 0 or B == 0:
        return k_out, v_out
    t = torch.arange(max_ctx)
    valid = t[None, :] < context_lens.to(torch.int64)[:, None]            # [B, max_ctx]
    blk_idx = torch.clamp(t // bs, max=max(block_table.shape[1] - 1, 0))  # logical block per t
    pages = block_table.to(torch.int64)[:, blk_idx]                       # [B, max_ctx]
    pages = torch.where(valid, pages, torch.zeros_like(pages))            # any in-range page for the tail
    pos = (t % bs)[None, :].expand(B, -1)
    k_g = k_cache[pages, :, pos, :]                                       # [B, max_ctx, H, D]
    v_g = v_cache[pages, :, pos, :]
    mask = valid[:, :, None, None]
    k_out.copy_(torch.where(mask, k_g, torch.zeros_like(k_g)).permute(0, 2, 1, 3))
    v_out.copy_(torch.where(mask, v_g, torch.zeros_like(v_g)).permute(0, 2, 1, 3))
    return k_out, v_out


def kv_paged_lookup_as_written(k_cache, v_cache, block_table, context_lens, max_ctx: int):
    """The per-token form the reference's torch path runs (triton_kv_paged.py:305-317):
    zero-filled outputs, then one row copy per (request, token) with host reads of the
    length and the page number. Kept for timing the reference's CPU path as it is."""
    B = context_lens.shape[0]
    _, H, bs, D = k_cache.shape
    k_out = torch.zeros((B, H, max_ctx, D), dtype=k_cache.dtype)
    v_out = torch.zeros_like(k_out)
    for b in range(B):
        n = int(context_lens[b].item())
        for t in range(n):
            page = int(block_table[b, t // bs].item())
            k_out[b, :, t, :] = k_cache[page, :, t % bs, :]
            v_out[b, :, t, :] = v_cache[page, :, t % bs, :]
    return k_out, v_out


# ---- rope -----------------------------------------------------------------------------

def build_rope_tables(seq_len: int, head_dim: int, *, base: float = 10000.0,
                      dtype: torch.dtype = torch.float32, interleaved: bool = False):
    """cos/sin tables [seq_len, head_dim]; kernels/rope/triton_rope.py:247-285:
    theta = 1/base**(arange(half)/half) fp32 (:267), outer(positions, theta) (:269),
    cos/sin (:270-271), duplicate to width D (:273-280), cast (:285)."""
    if head_dim % 2:
        raise ValueError("head_dim must be even for RoPE")
    half = head_dim // 2
    theta = 1.0 / (base ** (torch.arange(0, half, dtype=torch.float32) / half))
    ang = torch.outer(torch.arange(seq_len, dtype=torch.float32), theta)
    c, s = torch.cos(ang), torch.sin(ang)
    if interleaved:
        c, s = c.repeat_interleave(2, dim=-1), s.repeat_interleave(2, dim=-1)
    else:
        c, s = torch.cat((c, c), dim=-1), torch.cat((s, s), dim=-1)
    return c.to(dtype), s.to(dtype)


def apply_rope(x, cos, sin, *, interleaved: bool = False, layout: str = "bshd"):
    """torch_reference_rope, kernels/rope/triton_rope.py:199-244. Eager ops in x's dtype:
    each product and each sum is rounded separately, which is what makes 16-bit results
    differ from a fused fp32 evaluation."""
    if layout not in ("bshd", "bhsd"):
        raise ValueError(f"unknown layout {layout!r}; want 'bshd' or 'bhsd'")
    if layout == "bhsd":
        x = x.transpose(1, 2)
    _, S, _, D = x.shape
    c, s = cos.view(1, S, 1, D), sin.view(1, S, 1, D)
    if interleaved:
        a, b = x[..., 0::2], x[..., 1::2]
        ce, se = c[..., 0::2], s[..., 0::2]
        y = torch.stack((a * ce - b * se, a * se + b * ce), dim=-1).flatten(-2)
    else:
        h = D // 2
        a, b = x[..., :h], x[..., h:]
        c1, s1 = c[..., :h], s[..., :h]
        y = torch.cat((a * c1 - b * s1, a * s1 + b * c1), dim=-1)
    if layout == "bhsd":
        y = y.transpose(1, 2).contiguous()
    return y


# ---- softmax --------------------------------------------------------------------------

def online_softmax(x, *, is_causal: bool = False, log: bool = False):
    """torch_reference_softmax, kernels/softmax/triton_softmax.py:178-202: optional square
    causal mask (-inf above the diagonal, added to x), then F.softmax / F.log_softmax."""
    if is_causal:
        if x.dim() < 2 or x.shape[-2] != x.shape[-1]:
            raise ValueError(f"causal mode requires square input (last two dims equal); got {tuple(x.shape)}.")
        n = x.shape[-1]
        x = x + torch.triu(torch.full((n, n), float("-inf"), dtype=x.dtype), diagonal=1)
    return F.log_softmax(x, dim=-1) if log else F.softmax(x, dim=-1)


# ---- attention ------------------------------------------------------------------------

def attention(q, k, v, *, is_causal: bool = False, attn_mask=None, sm_scale: Optional[float] = None):
    """torch_reference_attention, kernels/attention/triton_fused_attention.py:350-371
    (one SDPA call), preceded by the GQA expansion the reference's tests apply because
    that call has no GQA (tests/test_attention_parity.py:72-76):
    query head h reads kv head h // (H/H_kv) (triton_fused_attention.py:130-132)."""
    H, Hkv = q.shape[1], k.shape[1]
    if H != Hkv:
        if H % Hkv:
            raise ValueError(f"GQA requires num_heads_q ({H}) divisible by num_heads_kv ({Hkv})")
        k = k.repeat_interleave(H // Hkv, dim=1)
        v = v.repeat_interleave(H // Hkv, dim=1)
    return F.scaled_dot_product_attention(q, k, v, attn_mask=attn_mask, is_causal=is_causal, scale=sm_scale)


def naive_attention_f64(q, k, v, *, sm_scale: Optional[float] = None, mask=None):
    """softmax(q k^T * scale + mask) v in float64 with GQA expansion: the independent
    known-answer form named by the first benchmark configuration."""
    q, k, v = q.double(), k.double(), v.double()
    H, Hkv = q.shape[1], k.shape[1]
    if H != Hkv:
        k = k.repeat_interleave(H // Hkv, dim=1)
        v = v.repeat_interleave(H // Hkv, dim=1)
    scale = 1.0 / math.sqrt(q.shape[-1]) if sm_scale is None else sm_scale
    s = torch.matmul(q, k.transpose(-1, -2)) * scale
    if mask is not None:
        s = s + mask.double()
    return torch.matmul(torch.softmax(s, dim=-1), v)


def bottom_right_mask(n_q: int, n_k: int, dtype=torch.float32):
    """Additive [n_q, n_k] mask where query row i sees keys 0..n_k-n_q+i: the chunked-
    prefill rule of src/kernels/attention.cu:187 (seq_len = start_pos + token + 1)."""
    i = torch.arange(n_q)[:, None]
    j = torch.arange(n_k)[None, :]
    m = torch.zeros((n_q, n_k), dtype=dtype)
    m.masked_fill_(j > (n_k - n_q + i), float("-inf"))
    return m


def paged_attention_composed(q, k_cache, v_cache, block_table, context_lens, *,
                             q_start: Optional[Sequence[int]] = None, is_causal: bool = True,
                             sm_scale: Optional[float] = None, as_written: bool = False):
    """The reference's paged decode / chunked prefill, which it has only as a composition:
    per request, kv_paged_lookup with max_ctx = that request's length (a padded lookup
    would hand zero keys to an attention call that has no key-length argument), GQA
    expansion, then one attention call -- unmasked for a single query row, bottom-right
    masked for a chunk. q: [N_q, H, D] -> [N_q, H, D]."""
    B = int(context_lens.shape[0])
    lookup = kv_paged_lookup_as_written if as_written else kv_paged_lookup
    out = torch.zeros_like(q)
    for b in range(B):
        r0, r1 = (b, b + 1) if q_start is None else (int(q_start[b]), int(q_start[b + 1]))
        n_q, ctx = r1 - r0, int(context_lens[b])
        if n_q == 0 or ctx == 0:
            continue
        kd, vd = lookup(k_cache, v_cache, block_table[b:b + 1], context_lens[b:b + 1], ctx)
        qb = q[r0:r1].transpose(0, 1).unsqueeze(0)  # [1, H, n_q, D]
        mask = None
        if is_causal and n_q > 1:
            mask = bottom_right_mask(n_q, ctx, dtype=q.dtype)[None, None].expand(1, q.shape[1], n_q, ctx)
        ob = attention(qb, kd, vd, attn_mask=mask, sm_scale=sm_scale)
        out[r0:r1] = ob[0].transpose(0, 1)
    return out


# ---- int8 KV ------------------------------------------------------------------------
# The reference has the reading side only: its decode kernel takes `kv_int8` with one fp32 scale per
# (position, kv head) and widens a stored byte as int8 * scale (src/kernels/attention.cu:91-96,141-150;
# args include/reflex/infer.h:189-203). It ships no quantiser, so the writing side is defined here and
# the CUDA path is held to it bit for bit: symmetric absmax per row, fp32 arithmetic.

def kv_quantize_rows(x: torch.Tensor):
    """x [..., D] -> (int8 [..., D], float32 scale [...]): scale = max|x| / 127 (1 where the row is
    all zero), q = round-half-even(x / scale), clamped to [-127, 127]."""
    xf = x.float()
    amax = xf.abs().amax(dim=-1)
    scale = torch.where(amax > 0, amax / 127.0, torch.ones_like(amax))
    q = torch.round(xf / scale.unsqueeze(-1)).clamp_(-127, 127).to(torch.int8)
    return q, scale


def kv_paged_append_q8(k_in, v_in, k_cache, v_cache, k_scales, v_scales, slot_mapping) -> None:
    """kv_paged_append (triton_kv_paged.py:279-292) into an int8 pool: caches int8
    [num_blocks, H, bs, D], scales float32 [num_blocks, H, bs]."""
    block_size = k_cache.shape[2]
    page = torch.div(slot_mapping, block_size, rounding_mode="floor")
    pos = torch.remainder(slot_mapping, block_size)
    kq, ks = kv_quantize_rows(k_in)
    vq, vs = kv_quantize_rows(v_in)
    k_cache[page, :, pos, :] = kq
    v_cache[page, :, pos, :] = vq
    k_scales[page, :, pos] = ks
    v_scales[page, :, pos] = vs


def kv_dequantize(cache: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    """int8 * scale in float32, the widening of src/kernels/attention.cu:94-96,145-147."""
    return cache.float() * scales.unsqueeze(-1)


def merge_partials(m: torch.Tensor, l: torch.Tensor, acc: torch.Tensor) -> torch.Tensor:
    """Sequential running-max merge of split partials, the recurrence of
    kernels/softmax/triton_softmax.py:84-89 with the accumulator of
    triton_fused_attention.py:205-227: m [S], l [S], acc [S, D] -> [D] (float64 inside)."""
    M = torch.tensor(float("-inf"), dtype=torch.float64)
    L = torch.tensor(0.0, dtype=torch.float64)
    A = torch.zeros(acc.shape[1], dtype=torch.float64)
    for s in range(m.shape[0]):
        mi = m[s].double()
        if torch.isinf(mi) and mi < 0:
            continue
        Mn = torch.maximum(M, mi)
        a, bta = torch.exp(M - Mn), torch.exp(mi - Mn)
        L = L * a + l[s].double() * bta
        A = A * a + acc[s].double() * bta
        M = Mn
    return (A / L) if L > 0 else A


def fused_linear_norm(x, weight, *, bias=None, gamma=None, beta=None, eps: float = 1e-5, norm_type: str = "layer"):
    """torch_reference_fused_linear_norm, kernels/fused_linear_norm/triton_kernel.py:204-233:
    ``F.linear`` in the activation dtype, then ``F.layer_norm`` (``:221-227``) or RMSNorm spelled
    out (``:229-233``: statistics and scaling in fp32, one rounding, then ``* gamma`` in the
    activation dtype)."""
    y = F.linear(x, weight, bias)
    n = weight.shape[0]
    if norm_type.lower() == "layer":
        return F.layer_norm(y, (n,), weight=gamma, bias=beta, eps=eps)
    rms = y.float().pow(2).mean(dim=-1, keepdim=True).add(eps).rsqrt()
    out = (y.float() * rms).to(y.dtype)
    if gamma is not None:
        out = out * gamma
    return out
