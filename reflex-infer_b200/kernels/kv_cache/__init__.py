"""Paged KV pool operations; same surface as the reference's ``kernels/kv_cache/__init__.py``.

* ``kv_paged_append``  : write new K/V rows at flat slots (``kv_cache/__init__.py:31-51``).
* ``kv_paged_lookup``  : gather pages into dense ``[B, H, max_ctx, D]`` with a zero tail
  (``kv_cache/__init__.py:54-71``).
* ``kv_paged_scatter`` : overwrite slots; the same operation as append
  (``kv_cache/__init__.py:74-90``).

Pool layout ``[num_blocks, num_heads, block_size, head_dim]``, ``slot = page*block_size + pos``
(``triton_kv_paged.py:9-15``). The caches are mutated in place.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _native as N


def _check_pool(name, k_cache, v_cache):
    if k_cache.dim() != 4 or v_cache.shape != k_cache.shape:
        raise ValueError(f"{name}: caches must both be [num_blocks, num_heads, block_size, head_dim]; "
                         f"got {tuple(k_cache.shape)} and {tuple(v_cache.shape)}")
    if k_cache.dtype != v_cache.dtype:
        raise ValueError(f"{name}: k_cache and v_cache dtypes differ")
    if k_cache.stride() != v_cache.stride():
        raise ValueError(f"{name}: k_cache and v_cache must share one stride pattern")
    if k_cache.stride(3) != 1:
        raise ValueError(f"{name}: the head_dim axis of the caches must be contiguous")


def _write_slots(entry, name, k_in, v_in, k_cache, v_cache, slot_mapping):
    dev = N.require_cuda(name, k_in, v_in, k_cache, v_cache, slot_mapping)
    _check_pool(name, k_cache, v_cache)
    if k_in.dim() != 3 or v_in.shape != k_in.shape:
        raise ValueError(f"{name}: k_in and v_in must both be [N, num_heads, head_dim]")
    n, heads, dim = k_in.shape
    nb, ch, bs, cd = k_cache.shape
    if (heads, dim) != (ch, cd):
        raise ValueError(f"{name}: input heads/head_dim {(heads, dim)} do not match the cache {(ch, cd)}")
    if k_in.dtype != k_cache.dtype or v_in.dtype != k_cache.dtype:
        # torch's index_put_ refuses this too ("source and destination dtypes match")
        raise RuntimeError(f"{name}: input dtype {k_in.dtype} does not match cache dtype {k_cache.dtype}")
    if slot_mapping.dim() != 1 or slot_mapping.shape[0] != n:
        raise ValueError(f"{name}: slot_mapping must be [N]={n}, got {tuple(slot_mapping.shape)}")
    if slot_mapping.dtype != torch.int64:
        slot_mapping = slot_mapping.to(torch.int64)
    slot_mapping = slot_mapping.contiguous()
    if k_in.stride(2) != 1 or v_in.stride() != k_in.stride():
        k_in, v_in = k_in.contiguous(), v_in.contiguous()
    a = N.KvAppendArgs(
        k_in=N.ptr(k_in), v_in=N.ptr(v_in), k_cache=N.ptr(k_cache), v_cache=N.ptr(v_cache),
        slot_mapping=N.ptr(slot_mapping),
        n_tokens=n, num_kv_heads=heads, head_dim=dim, num_blocks=nb, block_size=bs,
        in_stride_n=k_in.stride(0), in_stride_h=k_in.stride(1),
        cache_stride_blk=k_cache.stride(0), cache_stride_h=k_cache.stride(1), cache_stride_pos=k_cache.stride(2),
        dtype=N.dtype_code(k_cache), stream=N.stream_handle(dev),
    )
    N.call(entry, a, dev)


def kv_paged_append(
    k_in: torch.Tensor,
    v_in: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    slot_mapping: torch.Tensor,
    *,
    backend: Optional[str] = None,
) -> None:
    """Append new K, V into the paged KV cache (in place).

    ``k_in``/``v_in``: ``[N, num_heads, head_dim]``; ``slot_mapping``: ``[N]`` int64 flat
    slots. Slots must be distinct; a slot outside the pool is skipped.
    """
    N.check_backend(backend)
    _write_slots("rfx_kv_paged_append", "kv_paged_append", k_in, v_in, k_cache, v_cache, slot_mapping)


def kv_paged_lookup(
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    block_table: torch.Tensor,
    context_lens: torch.Tensor,
    max_ctx: int,
    *,
    backend: Optional[str] = None,
) -> tuple:
    """Gather K, V from the paged cache into dense ``[B, num_heads, max_ctx, head_dim]``
    tensors; positions at or beyond ``context_lens[b]`` are zero in both."""
    N.check_backend(backend)
    name = "kv_paged_lookup"
    dev = N.require_cuda(name, k_cache, v_cache, block_table, context_lens)
    _check_pool(name, k_cache, v_cache)
    if block_table.dim() != 2:
        raise ValueError(f"{name}: block_table must be [B, max_blocks]")
    B = context_lens.shape[0]
    if block_table.shape[0] != B:
        raise ValueError(f"{name}: block_table has {block_table.shape[0]} rows, context_lens {B}")
    if block_table.dtype != torch.int64:
        block_table = block_table.to(torch.int64)
    if block_table.stride(1) != 1:
        block_table = block_table.contiguous()
    if context_lens.dtype != torch.int32:
        context_lens = context_lens.to(torch.int32)
    context_lens = context_lens.contiguous()
    nb, heads, bs, dim = k_cache.shape
    max_ctx = int(max_ctx)
    k_out = torch.empty((B, heads, max_ctx, dim), dtype=k_cache.dtype, device=dev)
    v_out = torch.empty_like(k_out)
    a = N.KvLookupArgs(
        k_cache=N.ptr(k_cache), v_cache=N.ptr(v_cache), k_out=N.ptr(k_out), v_out=N.ptr(v_out),
        block_table=N.ptr(block_table), context_lens=N.ptr(context_lens),
        batch=B, num_kv_heads=heads, head_dim=dim, num_blocks=nb, block_size=bs,
        max_ctx=max_ctx, max_blocks=block_table.shape[1],
        cache_stride_blk=k_cache.stride(0), cache_stride_h=k_cache.stride(1), cache_stride_pos=k_cache.stride(2),
        bt_stride_b=block_table.stride(0),
        dtype=N.dtype_code(k_cache), stream=N.stream_handle(dev),
    )
    N.call("rfx_kv_paged_lookup", a, dev)
    return k_out, v_out


def kv_paged_scatter(
    k_updates: torch.Tensor,
    v_updates: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    slot_mapping: torch.Tensor,
    *,
    backend: Optional[str] = None,
) -> None:
    """Overwrite specific slots (speculative decoding rollback, page compaction)."""
    N.check_backend(backend)
    _write_slots("rfx_kv_paged_scatter", "kv_paged_scatter", k_updates, v_updates, k_cache, v_cache, slot_mapping)


__all__ = [
    "kv_paged_append",
    "kv_paged_lookup",
    "kv_paged_scatter",
]
