"""Seeded synthetic workloads with the shapes of the five benchmark configurations.

The reference measures on no dataset; every configuration is a generator. One
``torch.Generator`` per batch, draws in a fixed order: context lengths, new-token counts,
free-page mask, page permutation, compaction choice, then q / k / v, then the pool fill.
Tensors are created on CPU when ``device`` is CPU (small parity cases, so the CPU oracle
and the GPU path see identical bits after a copy) or directly on the GPU (full-size
benchmark pools, tens of GB).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple

import torch


@dataclass
class PagedBatch:
    name: str
    dtype: torch.dtype
    Hq: int
    Hkv: int
    D: int
    block_size: int
    num_blocks: int
    theta: float
    old_lens: torch.Tensor       # [B] int32, keys in the pool before the step
    n_new: torch.Tensor          # [B] int32, new tokens per request
    context_lens: torch.Tensor   # [B] int32, old_lens + n_new
    q_start: torch.Tensor        # [B+1] int32, first query row of each request
    block_table: torch.Tensor    # [B, max_blocks] int64, -1 where unassigned
    slot_mapping: torch.Tensor   # [N] int64, pool slot of each new token
    positions: torch.Tensor      # [N] int32, sequence position (RoPE table row) of each new token
    q_new: torch.Tensor          # [N, Hq, D]
    k_new: torch.Tensor          # [N, Hkv, D]
    v_new: torch.Tensor          # [N, Hkv, D]
    k_cache: torch.Tensor        # [num_blocks, Hkv, block_size, D]
    v_cache: torch.Tensor
    cos: Optional[torch.Tensor] = None   # [max_pos+1, D] in dtype
    sin: Optional[torch.Tensor] = None
    max_q_len: int = 1
    extra: dict = field(default_factory=dict)

    @property
    def B(self) -> int:
        return int(self.old_lens.shape[0])

    @property
    def n_tokens(self) -> int:
        return int(self.q_new.shape[0])

    def kv_bytes(self) -> int:
        """Algorithmic bytes of one attention step: K and V of every visible key read once
        (the reference's accounting, benchmark/bench_attention.py:53-56)."""
        e = torch.empty((), dtype=self.dtype).element_size()
        return int(2 * self.Hkv * self.D * e * int(self.context_lens.sum().item()))

    def to(self, device) -> "PagedBatch":
        kw = {}
        for k, v in self.__dict__.items():
            kw[k] = v.to(device) if isinstance(v, torch.Tensor) else v
        return PagedBatch(**kw)


def make_paged_batch(
    name: str,
    *,
    B: int,
    Hq: int,
    Hkv: int,
    D: int,
    block_size: int,
    ctx_range: Tuple[int, int],
    new_range: Tuple[int, int] = (1, 1),
    decode_fraction: float = 0.0,
    num_blocks: Optional[int] = None,
    free_fraction: Optional[float] = None,
    theta: float = 1e6,
    dtype: torch.dtype = torch.bfloat16,
    device="cpu",
    seed: int = 0,
    input_scale: float = 1.0,
    fill_pool: bool = True,
    tables: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
    contiguous_pages: bool = False,
) -> PagedBatch:
    """Draw one batch. ``ctx_range`` / ``new_range`` are inclusive. ``free_fraction``: that
    share of the pool is marked free at random and only free pages are handed out (a
    fragmented pool); otherwise all pages are available. Pages go to requests in index
    order from a seeded permutation (or in ascending order with ``contiguous_pages``)."""
    device = torch.device(device)
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    old = torch.randint(ctx_range[0], ctx_range[1] + 1, (B,), generator=g, dtype=torch.int64)
    new = torch.randint(new_range[0], new_range[1] + 1, (B,), generator=g, dtype=torch.int64)
    if decode_fraction > 0:
        is_decode = torch.rand(B, generator=g) < decode_fraction
        new = torch.where(is_decode, torch.ones_like(new), new)
    total = old + new
    pages_per_req = (total + block_size - 1) // block_size
    need = int(pages_per_req.sum().item())
    if num_blocks is None:
        num_blocks = max(need, 1)
    free_mask = None
    if free_fraction is not None:
        free_mask = torch.rand(num_blocks, generator=g) < free_fraction
    perm = torch.arange(num_blocks) if contiguous_pages else torch.randperm(num_blocks, generator=g)
    if free_mask is not None:
        perm = perm[free_mask[perm]]
    if perm.numel() < need:
        raise ValueError(f"{name}: pool has {perm.numel()} usable pages, batch needs {need}")
    max_blocks = int(pages_per_req.max().item()) if B else 0
    block_table = torch.full((B, max_blocks), -1, dtype=torch.int64)
    page_start = torch.zeros(B + 1, dtype=torch.int64)
    page_start[1:] = torch.cumsum(pages_per_req, 0)
    # scatter the permutation into the table rows
    row = torch.repeat_interleave(torch.arange(B), pages_per_req)
    col = torch.arange(need) - page_start[row]
    block_table[row, col] = perm[:need]

    q_start = torch.zeros(B + 1, dtype=torch.int64)
    q_start[1:] = torch.cumsum(new, 0)
    N = int(q_start[-1].item())
    tok_req = torch.repeat_interleave(torch.arange(B), new)
    tok_idx = torch.arange(N) - q_start[tok_req]
    positions = old[tok_req] + tok_idx                      # sequence position of each new token
    slot_mapping = block_table[tok_req, positions // block_size] * block_size + positions % block_size

    gd = g
    if device.type == "cuda":
        gd = torch.Generator(device=device)
        gd.manual_seed(seed + 1)

    def randn(*shape):
        t = torch.randn(*shape, generator=gd, device=device, dtype=torch.float32)
        if input_scale != 1.0:
            t = t * input_scale
        return t.to(dtype)

    q_new, k_new, v_new = randn(N, Hq, D), randn(N, Hkv, D), randn(N, Hkv, D)
    if fill_pool:
        if device.type == "cuda":
            k_cache = torch.empty((num_blocks, Hkv, block_size, D), dtype=dtype, device=device)
            v_cache = torch.empty_like(k_cache)
            k_cache.normal_(generator=gd)
            v_cache.normal_(generator=gd)
            if input_scale != 1.0:
                k_cache.mul_(input_scale)
                v_cache.mul_(input_scale)
        else:
            k_cache, v_cache = randn(num_blocks, Hkv, block_size, D), randn(num_blocks, Hkv, block_size, D)
    else:
        k_cache = torch.zeros((num_blocks, Hkv, block_size, D), dtype=dtype, device=device)
        v_cache = torch.zeros_like(k_cache)

    cos = sin = None
    if tables is not None:
        cos, sin = tables[0].to(device=device, dtype=dtype), tables[1].to(device=device, dtype=dtype)
    elif device.type == "cuda":
        from kernels.rope import build_rope_tables
        cos, sin = build_rope_tables(int(total.max().item()) + 1 if B else 1, D, base=theta, device=device, dtype=dtype)

    return PagedBatch(
        name=name, dtype=dtype, Hq=Hq, Hkv=Hkv, D=D, block_size=block_size, num_blocks=num_blocks, theta=theta,
        old_lens=old.to(torch.int32).to(device), n_new=new.to(torch.int32).to(device),
        context_lens=total.to(torch.int32).to(device), q_start=q_start.to(torch.int32).to(device),
        block_table=block_table.to(device), slot_mapping=slot_mapping.to(device),
        positions=positions.to(torch.int32).to(device),
        q_new=q_new, k_new=k_new, v_new=v_new, k_cache=k_cache, v_cache=v_cache, cos=cos, sin=sin,
        max_q_len=int(new.max().item()) if B else 1,
        extra={"free_mask": free_mask, "pages_needed": need},
    )


# ---- the five configurations -----------------------------------------------------------
# `scale` shrinks batch and context for parity tests; 1.0 is the configuration as stated.

def cfg1(device="cpu", seed=0, tables=None) -> PagedBatch:
    """fp32 MHA decode: batch 1, 16 heads, head_dim 64, 256 keys in contiguous pages of 16,
    one new token, theta 1e4."""
    return make_paged_batch("cfg1", B=1, Hq=16, Hkv=16, D=64, block_size=16, ctx_range=(256, 256),
                            theta=1e4, dtype=torch.float32, device=device, seed=seed, tables=tables,
                            contiguous_pages=True)


def cfg2(device="cpu", seed=1, scale: float = 1.0, tables=None) -> PagedBatch:
    """bf16 GQA decode: 16 query / 2 kv heads, head_dim 128, batch 32, contexts uniform in
    [512, 8192], pages of 16 from a permuted 32768-page pool, theta 1e6."""
    B = max(1, round(32 * scale))
    lo, hi = max(1, round(512 * scale)), max(2, round(8192 * scale))
    return make_paged_batch("cfg2", B=B, Hq=16, Hkv=2, D=128, block_size=16, ctx_range=(lo, hi),
                            num_blocks=max(64, round(32768 * scale)), theta=1e6, device=device, seed=seed,
                            tables=tables)


def cfg4(device="cpu", seed=3, scale: float = 1.0, tables=None, B: Optional[int] = None) -> PagedBatch:
    """bf16 long-context decode: 256 requests, contexts uniform in [8192, 32768], 64 query /
    8 kv heads, head_dim 128, pages of 32, permuted pages."""
    if B is None:
        B = max(1, round(256 * scale))
    lo, hi = max(1, round(8192 * scale)), max(2, round(32768 * scale))
    return make_paged_batch("cfg4", B=B, Hq=64, Hkv=8, D=128, block_size=32, ctx_range=(lo, hi),
                            theta=1e6, device=device, seed=seed, tables=tables)


def cfg5(device="cpu", seed=4, scale: float = 1.0, tables=None, pool_pages: Optional[int] = None) -> PagedBatch:
    """bf16 mixed chunked-prefill + decode on a fragmented pool: 64 requests appending 1-64
    tokens (a share of them plain decode rows) to contexts uniform in [0, 16384], 28 query /
    4 kv heads, head_dim 128, pages of 16, 40 % of the pool free."""
    B = max(1, round(64 * scale))
    hi = max(1, round(16384 * scale))
    if pool_pages is None:
        pool_pages = max(256, round(1048576 * scale))
    return make_paged_batch("cfg5", B=B, Hq=28, Hkv=4, D=128, block_size=16, ctx_range=(0, hi),
                            new_range=(1, 64), decode_fraction=0.5, num_blocks=pool_pages, free_fraction=0.4,
                            theta=1e6, device=device, seed=seed, tables=tables)


def cfg3_shapes(scale: float = 1.0) -> dict:
    """Causal paged prefill: batch 8 x 2048 new tokens on an empty cache, 32 query / 8 kv
    heads, head_dim 128, pages of 16, theta 1e6, inputs scaled by 0.5."""
    return dict(B=max(1, round(8 * scale)), S=max(16, round(2048 * scale)), Hq=32, Hkv=8, D=128, block_size=16,
                theta=1e6, input_scale=0.5)


def cfg3(device="cpu", seed=2, scale: float = 1.0, tables=None, seq: Optional[int] = None) -> PagedBatch:
    """`scale` shrinks batch and sequence together (tests); `seq` pins the sequence length, so
    that `scale` then shrinks only the batch (small profiling cases of the full-length kernel)."""
    s = cfg3_shapes(scale)
    if seq is not None:
        s["S"] = int(seq)
    return make_paged_batch("cfg3", B=s["B"], Hq=s["Hq"], Hkv=s["Hkv"], D=s["D"], block_size=s["block_size"],
                            ctx_range=(0, 0), new_range=(s["S"], s["S"]), theta=s["theta"], device=device, seed=seed,
                            input_scale=s["input_scale"], fill_pool=False, tables=tables)
