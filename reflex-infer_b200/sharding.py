"""Multi-GPU partitioning of the paged decode step. One process per GPU.

The path shards two ways, neither with a collective inside the attention computation:

* by request   -- each rank owns whole requests (their pages, block-table rows, query rows
                  and outputs); requests are dealt out longest-first to the least loaded rank
                  so ranks read about the same number of KV bytes. No collective at all.
* by kv head   -- rank r owns kv heads [r*Hkv/g, (r+1)*Hkv/g) of every page and the query
                  heads that read them; the page table is replicated. One all-gather of the
                  output heads ([B, Hq/g, D] per rank -> [B, Hq, D]) follows the combine.

The reference has no multi-GPU code; these helpers are host-side index arithmetic plus
``torch.distributed`` calls and run unchanged on CPU tensors with the ``gloo`` backend.
"""
from __future__ import annotations

from typing import List, Sequence

import torch

from workloads import PagedBatch


def balance_requests(lengths: Sequence[int], world: int) -> List[List[int]]:
    """Greedy longest-first assignment of request indices to ``world`` ranks; each rank's
    list is returned in ascending request order. Deterministic (ties go to the lower rank,
    then to the lower request index)."""
    order = sorted(range(len(lengths)), key=lambda i: (-int(lengths[i]), i))
    load = [0] * world
    out: List[List[int]] = [[] for _ in range(world)]
    for i in order:
        r = min(range(world), key=lambda k: (load[k], k))
        out[r].append(i)
        load[r] += int(lengths[i])
    return [sorted(x) for x in out]


def shard_batch_by_request(batch: PagedBatch, rank: int, world: int, compact: bool = True) -> PagedBatch:
    """The sub-batch of ``rank``. With ``compact`` the pool is reduced to the pages the rank's
    requests own (renumbered in block-table order), which is what a rank of a real
    deployment would hold."""
    mine = balance_requests(batch.context_lens.tolist(), world)[rank]
    idx = torch.tensor(mine, dtype=torch.long, device=batch.context_lens.device)
    n_new = batch.n_new[idx]
    q0 = batch.q_start.long()
    rows = torch.cat([torch.arange(int(q0[i]), int(q0[i + 1]), device=idx.device) for i in mine]) if mine else \
        torch.zeros(0, dtype=torch.long, device=idx.device)
    bt = batch.block_table[idx]
    k_cache, v_cache, slot_mapping = batch.k_cache, batch.v_cache, batch.slot_mapping[rows]
    num_blocks = batch.num_blocks
    if compact:
        used = bt[bt >= 0]
        remap = torch.full((batch.num_blocks,), -1, dtype=torch.long, device=bt.device)
        remap[used] = torch.arange(used.numel(), device=bt.device)
        k_cache, v_cache = batch.k_cache[used].contiguous(), batch.v_cache[used].contiguous()
        bt = torch.where(bt >= 0, remap[bt.clamp(min=0)], bt)
        bs = batch.block_size
        slot_mapping = remap[torch.div(slot_mapping, bs, rounding_mode="floor")] * bs + slot_mapping % bs
        num_blocks = int(used.numel())
    q_start = torch.zeros(len(mine) + 1, dtype=torch.int32, device=idx.device)
    q_start[1:] = torch.cumsum(n_new, 0)
    return PagedBatch(
        name=f"{batch.name}[req {rank}/{world}]", dtype=batch.dtype, Hq=batch.Hq, Hkv=batch.Hkv, D=batch.D,
        block_size=batch.block_size, num_blocks=num_blocks, theta=batch.theta,
        old_lens=batch.old_lens[idx], n_new=n_new, context_lens=batch.context_lens[idx], q_start=q_start,
        block_table=bt.contiguous(), slot_mapping=slot_mapping, positions=batch.positions[rows],
        q_new=batch.q_new[rows].contiguous(), k_new=batch.k_new[rows].contiguous(),
        v_new=batch.v_new[rows].contiguous(), k_cache=k_cache, v_cache=v_cache, cos=batch.cos, sin=batch.sin,
        max_q_len=batch.max_q_len, extra={"requests": mine},
    )


def head_slices(Hq: int, Hkv: int, rank: int, world: int):
    """(kv head range, query head range) of ``rank``; needs ``Hkv % world == 0``."""
    if Hkv % world != 0:
        raise ValueError(f"kv heads ({Hkv}) must divide evenly over {world} ranks")
    per = Hkv // world
    g = Hq // Hkv
    return (rank * per, (rank + 1) * per), (rank * per * g, (rank + 1) * per * g)


def shard_batch_by_kv_head(batch: PagedBatch, rank: int, world: int) -> PagedBatch:
    (k0, k1), (q0, q1) = head_slices(batch.Hq, batch.Hkv, rank, world)
    return PagedBatch(
        name=f"{batch.name}[heads {rank}/{world}]", dtype=batch.dtype, Hq=q1 - q0, Hkv=k1 - k0, D=batch.D,
        block_size=batch.block_size, num_blocks=batch.num_blocks, theta=batch.theta,
        old_lens=batch.old_lens, n_new=batch.n_new, context_lens=batch.context_lens, q_start=batch.q_start,
        block_table=batch.block_table, slot_mapping=batch.slot_mapping, positions=batch.positions,
        q_new=batch.q_new[:, q0:q1].contiguous(), k_new=batch.k_new[:, k0:k1].contiguous(),
        v_new=batch.v_new[:, k0:k1].contiguous(), k_cache=batch.k_cache[:, k0:k1].contiguous(),
        v_cache=batch.v_cache[:, k0:k1].contiguous(), cos=batch.cos, sin=batch.sin, max_q_len=batch.max_q_len,
        extra={"kv_heads": (k0, k1), "q_heads": (q0, q1)},
    )


class HeadGather:
    """All-gather of head-sharded outputs into ``[N, Hq, D]``; gather order = rank order =
    head order. Buffers are allocated once."""

    def __init__(self, out_local: torch.Tensor, dist):
        self.dist = dist
        self.world = dist.get_world_size()
        n, h, d = out_local.shape
        self.stage = torch.empty((self.world * n, h, d), dtype=out_local.dtype, device=out_local.device)
        self.full = torch.empty((n, self.world * h, d), dtype=out_local.dtype, device=out_local.device)

    def run(self, out_local: torch.Tensor) -> torch.Tensor:
        self.dist.all_gather_into_tensor(self.stage, out_local.contiguous())
        n, h, d = out_local.shape
        self.full.view(n, self.world, h, d).copy_(self.stage.view(self.world, n, h, d).permute(1, 0, 2, 3))
        return self.full


def merge_request_outputs(parts: Sequence[torch.Tensor], assignment: Sequence[Sequence[int]], q_start) -> torch.Tensor:
    """Host-side reassembly of request-sharded outputs (used by tests; a deployment keeps the
    rows where they are): parts[r] holds the rows of assignment[r]'s requests in order."""
    total = int(q_start[-1])
    out = torch.empty((total,) + tuple(parts[0].shape[1:]), dtype=parts[0].dtype, device=parts[0].device)
    for part, reqs in zip(parts, assignment):
        o = 0
        for i in reqs:
            n = int(q_start[i + 1]) - int(q_start[i])
            out[int(q_start[i]):int(q_start[i + 1])] = part[o:o + n]
            o += n
    return out
