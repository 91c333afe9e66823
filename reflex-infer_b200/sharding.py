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


class FusedHeadGather:
    """The head gather without a collective call: each rank's combine kernel stores its head
    slice of every output row straight into all ranks' full outputs through peer-mapped
    pointers, and the ranks meet at a flag barrier inside the same kernel (bounded wait).

    One buffer per rank holds the flag array and two full outputs (used alternately: a peer may
    already write step k+1 while this rank still reads step k). It is exported once through
    CUDA IPC; the handles travel through ``dist.all_gather_object``. One process per GPU."""

    FLAG_BYTES = 256

    def __init__(self, n_rows: int, local_heads: int, head_dim: int, dtype: torch.dtype, device, dist,
                 spin_limit: int = 0, emulate_world: int = 0):
        from kernels import _native as N
        self.dist = dist
        self.world = dist.get_world_size() if dist is not None else max(1, emulate_world)
        self.rank = dist.get_rank() if dist is not None else 0
        if self.world > N.RFX_MAX_PEERS:
            raise ValueError(f"at most {N.RFX_MAX_PEERS} ranks, got {self.world}")
        self.shape = (n_rows, self.world * local_heads, head_dim)
        elt = torch.empty((), dtype=dtype).element_size()
        self.out_bytes = -(-n_rows * self.world * local_heads * head_dim * elt // 256) * 256
        self.buf = torch.zeros(self.FLAG_BYTES + 2 * self.out_bytes, dtype=torch.uint8, device=device)
        self.counter = torch.zeros(1, dtype=torch.int32, device=device)
        self.full = [self.buf[self.FLAG_BYTES + i * self.out_bytes:][:n_rows * self.shape[1] * head_dim * elt]
                     .view(dtype).view(self.shape) for i in range(2)]
        torch.cuda.synchronize(device)  # the zeros are in place before any peer can write
        self._bases = []
        self.ptrs = [0] * self.world
        if self.world > 1 and dist is not None:
            mine = N.peer_export(self.buf.data_ptr(), device)
            handles = [None] * self.world
            dist.all_gather_object(handles, mine)
            for p, h in enumerate(handles):
                if p == self.rank:
                    self.ptrs[p] = self.buf.data_ptr()
                else:
                    mapped, base = N.peer_open(h, device)
                    self.ptrs[p] = mapped
                    self._bases.append(base)
            dist.barrier()
        else:
            self.ptrs[0] = self.buf.data_ptr()
        self.epoch = 0
        self.device = device
        self._args = N.HeadGatherArgs()
        self._bind(spin_limit)

    def _bind(self, spin_limit: int = 0, wait: bool = True) -> None:
        a = self._args
        a.world, a.rank = self.world, self.rank
        a.arrival_counter = self.counter.data_ptr()
        a.wait = int(bool(wait))
        a.spin_limit = int(spin_limit)
        for p in range(self.world):
            a.peer_flags[p] = self.ptrs[p]

    @classmethod
    def over_local_buffers(cls, members, rank: int, wait: bool, spin_limit: int = 0):
        """A member of a group whose buffers all live in this process (``members``: one gather
        per emulated rank, each built with ``dist=None, emulate_world=len(members)``). For
        single-GPU tests of the addressing and the flags; emulated ranks run one after another
        and only the last one may wait."""
        g = members[rank]
        g.rank = rank
        g.ptrs = [m.buf.data_ptr() for m in members]
        g._args = type(g._args)()
        g._bind(spin_limit, wait)
        return g

    def next_args(self):
        """Arguments of the next step (advances the epoch) and the tensor that will hold its output."""
        self.epoch += 1
        a = self._args
        a.epoch = self.epoch
        off = self.FLAG_BYTES + (self.epoch & 1) * self.out_bytes
        for p in range(self.world):
            a.peer_out[p] = self.ptrs[p] + off
        return a, self.full[self.epoch & 1]

    def replayable_args(self):
        """Arguments for a step that is captured once in a CUDA graph and replayed: the epoch lives in
        a device word the kernel advances itself, and the kernel picks the output buffer from the
        epoch's parity. ``output_of(n)`` is the tensor the n-th launch (n = 1, 2, ...) wrote."""
        if not hasattr(self, "epoch_word"):
            self.epoch_word = torch.zeros(1, dtype=torch.int32, device=self.device)
        a = self._args
        a.epoch = 0
        a.epoch_word = self.epoch_word.data_ptr()
        a.out_alt_offset = self.out_bytes
        for p in range(self.world):
            a.peer_out[p] = self.ptrs[p] + self.FLAG_BYTES
        return a

    def output_of(self, n: int) -> torch.Tensor:
        return self.full[n & 1]

    def close(self) -> None:
        from kernels import _native as N
        torch.cuda.synchronize(self.device)
        if self.dist is not None and self.world > 1:
            self.dist.barrier()  # nobody unmaps while a peer may still store
        for base in self._bases:
            N.peer_close(base, self.device)
        self._bases = []


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
