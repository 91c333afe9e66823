"""Multi-rank host logic on CPU: two ``gloo`` ranks shard a batch by request (no collective)
and by kv head (one all-gather) and must reproduce the unsharded result. The per-rank
compute here is the CPU oracle -- the partitioning, remapping and gather order are what is
under test; the same helpers drive the GPU ranks in bench.py."""
from __future__ import annotations

import os
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def _setup_paths():
    for p in (ROOT / "reflex-infer_b200", ROOT, ROOT / "tests"):
        if str(p) not in sys.path:
            sys.path.insert(0, str(p))


def _attend(batch):
    import oracle
    qs = None if batch.max_q_len == 1 else batch.q_start.tolist()
    return oracle.paged_attention_composed(batch.q_new, batch.k_cache, batch.v_cache, batch.block_table,
                                           batch.context_lens, q_start=qs)


def _make_batch():
    import workloads
    return workloads.make_paged_batch("shard", B=7, Hq=8, Hkv=4, D=32, block_size=8, ctx_range=(0, 90),
                                      new_range=(1, 5), num_blocks=200, free_fraction=0.7, dtype=torch.float32, seed=11)


def _worker(rank, world, port, mode, q):
    _setup_paths()
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import sharding
        full = _make_batch()
        if mode == "request":
            mine = sharding.shard_batch_by_request(full, rank, world)
            out = _attend(mine)
            gathered = [None] * world
            dist.all_gather_object(gathered, (out, mine.extra["requests"]))
            if rank == 0:
                merged = sharding.merge_request_outputs([g[0] for g in gathered], [g[1] for g in gathered],
                                                        full.q_start.tolist())
                q.put(("request", merged))
        else:
            mine = sharding.shard_batch_by_kv_head(full, rank, world)
            out = _attend(mine)
            g = sharding.HeadGather(out, dist)
            merged = g.run(out)
            if rank == 0:
                q.put(("head", merged.clone()))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode,port", [("request", 29611), ("head", 29612)])
def test_two_ranks_reproduce_unsharded(mode, port):
    _setup_paths()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, mode, q)) for r in range(2)]
    for p in procs:
        p.start()
    kind, merged = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    ref = _attend(_make_batch())
    assert kind == mode
    torch.testing.assert_close(merged, ref, atol=1e-6, rtol=1e-6)


def test_balance_requests_properties():
    _setup_paths()
    import sharding
    lens = [8192, 32768, 9000, 20000, 20000, 15000, 31000, 8200, 12000]
    for world in (1, 2, 4, 8):
        parts = sharding.balance_requests(lens, world)
        flat = sorted(i for p in parts for i in p)
        assert flat == list(range(len(lens)))          # a partition
        loads = [sum(lens[i] for i in p) for p in parts]
        assert max(loads) - min(loads) <= max(lens)    # greedy bound
        assert parts == sharding.balance_requests(lens, world)  # deterministic


def test_request_shard_compaction_keeps_contents():
    _setup_paths()
    import sharding
    full = _make_batch()
    for rank in range(3):
        s = sharding.shard_batch_by_request(full, rank, 3)
        for j, req in enumerate(s.extra["requests"]):
            n = int(full.context_lens[req])
            for t in (0, n // 2, n - 1):
                if n == 0:
                    continue
                a = full.k_cache[full.block_table[req, t // 8], :, t % 8]
                b = s.k_cache[s.block_table[j, t // 8], :, t % 8]
                assert torch.equal(a, b)
        # new-token slots still point at the request's own position
        rows = 0
        for j, req in enumerate(s.extra["requests"]):
            for i in range(int(s.n_new[j])):
                pos = int(s.positions[rows])
                assert int(s.slot_mapping[rows]) == int(s.block_table[j, pos // 8]) * 8 + pos % 8
                rows += 1


def test_head_slices():
    _setup_paths()
    import sharding
    assert sharding.head_slices(64, 8, 3, 8) == ((3, 4), (24, 32))
    assert sharding.head_slices(64, 8, 1, 2) == ((4, 8), (32, 64))
    with pytest.raises(ValueError):
        sharding.head_slices(28, 4, 0, 8)
