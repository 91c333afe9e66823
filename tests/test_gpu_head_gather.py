"""The head gather fused into the combine kernel (kv-head sharding without a collective call):
addressing, flags and the bounded wait, on one GPU. Ranks are emulated one launch after another
with every buffer in this process, and only a launch whose peers have already published may wait
-- two launches that wait on each other never share a GPU. The real multi-process path (CUDA IPC
mappings, concurrent ranks) is exercised by ``bench.py --gpus N --shard head --gather fused``."""
import pytest
import torch

import oracle
import workloads
from kernels.attention import PagedAttentionCall, PagedWorkspace
from sharding import FusedHeadGather, shard_batch_by_kv_head

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0)


def _batch(seed=11, Hq=16, Hkv=4):
    cpu = workloads.make_paged_batch("gather", B=6, Hq=Hq, Hkv=Hkv, D=128, block_size=16, ctx_range=(40, 900),
                                     num_blocks=512, seed=seed)
    return cpu, cpu.to(DEV)


def _call(b, ws=None):
    return PagedAttentionCall(b.q_new, b.k_cache, b.v_cache, b.block_table, b.context_lens,
                              workspace=ws or PagedWorkspace(DEV))


def test_single_rank_gather_equals_plain_combine(native):
    _, g = _batch()
    call = _call(g)
    want = _staged(call)
    gather = FusedHeadGather(g.q_new.shape[0], g.Hq, g.D, g.dtype, DEV, None)
    first = call.run_gather(gather)
    assert call.workspace.status() == 0
    assert torch.equal(first, want)
    second = call.run_gather(gather)           # the other buffer, next epoch
    assert second.data_ptr() != first.data_ptr() and torch.equal(second, want)
    flags = gather.buf[:4].view(torch.int32)
    assert int(flags[0]) == 2                  # rank 0 published epoch 2 to itself


def _staged(call):
    """plan, partial kernel, combine kernel as three calls: the arithmetic of the gathering combine."""
    call.plan()
    call.partials()
    return call.combine().clone()


@pytest.mark.parametrize("world", [2, 4])
def test_emulated_ranks_assemble_all_heads(world, native):
    cpu, g = _batch(seed=20 + world)
    whole = _call(g).run()
    n = g.q_new.shape[0]
    members = [FusedHeadGather(n, g.Hq // world, g.D, g.dtype, DEV, None, emulate_world=world) for _ in range(world)]
    calls = []
    for r in range(world):
        shard = shard_batch_by_kv_head(g, r, world)
        calls.append(_call(shard))
    # the same sharded computation with the plain combine, heads concatenated in rank order
    want = torch.cat([_staged(c) for c in calls], dim=1)
    # ... and as one call (the decode kernel merges its cut pairs itself, summing in another order)
    fused = torch.cat([c.run().clone() for c in calls], dim=1)
    torch.testing.assert_close(fused.float(), want.float(), atol=4e-3, rtol=1e-2)
    torch.testing.assert_close(want.float(), whole.float(), atol=1e-2, rtol=1e-2)  # split points differ
    for step in (1, 2, 3):
        outs = []
        for r in range(world):
            # every earlier rank has published by the time the last one runs: only it waits
            gr = FusedHeadGather.over_local_buffers(members, r, wait=(r == world - 1), spin_limit=1000)
            gr.epoch = step - 1
            outs.append(calls[r].run_gather(gr))
            assert calls[r].workspace.status() == 0
        torch.cuda.synchronize()
        for r in range(world):
            assert torch.equal(outs[r], want), f"rank {r} step {step}"
            flags = members[r].buf[:4 * world].view(torch.int32)
            assert flags.tolist() == [step] * world
    ref = oracle.paged_attention_composed(cpu.q_new, cpu.k_cache, cpu.v_cache, cpu.block_table, cpu.context_lens)
    torch.testing.assert_close(want.cpu().float(), ref.float(), atol=2e-2, rtol=2e-2)


def test_wait_runs_out_and_reports(native):
    """A peer that never publishes: the wait gives up after its limit, sets bit 0 of the status
    word and the kernel returns; the next call works."""
    _, g = _batch(seed=31)
    n = g.q_new.shape[0]
    members = [FusedHeadGather(n, g.Hq // 2, g.D, g.dtype, DEV, None, emulate_world=2) for _ in range(2)]
    call = _call(shard_batch_by_kv_head(g, 0, 2))
    gr = FusedHeadGather.over_local_buffers(members, 0, wait=True, spin_limit=2000)  # ~0.2 ms of polling
    call.run_gather(gr)
    assert call.workspace.status() & 1
    plain = _call(g)
    out = plain.run()
    assert plain.workspace.status() == 0 and torch.isfinite(out).all()


def test_gather_argument_checks(native):
    _, g = _batch(seed=32)
    call = _call(g)
    gather = FusedHeadGather(g.q_new.shape[0], g.Hq, g.D, g.dtype, DEV, None)
    gather._args.rank = 3                      # outside the group
    with pytest.raises(ValueError):
        call.run_gather(gather)


def test_gather_step_replays_from_a_cuda_graph(native):
    """The step with the gathering combine captured once and replayed: the epoch advances in a device
    word and the kernel alternates between the two output buffers by itself (one rank; its own flag
    is the only one it waits for)."""
    cpu, g = _batch(seed=31)
    call = _call(g)
    want = _staged(call)
    gather = FusedHeadGather(g.q_new.shape[0], g.Hq, g.D, g.dtype, DEV, None)
    call.run_gather_replayable(gather)          # launch 1, outside the graph (first use of the kernels)
    torch.cuda.synchronize()
    assert torch.equal(gather.output_of(1), want)
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            call.run_gather_replayable(gather)
    torch.cuda.synchronize()
    for n in (2, 3, 4):
        gather.output_of(n).fill_(float("nan"))
        graph.replay()
        torch.cuda.synchronize()
        assert call.workspace.status() == 0
        assert int(gather.epoch_word.item()) == n
        assert torch.equal(gather.output_of(n), want), f"replay {n}"
        flags = gather.buf[:4].view(torch.int32)
        assert int(flags[0]) == n
