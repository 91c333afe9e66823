"""GPU parity of the fused paged path through the C ABI: RoPE + append, split-K paged
attention (both the TMA/MMA kernel and the scalar kernel) and combine, against the golden
decode steps of the reference and the CPU oracle. Pool contents bit-exact; outputs within
2e-2 (bf16/fp16) or 1e-5 (fp32)."""
from __future__ import annotations

import pytest
import torch

import golden_cases as gc
import golden_io
import oracle
import workloads
from kernels.attention import (PagedWorkspace, paged_attention, paged_decode, paged_decode_step, rope_append,
                               splitk_combine)
from kernels.kv_cache import kv_paged_append, kv_paged_scatter

pytestmark = [pytest.mark.gpu]
DEV = "cuda"
TOL = {torch.float32: 1e-5, torch.bfloat16: 2e-2, torch.float16: 5e-3}


def _clean(ws):
    assert ws.status() == 0, f"device status word {ws.status()}"


@pytest.mark.parametrize("force_generic", [False, True])
@pytest.mark.parametrize("name", sorted(gc.step_cases()))
def test_decode_step_golden(name, force_generic, native):
    c = gc.step_cases()[name]
    t, meta = golden_io.load(name)
    cos, sin = oracle.build_rope_tables(c["table_rows"], c["D"], base=c["theta"], dtype=c["dtype"])
    kc, vc = c["k_cache0"].to(DEV), c["v_cache0"].to(DEV)
    ws = PagedWorkspace(DEV)
    out = paged_decode_step(c["q"].to(DEV), c["k"].to(DEV), c["v"].to(DEV), kc, vc, c["block_table"].to(DEV),
                            c["context_lens"].to(DEV), c["slots"].to(DEV), c["positions"].to(DEV), cos.to(DEV),
                            sin.to(DEV), workspace=ws, force_generic=force_generic)
    _clean(ws)
    assert golden_io.digest(kc) == meta["k_digest"] and golden_io.digest(vc) == meta["v_digest"]
    tol = TOL[c["dtype"]]
    torch.testing.assert_close(out.cpu().float(), t["out"].float(), atol=tol, rtol=tol)


@pytest.mark.parametrize("name", sorted(gc.step_cases()))
def test_rope_append_returns_rotated_q(name, native):
    c = gc.step_cases()[name]
    t, meta = golden_io.load(name)
    cos, sin = oracle.build_rope_tables(c["table_rows"], c["D"], base=c["theta"], dtype=c["dtype"])
    kc, vc = c["k_cache0"].to(DEV), c["v_cache0"].to(DEV)
    q_rot = rope_append(c["k"].to(DEV), c["v"].to(DEV), kc, vc, c["slots"].to(DEV), c["positions"].to(DEV),
                        cos.to(DEV), sin.to(DEV), q=c["q"].to(DEV))
    assert torch.equal(q_rot.cpu(), t["q_rot"])
    assert golden_io.digest(kc) == meta["k_digest"] and golden_io.digest(vc) == meta["v_digest"]
    # fused Q rotation inside attention == attention on the pre-rotated q
    a = paged_decode(q_rot, kc, vc, c["block_table"].to(DEV), c["context_lens"].to(DEV))
    b = paged_decode(c["q"].to(DEV), kc, vc, c["block_table"].to(DEV), c["context_lens"].to(DEV),
                     rope_cos=cos.to(DEV), rope_sin=sin.to(DEV), rope_positions=c["positions"].to(DEV))
    assert torch.equal(a, b)


def _oracle_step(cpu, cos, sin):
    pos = cpu.positions.long()
    q_rot = oracle.apply_rope(cpu.q_new.unsqueeze(0), cos[pos], sin[pos])[0]
    k_rot = oracle.apply_rope(cpu.k_new.unsqueeze(0), cos[pos], sin[pos])[0]
    kc, vc = cpu.k_cache.clone(), cpu.v_cache.clone()
    oracle.kv_paged_append(k_rot, cpu.v_new, kc, vc, cpu.slot_mapping)
    qs = None if cpu.max_q_len == 1 else cpu.q_start.tolist()
    out = oracle.paged_attention_composed(q_rot, kc, vc, cpu.block_table, cpu.context_lens, q_start=qs)
    return q_rot, kc, vc, out


@pytest.mark.parametrize("cfg,scale", [("cfg2", 0.12), ("cfg4", 0.02), ("cfg1", 1.0)])
@pytest.mark.parametrize("chunk", [0, 64, 448, 1 << 20])
def test_decode_configs_split_invariance(cfg, scale, chunk, native):
    """Scaled benchmark configurations vs the oracle, for several split lengths (1 << 20 means
    a single split per request): the output may move within tolerance, the pool not at all."""
    theta = 1e4 if cfg == "cfg1" else 1e6
    dtype = torch.float32 if cfg == "cfg1" else torch.bfloat16
    D = 64 if cfg == "cfg1" else 128
    rows = {"cfg1": 258, "cfg2": 1100, "cfg4": 800}[cfg]
    cos, sin = oracle.build_rope_tables(rows, D, base=theta, dtype=dtype)
    cpu = getattr(workloads, cfg)(tables=(cos, sin)) if cfg == "cfg1" else getattr(workloads, cfg)(scale=scale, tables=(cos, sin))
    q_rot, kc, vc, ref = _oracle_step(cpu, cos, sin)
    gpu = cpu.to(DEV)
    ws = PagedWorkspace(DEV)
    out = paged_decode_step(gpu.q_new, gpu.k_new, gpu.v_new, gpu.k_cache, gpu.v_cache, gpu.block_table,
                            gpu.context_lens, gpu.slot_mapping, gpu.positions, gpu.cos, gpu.sin, workspace=ws,
                            target_chunk=chunk)
    _clean(ws)
    assert torch.equal(gpu.k_cache.cpu(), kc) and torch.equal(gpu.v_cache.cpu(), vc)
    tol = TOL[dtype]
    torch.testing.assert_close(out.cpu().float(), ref.float(), atol=tol, rtol=tol)
    # the scalar kernel agrees with the tensor-core kernel on the same plan
    out_g = paged_decode(gpu.q_new, gpu.k_cache, gpu.v_cache, gpu.block_table, gpu.context_lens,
                         rope_cos=gpu.cos, rope_sin=gpu.sin, rope_positions=gpu.positions, workspace=ws,
                         force_generic=True, target_chunk=chunk)
    torch.testing.assert_close(out_g.float(), out.float(), atol=tol, rtol=tol)


@pytest.mark.parametrize("dtype,bs,D,G", [(torch.float16, 8, 64, 4), (torch.bfloat16, 64, 128, 16),
                                          (torch.bfloat16, 128, 128, 1), (torch.float16, 16, 128, 12),
                                          (torch.bfloat16, 4, 128, 8), (torch.bfloat16, 16, 96, 2)])
def test_decode_shape_coverage(dtype, bs, D, G, native):
    """Page sizes, head dims and group sizes inside and outside the tensor-core kernel's
    coverage (pages of 4 and head_dim 96 take the scalar kernel)."""
    Hkv = 2
    cos, sin = oracle.build_rope_tables(600, D, base=1e6, dtype=dtype)
    cpu = workloads.make_paged_batch("cov", B=5, Hq=Hkv * G, Hkv=Hkv, D=D, block_size=bs, ctx_range=(1, 500),
                                     dtype=dtype, seed=bs + G, tables=(cos, sin))
    q_rot, kc, vc, ref = _oracle_step(cpu, cos, sin)
    gpu = cpu.to(DEV)
    ws = PagedWorkspace(DEV)
    out = paged_decode_step(gpu.q_new, gpu.k_new, gpu.v_new, gpu.k_cache, gpu.v_cache, gpu.block_table,
                            gpu.context_lens, gpu.slot_mapping, gpu.positions, gpu.cos, gpu.sin, workspace=ws)
    _clean(ws)
    assert torch.equal(gpu.k_cache.cpu(), kc) and torch.equal(gpu.v_cache.cpu(), vc)
    torch.testing.assert_close(out.cpu().float(), ref.float(), atol=TOL[dtype], rtol=TOL[dtype])


def test_stale_tail_and_nan_pages_do_not_leak(native):
    """Keys past a request's length share its last page; fill them (and unused pages) with
    NaN patterns and check that nothing reaches the output."""
    cos, sin = oracle.build_rope_tables(400, 128, base=1e6, dtype=torch.bfloat16)
    cpu = workloads.make_paged_batch("nan", B=4, Hq=16, Hkv=2, D=128, block_size=16, ctx_range=(3, 300), seed=9,
                                     tables=(cos, sin), num_blocks=128)
    for b in range(cpu.B):
        n = int(cpu.context_lens[b])
        page = int(cpu.block_table[b, (n - 1) // 16])
        if n % 16:
            cpu.k_cache[page, :, n % 16:] = float("nan")
            cpu.v_cache[page, :, n % 16:] = float("nan")
    unused = torch.ones(128, dtype=torch.bool)
    unused[cpu.block_table[cpu.block_table >= 0]] = False
    cpu.k_cache[unused] = float("nan")
    cpu.v_cache[unused] = float("nan")
    ref = oracle.paged_attention_composed(cpu.q_new, cpu.k_cache, cpu.v_cache, cpu.block_table, cpu.context_lens)
    gpu = cpu.to(DEV)
    for force in (False, True):
        out = paged_decode(gpu.q_new, gpu.k_cache, gpu.v_cache, gpu.block_table, gpu.context_lens, force_generic=force)
        assert torch.isfinite(out).all()
        torch.testing.assert_close(out.cpu().float(), ref.float(), atol=2e-2, rtol=2e-2)


def test_tensor_core_kernel_is_selected(native):
    """The benchmark shapes must run on the TMA/MMA kernel, the odd ones on the scalar one."""
    from kernels.attention import PagedAttentionCall
    def kind(dtype, bs, D, G, **kw):
        kc = torch.zeros(8, 2, bs, D, dtype=dtype, device=DEV)
        q = torch.zeros(3, 2 * G, D, dtype=dtype, device=DEV)
        bt = torch.zeros(3, 2, dtype=torch.int64, device=DEV)
        return PagedAttentionCall(q, kc, kc.clone(), bt, torch.ones(3, dtype=torch.int32, device=DEV), **kw).kernel_kind
    assert kind(torch.bfloat16, 16, 128, 8) == 1      # configuration 2
    assert kind(torch.bfloat16, 32, 128, 8) == 1      # configuration 4
    assert kind(torch.bfloat16, 16, 128, 7) == 1      # configuration 5's head ratio
    assert kind(torch.float16, 64, 64, 16) == 1
    assert kind(torch.float32, 16, 64, 1) == 0        # configuration 1 is fp32
    assert kind(torch.bfloat16, 4, 128, 8) == 0
    assert kind(torch.bfloat16, 16, 128, 8, force_generic=True) == 0


def test_empty_requests_give_zeros(native):
    kc = golden_io.pattern((8, 2, 16, 128), torch.bfloat16, 1).to(DEV)
    vc = golden_io.pattern((8, 2, 16, 128), torch.bfloat16, 2).to(DEV)
    bt = torch.arange(8, device=DEV).view(2, 4)
    q = golden_io.pattern((2, 8, 128), torch.bfloat16, 3).to(DEV)
    for force in (False, True):
        out = paged_decode(q, kc, vc, bt, torch.tensor([0, 20], dtype=torch.int32, device=DEV), force_generic=force)
        assert not out[0].any() and out[1].any()  # src/kernels/attention.cu:163: no keys -> zeros, never NaN


def test_chunked_prefill_mixed_batch(native):
    """Configuration 5 in small: ragged new-token chunks (decode rows among them) on a
    fragmented pool, 28/4 heads, bottom-right causal, after compacting some requests to new
    pages with kv_paged_scatter."""
    cos, sin = oracle.build_rope_tables(700, 128, base=1e6, dtype=torch.bfloat16)
    cpu = workloads.cfg5(scale=0.03, tables=(cos, sin), pool_pages=600)
    q_rot, kc, vc, ref = _oracle_step(cpu, cos, sin)
    gpu = cpu.to(DEV)
    rope_append(gpu.k_new, gpu.v_new, gpu.k_cache, gpu.v_cache, gpu.slot_mapping, gpu.positions, gpu.cos, gpu.sin)
    assert torch.equal(gpu.k_cache.cpu(), kc) and torch.equal(gpu.v_cache.cpu(), vc)
    # compaction: move request 0 onto fresh free pages (gather its rows, scatter to new slots)
    used = torch.zeros(600, dtype=torch.bool)
    used[cpu.block_table[cpu.block_table >= 0]] = True
    fresh = torch.nonzero(cpu.extra["free_mask"] & ~used).flatten()
    n0 = int(cpu.context_lens[0])
    npages = (n0 + 15) // 16
    if n0 > 0 and fresh.numel() >= npages:
        t = torch.arange(n0)
        old_slots = cpu.block_table[0, t // 16] * 16 + t % 16
        new_bt = cpu.block_table.clone()
        new_bt[0, :npages] = fresh[:npages]
        new_slots = new_bt[0, t // 16] * 16 + t % 16
        rows_k = kc.permute(0, 2, 1, 3).reshape(-1, 4, 128)[old_slots]
        rows_v = vc.permute(0, 2, 1, 3).reshape(-1, 4, 128)[old_slots]
        oracle.kv_paged_scatter(rows_k, rows_v, kc, vc, new_slots)
        kv_paged_scatter(rows_k.to(DEV), rows_v.to(DEV), gpu.k_cache, gpu.v_cache, new_slots.to(DEV))
        assert torch.equal(gpu.k_cache.cpu(), kc) and torch.equal(gpu.v_cache.cpu(), vc)
        cpu.block_table, gpu.block_table = new_bt, new_bt.to(DEV)
        ref2 = oracle.paged_attention_composed(q_rot, kc, vc, new_bt, cpu.context_lens, q_start=cpu.q_start.tolist())
        torch.testing.assert_close(ref2, ref)  # moving pages changes nothing
    ws = PagedWorkspace(DEV)
    out = paged_attention(gpu.q_new, gpu.k_cache, gpu.v_cache, gpu.block_table, gpu.context_lens, q_start=gpu.q_start,
                          max_q_len=cpu.max_q_len, rope_cos=gpu.cos, rope_sin=gpu.sin, rope_positions=gpu.positions,
                          workspace=ws)
    _clean(ws)
    torch.testing.assert_close(out.cpu().float(), ref.float(), atol=2e-2, rtol=2e-2)


def test_splitk_combine_matches_recurrence(native):
    g = torch.Generator().manual_seed(0)
    splits = [1, 3, 7, 2, 64]
    begin = torch.tensor([0] + list(torch.tensor(splits).cumsum(0)), dtype=torch.int32)
    P, D = int(begin[-1]), 128
    m = torch.randn(P, generator=g) * 4
    l = torch.rand(P, generator=g) * 50 + 0.1
    acc = torch.randn(P, D, generator=g) * 10
    m[4] = float("-inf"); l[4] = 0; acc[4] = 0  # an empty split among live ones
    out = splitk_combine(acc.to(DEV), m.to(DEV), l.to(DEV), begin.to(DEV))
    for r in range(len(splits)):
        s0, s1 = int(begin[r]), int(begin[r + 1])
        ref = oracle.merge_partials(m[s0:s1], l[s0:s1], acc[s0:s1])
        torch.testing.assert_close(out[r].cpu().double(), ref, atol=1e-5, rtol=1e-5)


def test_plan_reuse_across_layers(native):
    """One plan, several launches (layers): the combine re-arms the work counter."""
    cos, sin = oracle.build_rope_tables(1100, 128, base=1e6, dtype=torch.bfloat16)
    gpu = workloads.cfg2(scale=0.1, tables=(cos, sin)).to(DEV)
    ws = PagedWorkspace(DEV)
    first = paged_decode(gpu.q_new, gpu.k_cache, gpu.v_cache, gpu.block_table, gpu.context_lens, workspace=ws)
    for _ in range(3):
        again = paged_decode(gpu.q_new, gpu.k_cache, gpu.v_cache, gpu.block_table, gpu.context_lens, workspace=ws,
                             reuse_plan=True)
        assert torch.equal(first, again)
    _clean(ws)


def test_decode_step_is_cuda_graph_capturable(native):
    """The library neither allocates nor synchronises, so a whole decode step (RoPE + append,
    plan, partials, combine; the last three launched programmatically behind each other) can
    be captured once and replayed; new inputs are written into the same buffers."""
    from kernels.attention import PagedAttentionCall, RopeAppendCall
    cos, sin = oracle.build_rope_tables(1100, 128, base=1e6, dtype=torch.bfloat16)
    cpu = workloads.cfg2(scale=0.1, tables=(cos, sin))
    gpu = cpu.to(DEV)
    ws = PagedWorkspace(DEV)
    app = RopeAppendCall(gpu.k_new, gpu.v_new, gpu.k_cache, gpu.v_cache, gpu.slot_mapping, gpu.positions, gpu.cos, gpu.sin)
    att = PagedAttentionCall(gpu.q_new, gpu.k_cache, gpu.v_cache, gpu.block_table, gpu.context_lens, rope_cos=gpu.cos,
                             rope_sin=gpu.sin, rope_positions=gpu.positions, workspace=ws)
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        app.run(); att.run()          # first calls outside capture (function attributes, lazy module load)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            app.run()
            att.run()
    eager = att.out.clone()
    # replay on fresh queries: same buffers, new contents
    new_q = golden_io.pattern(tuple(gpu.q_new.shape), torch.bfloat16, 77).to(DEV)
    gpu.q_new.copy_(new_q)
    att.out.zero_()
    graph.replay()
    torch.cuda.synchronize()
    replayed = att.out.clone()
    app.run(); att.run()
    torch.cuda.synchronize()
    assert torch.equal(replayed, att.out) and not torch.equal(replayed, eager)
    _clean(ws)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("interleaved", [False, True])
@pytest.mark.parametrize("force_generic", [False, True])
def test_fused_decode_step_rope_variants(dtype, interleaved, force_generic, native):
    """The fused step (RoPE + append, RoPE in the Q load) in both RoPE layouts and both 16-bit
    types, on the TMA/MMA kernel and on the scalar one: pool bit-exact against the reference's
    op-by-op rounding, outputs within the type's tolerance."""
    cos, sin = oracle.build_rope_tables(700, 128, base=1e6, dtype=dtype, interleaved=interleaved)
    cpu = workloads.make_paged_batch("variants", B=5, Hq=16, Hkv=4, D=128, block_size=16, ctx_range=(1, 600),
                                     num_blocks=256, dtype=dtype, seed=41, tables=(cos, sin))
    g = cpu.to(DEV)
    ws = PagedWorkspace(DEV)
    out = paged_decode_step(g.q_new, g.k_new, g.v_new, g.k_cache, g.v_cache, g.block_table, g.context_lens,
                            g.slot_mapping, g.positions, g.cos, g.sin, interleaved=interleaved, workspace=ws,
                            force_generic=force_generic)
    assert ws.status() == 0
    pos = cpu.positions.long()
    q_rot = oracle.apply_rope(cpu.q_new.unsqueeze(0), cos[pos], sin[pos], interleaved=interleaved)[0]
    k_rot = oracle.apply_rope(cpu.k_new.unsqueeze(0), cos[pos], sin[pos], interleaved=interleaved)[0]
    oracle.kv_paged_append(k_rot, cpu.v_new, cpu.k_cache, cpu.v_cache, cpu.slot_mapping)
    assert torch.equal(g.k_cache.cpu(), cpu.k_cache) and torch.equal(g.v_cache.cpu(), cpu.v_cache)
    ref = oracle.paged_attention_composed(q_rot, cpu.k_cache, cpu.v_cache, cpu.block_table, cpu.context_lens)
    torch.testing.assert_close(out.cpu().float(), ref.float(), atol=TOL[dtype], rtol=TOL[dtype])
