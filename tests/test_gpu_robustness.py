"""What the paged kernels do with inputs that break their contract, through the C ABI:
a page index outside the pool (its keys are left out, by every kernel alike, and status
bit 1 is raised) and row counts on the device that exceed what the host sized the workspace
for (nothing is computed, nothing is written past the workspace, status bit 2)."""
from __future__ import annotations

import pytest
import torch

import oracle
import workloads
from kernels.attention import PagedAttentionCall, PagedWorkspace, paged_attention

pytestmark = [pytest.mark.gpu]
DEV = "cuda"
BAD_PAGE, CAPACITY = 2, 4


def _without_page(cpu, q_rot, kc, vc, req, blk):
    """Oracle output when logical block `blk` of request `req` does not exist: its keys are taken
    out of the key sequence (bottom-right causal masking keeps the positions of the others)."""
    bs = cpu.block_size
    out = oracle.paged_attention_composed(q_rot, kc, vc, cpu.block_table, cpu.context_lens,
                                          q_start=None if cpu.max_q_len == 1 else cpu.q_start.tolist())
    ctx = int(cpu.context_lens[req])
    kd, vd = oracle.kv_paged_lookup(kc, vc, cpu.block_table[req:req + 1], cpu.context_lens[req:req + 1], ctx)
    r0, r1 = (req, req + 1) if cpu.max_q_len == 1 else (int(cpu.q_start[req]), int(cpu.q_start[req + 1]))
    n = r1 - r0
    mask = torch.zeros(n, ctx)
    if n > 1:
        mask = oracle.bottom_right_mask(n, ctx, dtype=torch.float32).clone()
    mask[:, blk * bs:min(ctx, (blk + 1) * bs)] = float("-inf")
    qb = q_rot[r0:r1].transpose(0, 1).unsqueeze(0)
    out[r0:r1] = oracle.naive_attention_f64(qb, kd, vd, mask=mask)[0].transpose(0, 1).to(out.dtype)
    return out


@pytest.mark.parametrize("mode", ["decode", "chunks_split", "chunks_whole"])
def test_page_index_outside_the_pool_is_left_out_by_every_kernel(mode, native):
    cos, sin = oracle.build_rope_tables(1000, 128, base=1e6, dtype=torch.bfloat16)
    if mode == "decode":
        cpu = workloads.make_paged_batch("bad", B=4, Hq=16, Hkv=2, D=128, block_size=16, ctx_range=(200, 700),
                                         num_blocks=512, seed=31, tables=(cos, sin))
    else:
        cpu = workloads.make_paged_batch("bad", B=3, Hq=8, Hkv=2, D=128, block_size=16, ctx_range=(200, 700),
                                         new_range=(20, 40), num_blocks=512, seed=32, tables=(cos, sin))
    pos = cpu.positions.long()
    q_rot = oracle.apply_rope(cpu.q_new.unsqueeze(0), cos[pos], sin[pos])[0]
    k_rot = oracle.apply_rope(cpu.k_new.unsqueeze(0), cos[pos], sin[pos])[0]
    kc, vc = cpu.k_cache.clone(), cpu.v_cache.clone()
    oracle.kv_paged_append(k_rot, cpu.v_new, kc, vc, cpu.slot_mapping)
    req, blk = 1, 3  # block 3 of request 1: keys 48..63, well inside its context
    want = _without_page(cpu, q_rot, kc, vc, req, blk)
    table = cpu.block_table.clone()
    table[req, blk] = cpu.num_blocks + 7
    kw = {} if mode == "decode" else dict(q_start=cpu.q_start.to(DEV), max_q_len=cpu.max_q_len)
    if mode == "chunks_whole":
        kw["target_chunk"] = -1
    outs = {}
    for generic in (False, True):
        ws = PagedWorkspace(DEV)
        call = PagedAttentionCall(q_rot.to(DEV), kc.to(DEV), vc.to(DEV), table.to(DEV), cpu.context_lens.to(DEV),
                                  workspace=ws, force_generic=generic, **kw)
        if not generic:
            assert call.kernel_kind == {"decode": 1, "chunks_whole": 2}.get(mode, 3)
        out = call.run()
        assert ws.status() & BAD_PAGE, "the bad page must be reported"
        assert torch.isfinite(out).all()
        torch.testing.assert_close(out.cpu().float(), want.float(), atol=2e-2, rtol=2e-2)
        outs[generic] = out
    torch.testing.assert_close(outs[False].float(), outs[True].float(), atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("force_generic", [False, True])
def test_understated_max_q_len_computes_nothing_and_says_so(force_generic, native):
    """A request with more query rows than the host's bound: the plan kernel leaves an empty plan,
    so no partial row is written anywhere, the combine writes zeros, and status bit 2 is set. The
    bytes right behind the workspace (where partial rows beyond the capacity would land) stay put."""
    cos, sin = oracle.build_rope_tables(1400, 128, base=1e6, dtype=torch.bfloat16)
    cpu = workloads.make_paged_batch("cap", B=4, Hq=8, Hkv=2, D=128, block_size=16, ctx_range=(900, 1100),
                                     new_range=(60, 64), num_blocks=512, seed=41, tables=(cos, sin))
    g = cpu.to(DEV)
    probe = PagedAttentionCall(g.q_new, g.k_cache, g.v_cache, g.block_table, g.context_lens, q_start=g.q_start,
                               max_q_len=1, force_generic=force_generic)
    need = probe.workspace.buffer.numel()
    # a workspace followed by canary bytes inside one allocation
    ws = PagedWorkspace(DEV)
    ws.buffer = torch.full((need + (1 << 20),), 0x5A, dtype=torch.uint8, device=DEV)
    call = PagedAttentionCall(g.q_new, g.k_cache, g.v_cache, g.block_table, g.context_lens, q_start=g.q_start,
                              max_q_len=1, workspace=ws, force_generic=force_generic)
    call._args.workspace_bytes = need  # what a caller with exactly the advertised size would pass
    out = call.run()
    torch.cuda.synchronize()
    assert ws.status() & CAPACITY
    assert torch.count_nonzero(out) == 0
    assert bool((ws.buffer[need:] == 0x5A).all()), "something was written past the workspace"
    # the default bound (the number of query rows) is always safe
    good = paged_attention(g.q_new, g.k_cache, g.v_cache, g.block_table, g.context_lens, q_start=g.q_start,
                           force_generic=force_generic)
    ref = oracle.paged_attention_composed(cpu.q_new, cpu.k_cache, cpu.v_cache, cpu.block_table, cpu.context_lens,
                                          q_start=cpu.q_start.tolist())
    torch.testing.assert_close(good.cpu().float(), ref.float(), atol=2e-2, rtol=2e-2)


def test_q_start_that_disagrees_with_the_row_count_is_refused(native):
    cos, sin = oracle.build_rope_tables(400, 128, base=1e6, dtype=torch.bfloat16)
    cpu = workloads.make_paged_batch("cap2", B=3, Hq=8, Hkv=2, D=128, block_size=16, ctx_range=(100, 300),
                                     new_range=(4, 9), num_blocks=128, seed=42, tables=(cos, sin))
    g = cpu.to(DEV)
    qs = g.q_start.clone()
    qs[-1] -= 1  # one row fewer than q has
    ws = PagedWorkspace(DEV)
    out = paged_attention(g.q_new, g.k_cache, g.v_cache, g.block_table, g.context_lens, q_start=qs,
                          max_q_len=cpu.max_q_len, workspace=ws)
    assert ws.status() & CAPACITY
    assert torch.count_nonzero(out) == 0


def test_whole_row_prefill_reports_rows_beyond_the_grid(native):
    """Long chunks run without plan and combine; the grid comes from max_q_len. Rows beyond it
    cannot be computed, and the kernel says so instead of leaving stale output silently."""
    S = 700
    g = torch.Generator(device=DEV).manual_seed(5)
    q = (torch.randn(S, 8, 128, device=DEV, generator=g) * 0.5).to(torch.bfloat16)
    kc = (torch.randn(S // 16 + 1, 2, 16, 128, device=DEV, generator=g) * 0.5).to(torch.bfloat16)
    vc = torch.randn_like(kc)
    bt = torch.arange(S // 16 + 1, device=DEV).view(1, -1)
    ws = PagedWorkspace(DEV)
    paged_attention(q, kc, vc, bt, torch.tensor([S], dtype=torch.int32, device=DEV),
                    q_start=torch.tensor([0, S], dtype=torch.int32, device=DEV), max_q_len=600, workspace=ws)
    assert ws.status() & CAPACITY
