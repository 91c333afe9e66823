"""The benchmark configurations at the full size of one or two of their requests, compared with
the CPU oracle through the C ABI: a 2048-token causal prefill (32/8 heads), decode rows over
32 768 keys (64/8 heads, pages of 32) and over 8192 keys (16/2 heads, pages of 16), and a
64-token chunk behind a 16 k context on a fragmented pool (28/4 heads). The shapes follow the
reference's own parity grid, tests/test_attention_parity.py:37-78 (its decode-like (1, 2048) and
2048-square prefill cases), at the sizes the configurations state. Pool contents bit-exact,
outputs within 2e-2 (bf16)."""
from __future__ import annotations

import pytest
import torch

import oracle
import workloads
from kernels.attention import PagedAttentionCall, PagedWorkspace, paged_decode_step, rope_append

pytestmark = [pytest.mark.gpu]
DEV = "cuda"
TOL = 2e-2  # bf16, kernels/_common/dtype.py:47-52


def _oracle(cpu):
    pos = cpu.positions.long()
    q_rot = oracle.apply_rope(cpu.q_new.unsqueeze(0), cpu.cos[pos], cpu.sin[pos])[0]
    k_rot = oracle.apply_rope(cpu.k_new.unsqueeze(0), cpu.cos[pos], cpu.sin[pos])[0]
    kc, vc = cpu.k_cache.clone(), cpu.v_cache.clone()
    oracle.kv_paged_append(k_rot, cpu.v_new, kc, vc, cpu.slot_mapping)
    qs = None if cpu.max_q_len == 1 else cpu.q_start.tolist()
    return q_rot, kc, vc, oracle.paged_attention_composed(q_rot, kc, vc, cpu.block_table, cpu.context_lens, q_start=qs)


def test_cfg3_one_request_of_2048_tokens(native):
    cos, sin = oracle.build_rope_tables(2049, 128, base=1e6, dtype=torch.bfloat16)
    cpu = workloads.cfg3(scale=0.125, seq=2048, tables=(cos, sin))  # 1 request x 2048 new tokens, empty cache
    assert cpu.B == 1 and cpu.n_tokens == 2048
    q_rot, kc, vc, ref = _oracle(cpu)
    g = cpu.to(DEV)
    q_gpu = rope_append(g.k_new, g.v_new, g.k_cache, g.v_cache, g.slot_mapping, g.positions, g.cos, g.sin, q=g.q_new)
    assert torch.equal(q_gpu.cpu(), q_rot)
    assert torch.equal(g.k_cache.cpu(), kc) and torch.equal(g.v_cache.cpu(), vc)
    ws = PagedWorkspace(DEV)
    call = PagedAttentionCall(q_gpu, g.k_cache, g.v_cache, g.block_table, g.context_lens, q_start=g.q_start,
                              max_q_len=cpu.max_q_len, workspace=ws)
    assert call.kernel_kind == 2
    out = call.run()
    assert ws.status() == 0
    torch.testing.assert_close(out.cpu().float(), ref.float(), atol=TOL, rtol=TOL)


@pytest.mark.parametrize("cfg", ["cfg4", "cfg2"])
def test_decode_requests_at_full_context(cfg, native):
    if cfg == "cfg4":
        shape = dict(Hq=64, Hkv=8, block_size=32, ctx_range=(32767, 32767))  # + 1 new token = 32 768 keys
    else:
        shape = dict(Hq=16, Hkv=2, block_size=16, ctx_range=(8191, 8191))
    rows = shape["ctx_range"][1] + 2
    cos, sin = oracle.build_rope_tables(rows, 128, base=1e6, dtype=torch.bfloat16)
    cpu = workloads.make_paged_batch(cfg, B=2, D=128, theta=1e6, seed=7, tables=(cos, sin), **shape)
    q_rot, kc, vc, ref = _oracle(cpu)
    g = cpu.to(DEV)
    ws = PagedWorkspace(DEV)
    out = paged_decode_step(g.q_new, g.k_new, g.v_new, g.k_cache, g.v_cache, g.block_table, g.context_lens,
                            g.slot_mapping, g.positions, g.cos, g.sin, workspace=ws)
    assert ws.status() == 0
    assert torch.equal(g.k_cache.cpu(), kc) and torch.equal(g.v_cache.cpu(), vc)
    torch.testing.assert_close(out.cpu().float(), ref.float(), atol=TOL, rtol=TOL)


def test_cfg5_chunk_of_64_tokens_behind_a_16k_context(native):
    cos, sin = oracle.build_rope_tables(16384 + 65, 128, base=1e6, dtype=torch.bfloat16)
    cpu = workloads.make_paged_batch("cfg5", B=2, Hq=28, Hkv=4, D=128, block_size=16, ctx_range=(16320, 16384),
                                     new_range=(64, 64), num_blocks=8192, free_fraction=0.4, theta=1e6, seed=9,
                                     tables=(cos, sin))
    q_rot, kc, vc, ref = _oracle(cpu)
    g = cpu.to(DEV)
    q_gpu = rope_append(g.k_new, g.v_new, g.k_cache, g.v_cache, g.slot_mapping, g.positions, g.cos, g.sin, q=g.q_new)
    assert torch.equal(q_gpu.cpu(), q_rot)
    assert torch.equal(g.k_cache.cpu(), kc) and torch.equal(g.v_cache.cpu(), vc)
    ws = PagedWorkspace(DEV)
    call = PagedAttentionCall(q_gpu, g.k_cache, g.v_cache, g.block_table, g.context_lens, q_start=g.q_start,
                              max_q_len=cpu.max_q_len, workspace=ws)
    assert call.kernel_kind == 3  # split over the keys; the decode kernel in front finds no one-row request and returns
    out = call.run()
    assert ws.status() == 0
    torch.testing.assert_close(out.cpu().float(), ref.float(), atol=TOL, rtol=TOL)
