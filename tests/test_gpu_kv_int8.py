"""int8 KV with one fp32 scale per (position, kv head): the reference's `kv_int8` /
`k_scales[kv_pos * n_kv_heads + kv_head]` (src/kernels/attention.cu:91-96,141-150,
include/reflex/infer.h:189-203) on pages. The quantising append is held bit for bit to the
oracle's quantiser (pool bytes and scales), the decode kernel's int8 instantiation and the
scalar kernel to float32 attention over the dequantised pool, at the bf16 / fp16 tolerance."""
from __future__ import annotations

import pytest
import torch

import oracle
import workloads
from kernels.attention import PagedAttentionCall, PagedWorkspace, int8_pool, paged_attention, paged_decode_step, rope_append

pytestmark = [pytest.mark.gpu]
DEV = "cuda"
TOL = {torch.bfloat16: 2e-2, torch.float16: 5e-3}


def _quantised_copy(cpu):
    """The batch's 16-bit pool quantised row by row (oracle), as (k int8, v int8, k scales, v scales)."""
    kq, ks = oracle.kv_quantize_rows(cpu.k_cache)
    vq, vs = oracle.kv_quantize_rows(cpu.v_cache)
    return kq, vq, ks, vs


def _oracle_step(cpu, kq, vq, ks, vs):
    """Rotate, quantising append, then float32 attention over the dequantised pool."""
    pos = cpu.positions.long()
    q_rot = oracle.apply_rope(cpu.q_new.unsqueeze(0), cpu.cos[pos], cpu.sin[pos])[0]
    k_rot = oracle.apply_rope(cpu.k_new.unsqueeze(0), cpu.cos[pos], cpu.sin[pos])[0]
    oracle.kv_paged_append_q8(k_rot, cpu.v_new, kq, vq, ks, vs, cpu.slot_mapping)
    qs = None if cpu.max_q_len == 1 else cpu.q_start.tolist()
    ref = oracle.paged_attention_composed(q_rot.float(), oracle.kv_dequantize(kq, ks), oracle.kv_dequantize(vq, vs),
                                          cpu.block_table, cpu.context_lens, q_start=qs)
    return q_rot, ref


@pytest.mark.parametrize("dtype,bs,G,inter", [(torch.bfloat16, 16, 8, False), (torch.bfloat16, 32, 8, False),
                                              (torch.float16, 8, 4, True), (torch.bfloat16, 64, 16, False),
                                              (torch.bfloat16, 128, 1, False)])
def test_decode_step_on_an_int8_pool(dtype, bs, G, inter, native):
    Hkv = 2
    cos, sin = oracle.build_rope_tables(900, 128, base=1e6, dtype=dtype, interleaved=inter)
    cpu = workloads.make_paged_batch("q8", B=6, Hq=Hkv * G, Hkv=Hkv, D=128, block_size=bs, ctx_range=(1, 800),
                                     dtype=dtype, seed=bs + G, tables=(cos, sin))
    kq, vq, ks, vs = _quantised_copy(cpu)
    # poison what no request owns: unused pages, and the tails of last pages (bytes and scales)
    used = torch.zeros(cpu.num_blocks, dtype=torch.bool)
    used[cpu.block_table[cpu.block_table >= 0]] = True
    ks[~used] = float("nan"); vs[~used] = float("nan")
    for b in range(cpu.B):
        n = int(cpu.context_lens[b])
        if n % bs:
            page = int(cpu.block_table[b, (n - 1) // bs])
            ks[page, :, n % bs:] = float("nan"); vs[page, :, n % bs:] = float("nan")
    g = cpu.to(DEV)
    kq_g, vq_g, ks_g, vs_g = kq.to(DEV), vq.to(DEV), ks.to(DEV), vs.to(DEV)
    if inter:
        pos = cpu.positions.long()
        q_rot = oracle.apply_rope(cpu.q_new.unsqueeze(0), cos[pos], sin[pos], interleaved=True)[0]
        k_rot = oracle.apply_rope(cpu.k_new.unsqueeze(0), cos[pos], sin[pos], interleaved=True)[0]
        oracle.kv_paged_append_q8(k_rot, cpu.v_new, kq, vq, ks, vs, cpu.slot_mapping)
        ref = oracle.paged_attention_composed(q_rot.float(), oracle.kv_dequantize(kq, ks).nan_to_num(0.0),
                                              oracle.kv_dequantize(vq, vs).nan_to_num(0.0), cpu.block_table,
                                              cpu.context_lens)
    else:
        q_rot, _ = _oracle_step(cpu, kq, vq, ks, vs)
        ref = oracle.paged_attention_composed(q_rot.float(), oracle.kv_dequantize(kq, ks).nan_to_num(0.0),
                                              oracle.kv_dequantize(vq, vs).nan_to_num(0.0), cpu.block_table,
                                              cpu.context_lens)
    ws = PagedWorkspace(DEV)
    out = paged_decode_step(g.q_new, g.k_new, g.v_new, kq_g, vq_g, g.block_table, g.context_lens, g.slot_mapping,
                            g.positions, g.cos, g.sin, interleaved=inter, workspace=ws, k_scales=ks_g, v_scales=vs_g)
    assert ws.status() == 0
    # the pool: bytes and scales bit for bit (NaN poison compares equal through the bit pattern)
    assert torch.equal(kq_g.cpu(), kq) and torch.equal(vq_g.cpu(), vq)
    assert torch.equal(ks_g.cpu().view(torch.int32), ks.view(torch.int32))
    assert torch.equal(vs_g.cpu().view(torch.int32), vs.view(torch.int32))
    assert torch.isfinite(out).all()
    torch.testing.assert_close(out.cpu().float(), ref, atol=TOL[dtype], rtol=TOL[dtype])
    # the scalar kernel on the same pool
    out_s = paged_attention(g.q_new, kq_g, vq_g, g.block_table, g.context_lens, rope_cos=g.cos, rope_sin=g.sin,
                            rope_positions=g.positions, rope_interleaved=inter, k_scales=ks_g, v_scales=vs_g,
                            force_generic=True)
    torch.testing.assert_close(out_s.cpu().float(), ref, atol=TOL[dtype], rtol=TOL[dtype])


def test_int8_kernel_selection_and_errors(native):
    k, v, ks, vs = int8_pool(64, 2, 16, 128, DEV)
    q = torch.zeros(4, 16, 128, dtype=torch.bfloat16, device=DEV)
    bt = torch.zeros(4, 8, dtype=torch.int64, device=DEV)
    cl = torch.full((4,), 20, dtype=torch.int32, device=DEV)
    assert PagedAttentionCall(q, k, v, bt, cl, k_scales=ks, v_scales=vs).kernel_kind == 1
    qs = torch.tensor([0, 1, 2, 3, 4], dtype=torch.int32, device=DEV)
    assert PagedAttentionCall(q, k, v, bt, cl, q_start=qs, k_scales=ks, v_scales=vs).kernel_kind == 0  # chunks: scalar
    with pytest.raises(ValueError, match="int8 pool needs"):
        PagedAttentionCall(q, k, v, bt, cl)
    with pytest.raises(ValueError, match="scales must be"):
        PagedAttentionCall(q, k, v, bt, cl, k_scales=ks[:, :, :8], v_scales=vs)
    k64, v64, ks64, vs64 = int8_pool(64, 2, 16, 64, DEV)
    q64 = torch.zeros(4, 16, 64, dtype=torch.bfloat16, device=DEV)
    assert PagedAttentionCall(q64, k64, v64, bt, cl, k_scales=ks64, v_scales=vs64).kernel_kind == 0


def test_chunked_queries_on_an_int8_pool_scalar_kernel(native):
    cos, sin = oracle.build_rope_tables(500, 128, base=1e6, dtype=torch.bfloat16)
    cpu = workloads.make_paged_batch("q8c", B=3, Hq=8, Hkv=2, D=128, block_size=16, ctx_range=(50, 400),
                                     new_range=(3, 9), num_blocks=128, seed=3, tables=(cos, sin))
    kq, vq, ks, vs = _quantised_copy(cpu)
    q_rot, ref = _oracle_step(cpu, kq, vq, ks, vs)
    g = cpu.to(DEV)
    kq_g, vq_g, ks_g, vs_g = (t.to(DEV) for t in _quantised_copy(cpu))
    q_gpu = rope_append(g.k_new, g.v_new, kq_g, vq_g, g.slot_mapping, g.positions, g.cos, g.sin, q=g.q_new,
                        k_scales=ks_g, v_scales=vs_g)
    assert torch.equal(q_gpu.cpu(), q_rot)
    assert torch.equal(kq_g.cpu(), kq) and torch.equal(ks_g.cpu(), ks) and torch.equal(vs_g.cpu(), vs)
    out = paged_attention(q_gpu, kq_g, vq_g, g.block_table, g.context_lens, q_start=g.q_start,
                          max_q_len=cpu.max_q_len, k_scales=ks_g, v_scales=vs_g)
    torch.testing.assert_close(out.cpu().float(), ref, atol=2e-2, rtol=2e-2)
