"""GPU parity of the tcgen05 prefill kernel through the C ABI: dense causal prefill
(configuration 3 in small and at its full per-request size) and paged chunked prefill with
bottom-right causal masking (configuration 5 in small), against the CPU oracle."""
from __future__ import annotations

import pytest
import torch

import golden_io
import kernels.attention
import oracle
import workloads
from kernels.attention import PagedAttentionCall, PagedWorkspace, fused_attention, paged_attention, rope_append

pytestmark = [pytest.mark.gpu]
DEV = "cuda"


import contextlib


@contextlib.contextmanager
def _debug(native, words):
    """The library's debug switches for the duration of a block (rfx_debug_set_flags)."""
    native.lib().rfx_debug_set_flags(words.encode())
    try:
        yield
    finally:
        native.lib().rfx_debug_set_flags(None)


def _causal(n):
    return torch.triu(torch.full((n, n), float("-inf")), 1)


@pytest.mark.parametrize("B,H,Hkv,S,causal,dtype", [
    (1, 4, 4, 128, True, torch.bfloat16), (2, 8, 2, 300, True, torch.bfloat16), (1, 32, 8, 257, False, torch.bfloat16),
    (1, 6, 2, 130, True, torch.float16), (1, 7, 1, 64, True, torch.bfloat16), (1, 2, 2, 1000, True, torch.float16)])
def test_dense_prefill_vs_naive(B, H, Hkv, S, causal, dtype, native):
    q = golden_io.pattern((B, H, S, 128), dtype, 1, scale=0.5)
    k = golden_io.pattern((B, Hkv, S, 128), dtype, 2, scale=0.5)
    v = golden_io.pattern((B, Hkv, S, 128), dtype, 3)
    ref = oracle.naive_attention_f64(q, k, v, mask=_causal(S) if causal else None)
    o = fused_attention(q.to(DEV), k.to(DEV), v.to(DEV), is_causal=causal)
    tol = 2e-2 if dtype == torch.bfloat16 else 5e-3
    torch.testing.assert_close(o.cpu().double(), ref, atol=tol, rtol=tol)
    # and against the reference's own path (SDPA after GQA expansion) at its tolerance
    torch.testing.assert_close(o.cpu().float(), oracle.attention(q, k, v, is_causal=causal).float(), atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("B,H,Hkv,Sq,Sk,causal,dtype", [
    (2, 8, 2, 256, 256, False, torch.bfloat16),   # aligned rows of the mask: 16-byte loads
    (1, 8, 2, 300, 300, True, torch.bfloat16),    # ragged last tile, mask and causal together
    (1, 4, 4, 128, 517, False, torch.float16),    # odd key count: element loads
    (1, 32, 8, 70, 200, False, torch.bfloat16)])
def test_dense_additive_mask_on_tensor_core_kernel(B, H, Hkv, Sq, Sk, causal, dtype, native, monkeypatch):
    """`attn_mask` [B, H, S_q, S_k] added to the scaled scores (reference triton_fused_attention.py:190-202)
    on the tcgen05 kernel: a smooth bias, a band of -inf entries, and a boolean mask; cross-checked
    against the scalar kernel."""
    q = golden_io.pattern((B, H, Sq, 128), dtype, 11, scale=0.5)
    k = golden_io.pattern((B, Hkv, Sk, 128), dtype, 12, scale=0.5)
    v = golden_io.pattern((B, Hkv, Sk, 128), dtype, 13)
    bias = golden_io.pattern((B, H, Sq, Sk), dtype, 14, scale=2.0)
    far = (torch.arange(Sk).view(1, -1) - torch.arange(Sq).view(-1, 1)).abs() > 96   # keep a band around the diagonal
    far[:, 0] = False                                                                 # every row keeps a key
    bias = bias.masked_fill(far.view(1, 1, Sq, Sk), float("-inf"))
    tol = 2e-2 if dtype == torch.bfloat16 else 5e-3
    full = bias.double() + (_causal(Sq) if causal else 0.0)
    ref = oracle.naive_attention_f64(q, k, v, mask=full)
    o = fused_attention(q.to(DEV), k.to(DEV), v.to(DEV), attn_mask=bias.to(DEV), is_causal=causal)
    assert kernels.attention.last_dense_kernel_kind == 1
    torch.testing.assert_close(o.cpu().double(), ref, atol=tol, rtol=tol)
    keep = ~far.view(1, 1, Sq, Sk).expand(B, H, Sq, Sk)
    ob = fused_attention(q.to(DEV), k.to(DEV), v.to(DEV), attn_mask=keep.to(DEV), is_causal=causal)
    refb = oracle.naive_attention_f64(q, k, v, mask=torch.zeros(Sq, Sk).masked_fill(far, float("-inf")).double()
                                      + (_causal(Sq) if causal else 0.0))
    torch.testing.assert_close(ob.cpu().double(), refb, atol=tol, rtol=tol)
    with _debug(native, "no_tc"):
        os_ = fused_attention(q.to(DEV), k.to(DEV), v.to(DEV), attn_mask=bias.to(DEV), is_causal=causal)
        assert kernels.attention.last_dense_kernel_kind == 0
    torch.testing.assert_close(o.float(), os_.float(), atol=tol, rtol=tol)


def test_dense_prefill_matches_scalar_kernel(native, monkeypatch):
    q = golden_io.pattern((1, 8, 384, 128), torch.bfloat16, 4, scale=0.5).to(DEV)
    k = golden_io.pattern((1, 2, 384, 128), torch.bfloat16, 5, scale=0.5).to(DEV)
    v = golden_io.pattern((1, 2, 384, 128), torch.bfloat16, 6).to(DEV)
    a = fused_attention(q, k, v, is_causal=True)
    with _debug(native, "no_tc"):
        b = fused_attention(q, k, v, is_causal=True)
    torch.testing.assert_close(a.float(), b.float(), atol=2e-2, rtol=2e-2)


def test_cfg3_paged_prefill_small_and_kv_bit_exact(native):
    """Configuration 3 scaled down: empty cache, bulk RoPE + append of every new token, then
    causal attention straight from the pool on the tensor-core kernel."""
    cos, sin = oracle.build_rope_tables(400, 128, base=1e6, dtype=torch.bfloat16)
    cpu = workloads.cfg3(scale=0.15, tables=(cos, sin))  # 1 request x 307 tokens, 32/8 heads
    pos = cpu.positions.long()
    q_rot = oracle.apply_rope(cpu.q_new.unsqueeze(0), cos[pos], sin[pos])[0]
    k_rot = oracle.apply_rope(cpu.k_new.unsqueeze(0), cos[pos], sin[pos])[0]
    kc, vc = cpu.k_cache.clone(), cpu.v_cache.clone()
    oracle.kv_paged_append(k_rot, cpu.v_new, kc, vc, cpu.slot_mapping)
    ref = oracle.paged_attention_composed(q_rot, kc, vc, cpu.block_table, cpu.context_lens, q_start=cpu.q_start.tolist())
    gpu = cpu.to(DEV)
    q_gpu = rope_append(gpu.k_new, gpu.v_new, gpu.k_cache, gpu.v_cache, gpu.slot_mapping, gpu.positions, gpu.cos,
                        gpu.sin, q=gpu.q_new)
    assert torch.equal(gpu.k_cache.cpu(), kc) and torch.equal(gpu.v_cache.cpu(), vc)
    assert torch.equal(q_gpu.cpu(), q_rot)
    ws = PagedWorkspace(DEV)
    call = PagedAttentionCall(q_gpu, gpu.k_cache, gpu.v_cache, gpu.block_table, gpu.context_lens, q_start=gpu.q_start,
                              max_q_len=cpu.max_q_len, workspace=ws)
    assert call.kernel_kind in (2, 3)  # 3: split over the keys, one-row requests on the decode kernel
    out = call.run()
    assert ws.status() == 0
    torch.testing.assert_close(out.cpu().float(), ref.float(), atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("bs", [8, 16, 64, 128, 256])
def test_chunked_prefill_mixed_batch_tensor_core(bs, native, monkeypatch):
    """Configuration 5 in small on the tensor-core kernel: ragged chunks with decode rows among
    them, 28/4 heads (group of 7: 18 tokens x 7 heads per tile), existing contexts, several page
    sizes; cross-checked against the scalar kernel too."""
    cos, sin = oracle.build_rope_tables(900, 128, base=1e6, dtype=torch.bfloat16)
    cpu = workloads.make_paged_batch("mix", B=5, Hq=28, Hkv=4, D=128, block_size=bs, ctx_range=(0, 700),
                                     new_range=(1, 64), decode_fraction=0.4, num_blocks=max(64, 6000 // bs),
                                     free_fraction=0.6, seed=bs, tables=(cos, sin))
    pos = cpu.positions.long()
    q_rot = oracle.apply_rope(cpu.q_new.unsqueeze(0), cos[pos], sin[pos])[0]
    k_rot = oracle.apply_rope(cpu.k_new.unsqueeze(0), cos[pos], sin[pos])[0]
    kc, vc = cpu.k_cache.clone(), cpu.v_cache.clone()
    oracle.kv_paged_append(k_rot, cpu.v_new, kc, vc, cpu.slot_mapping)
    # poison everything the requests do not own: unused pages and the tails of last pages
    used = torch.zeros(cpu.num_blocks, dtype=torch.bool)
    used[cpu.block_table[cpu.block_table >= 0]] = True
    kc[~used] = float("nan"); vc[~used] = float("nan")
    for b in range(cpu.B):
        n = int(cpu.context_lens[b])
        if n % bs:
            page = int(cpu.block_table[b, (n - 1) // bs])
            kc[page, :, n % bs:] = float("nan"); vc[page, :, n % bs:] = float("nan")
    ref = oracle.paged_attention_composed(q_rot, kc, vc, cpu.block_table, cpu.context_lens, q_start=cpu.q_start.tolist())
    g = cpu.to(DEV)
    ws = PagedWorkspace(DEV)
    kw = dict(q_start=g.q_start, max_q_len=cpu.max_q_len, workspace=ws)
    out = paged_attention(q_rot.to(DEV), kc.to(DEV), vc.to(DEV), g.block_table, g.context_lens, **kw)
    assert ws.status() == 0 and torch.isfinite(out).all()
    torch.testing.assert_close(out.cpu().float(), ref.float(), atol=2e-2, rtol=2e-2)
    out_s = paged_attention(q_rot.to(DEV), kc.to(DEV), vc.to(DEV), g.block_table, g.context_lens, force_generic=True, **kw)
    torch.testing.assert_close(out.float(), out_s.float(), atol=2e-2, rtol=2e-2)
    # key ranges cut at other places (192-key pieces) and not cut at all (whole rows per CTA)
    for chunk in (192, -1):
        out_c = paged_attention(q_rot.to(DEV), kc.to(DEV), vc.to(DEV), g.block_table, g.context_lens,
                                target_chunk=chunk, **kw)
        assert ws.status() == 0 and torch.isfinite(out_c).all()
        torch.testing.assert_close(out_c.cpu().float(), ref.float(), atol=2e-2, rtol=2e-2)
    # the one-row requests handed to the decode kernel (the default for a split batch), and kept on the
    # tensor-core kernel
    for words, kind in (("mixed=1", 3), ("mixed=0", 2)):
        with _debug(native, words):
            call = PagedAttentionCall(q_rot.to(DEV), kc.to(DEV), vc.to(DEV), g.block_table, g.context_lens, **kw)
            if bs <= 64:
                assert call.kernel_kind == kind
            out_m = call.run()
        assert ws.status() == 0
        torch.testing.assert_close(out_m.cpu().float(), ref.float(), atol=2e-2, rtol=2e-2)


def test_decode_heavy_mixed_batch_hands_rows_to_decode_kernel(native):
    """Twenty decode rows and two chunks in one batch: the decode rows run on the TMA/MMA decode
    kernel, the chunks on the tensor-core kernel, one combine merges both kinds of partials."""
    cos, sin = oracle.build_rope_tables(1200, 128, base=1e6, dtype=torch.bfloat16)
    cpu = workloads.make_paged_batch("heavy", B=22, Hq=16, Hkv=2, D=128, block_size=16, ctx_range=(30, 1000),
                                     new_range=(20, 21), decode_fraction=0.91, num_blocks=2048, seed=77, tables=(cos, sin))
    assert cpu.n_tokens <= 4 * cpu.B
    pos = cpu.positions.long()
    q_rot = oracle.apply_rope(cpu.q_new.unsqueeze(0), cos[pos], sin[pos])[0]
    k_rot = oracle.apply_rope(cpu.k_new.unsqueeze(0), cos[pos], sin[pos])[0]
    kc, vc = cpu.k_cache.clone(), cpu.v_cache.clone()
    oracle.kv_paged_append(k_rot, cpu.v_new, kc, vc, cpu.slot_mapping)
    ref = oracle.paged_attention_composed(q_rot, kc, vc, cpu.block_table, cpu.context_lens, q_start=cpu.q_start.tolist())
    g = cpu.to(DEV)
    ws = PagedWorkspace(DEV)
    call = PagedAttentionCall(q_rot.to(DEV), kc.to(DEV), vc.to(DEV), g.block_table, g.context_lens, q_start=g.q_start,
                              max_q_len=cpu.max_q_len, workspace=ws)
    assert call.kernel_kind == 3
    out = call.run()
    assert ws.status() == 0
    torch.testing.assert_close(out.cpu().float(), ref.float(), atol=2e-2, rtol=2e-2)


def test_cfg3_full_request_properties(native):
    """One request of configuration 3 at full length (2048 tokens, 32/8 heads): row 0 attends
    only key 0 (output = V[0] exactly), and the output is invariant to where the pages sit."""
    g = torch.Generator(device=DEV).manual_seed(0)
    S, Hq, Hkv, bs = 2048, 32, 8, 16
    q = (torch.randn(S, Hq, 128, device=DEV, generator=g) * 0.5).to(torch.bfloat16)
    k = (torch.randn(S, Hkv, 128, device=DEV, generator=g) * 0.5).to(torch.bfloat16)
    v = (torch.randn(S, Hkv, 128, device=DEV, generator=g) * 0.5).to(torch.bfloat16)
    outs = []
    for seed in (1, 2):
        perm = torch.randperm(S // bs, device=DEV, generator=torch.Generator(device=DEV).manual_seed(seed))
        kc = torch.zeros(S // bs, Hkv, bs, 128, dtype=torch.bfloat16, device=DEV)
        vc = torch.zeros_like(kc)
        t = torch.arange(S, device=DEV)
        slots = perm[t // bs] * bs + t % bs
        from kernels.kv_cache import kv_paged_append
        kv_paged_append(k, v, kc, vc, slots)
        outs.append(paged_attention(q, kc, vc, perm.view(1, -1), torch.tensor([S], dtype=torch.int32, device=DEV),
                                    q_start=torch.tensor([0, S], dtype=torch.int32, device=DEV), max_q_len=S))
    assert torch.equal(outs[0], outs[1])
    want0 = v[0].repeat_interleave(Hq // Hkv, dim=0)
    assert torch.equal(outs[0][0], want0)
    dense = fused_attention(q.permute(1, 0, 2)[None].contiguous(), k.permute(1, 0, 2)[None].contiguous(),
                            v.permute(1, 0, 2)[None].contiguous(), is_causal=True)
    torch.testing.assert_close(dense[0].permute(1, 0, 2).float(), outs[0].float(), atol=2e-2, rtol=2e-2)
