"""GPU parity of the paged KV pool ops through the C ABI: golden vectors of the reference,
the reference's own test shapes, and edge cases. Everything here is bit-exact."""
from __future__ import annotations

import pytest
import torch

import golden_cases as gc
import golden_io
import oracle
from kernels.kv_cache import kv_paged_append, kv_paged_lookup, kv_paged_scatter

pytestmark = [pytest.mark.gpu]
DEV = "cuda"


@pytest.mark.parametrize("name", sorted(gc.kv_write_cases()))
def test_write_golden(name, native):
    c = gc.kv_write_cases()[name]
    _, meta = golden_io.load(name)
    kc, vc = c["k_cache0"].to(DEV), c["v_cache0"].to(DEV)
    fn = kv_paged_scatter if c["op"] == "scatter" else kv_paged_append
    fn(c["k_in"].to(DEV), c["v_in"].to(DEV), kc, vc, c["slots"].to(DEV))
    assert golden_io.digest(kc) == meta["k_digest"] and golden_io.digest(vc) == meta["v_digest"]


@pytest.mark.parametrize("name", sorted(gc.kv_lookup_cases()))
def test_lookup_golden(name, native):
    c = gc.kv_lookup_cases()[name]
    _, meta = golden_io.load(name)
    ko, vo = kv_paged_lookup(c["k_cache"].to(DEV), c["v_cache"].to(DEV), c["block_table"].to(DEV),
                             c["context_lens"].to(DEV), c["max_ctx"])
    assert golden_io.digest(ko) == meta["k_digest"] and golden_io.digest(vo) == meta["v_digest"]


def test_scatter_equals_append(native):  # reference tests/test_kv_cache.py:125-145
    N, H, D, bs, nb = 8, 4, 32, 8, 4
    k_in, v_in = golden_io.pattern((N, H, D), torch.float16, 1).to(DEV), golden_io.pattern((N, H, D), torch.float16, 2).to(DEV)
    slots = torch.tensor([3, 9, 0, 31, 17, 8, 25, 12], device=DEV)
    a = [torch.zeros(nb, H, bs, D, dtype=torch.float16, device=DEV) for _ in range(4)]
    kv_paged_append(k_in, v_in, a[0], a[1], slots)
    kv_paged_scatter(k_in, v_in, a[2], a[3], slots, backend="triton")  # backend= is accepted, not dispatched
    assert torch.equal(a[0], a[2]) and torch.equal(a[1], a[3])


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("D", [128, 20, 7])
def test_append_exhaustive_slots(native, dtype, D):
    """Every slot of a small pool, one at a time and all together, vs the oracle."""
    H, bs, nb = 2, 4, 5
    base_k, base_v = golden_io.pattern((nb, H, bs, D), dtype, 3), golden_io.pattern((nb, H, bs, D), dtype, 4)
    for slots in ([s] for s in range(nb * bs)):
        k_in, v_in = golden_io.pattern((1, H, D), dtype, 5 + slots[0]), golden_io.pattern((1, H, D), dtype, 50 + slots[0])
        kc, vc = base_k.clone(), base_v.clone()
        oracle.kv_paged_append(k_in, v_in, kc, vc, torch.tensor(slots))
        gk, gv = base_k.to(DEV), base_v.to(DEV)
        kv_paged_append(k_in.to(DEV), v_in.to(DEV), gk, gv, torch.tensor(slots, device=DEV))
        assert torch.equal(gk.cpu(), kc) and torch.equal(gv.cpu(), vc)
    slots = torch.arange(nb * bs).flip(0)
    k_in, v_in = golden_io.pattern((nb * bs, H, D), dtype, 6), golden_io.pattern((nb * bs, H, D), dtype, 7)
    kc, vc = base_k.clone(), base_v.clone()
    oracle.kv_paged_append(k_in, v_in, kc, vc, slots)
    gk, gv = base_k.to(DEV), base_v.to(DEV)
    kv_paged_append(k_in.to(DEV), v_in.to(DEV), gk, gv, slots.to(DEV))
    assert torch.equal(gk.cpu(), kc) and torch.equal(gv.cpu(), vc)


def test_append_strided_input_int32_slots_and_skips(native):
    N, H, D, bs, nb = 6, 3, 64, 16, 2
    big = golden_io.pattern((N, 2 * H, D), torch.bfloat16, 8)
    k_in, v_in = big[:, :H], big[:, H:]  # non-contiguous views, as a fused QKV projection produces
    slots = torch.tensor([5, -1, 17, 10_000, 31, 0], dtype=torch.int32)
    kc, vc = torch.zeros(nb, H, bs, D, dtype=torch.bfloat16), torch.zeros(nb, H, bs, D, dtype=torch.bfloat16)
    keep = (slots >= 0) & (slots < nb * bs)  # out-of-pool slots are skipped by the library
    oracle.kv_paged_append(k_in[keep], v_in[keep], kc, vc, slots[keep].long())
    gk, gv = torch.zeros_like(kc, device=DEV), torch.zeros_like(vc, device=DEV)
    kv_paged_append(k_in.to(DEV)[:, :], v_in.to(DEV), gk, gv, slots.to(DEV))
    assert torch.equal(gk.cpu(), kc) and torch.equal(gv.cpu(), vc)
    gbig = big.to(DEV)
    gk.zero_(); gv.zero_()
    kv_paged_append(gbig[:, :H], gbig[:, H:], gk, gv, slots.to(DEV))
    assert torch.equal(gk.cpu(), kc) and torch.equal(gv.cpu(), vc)


def test_append_empty_and_errors(native):
    kc = torch.zeros(2, 2, 4, 8, dtype=torch.bfloat16, device=DEV)
    vc = torch.zeros_like(kc)
    kv_paged_append(torch.zeros(0, 2, 8, dtype=torch.bfloat16, device=DEV), torch.zeros(0, 2, 8, dtype=torch.bfloat16, device=DEV),
                    kc, vc, torch.zeros(0, dtype=torch.int64, device=DEV))
    with pytest.raises(RuntimeError, match="dtype"):
        kv_paged_append(torch.zeros(1, 2, 8, device=DEV), torch.zeros(1, 2, 8, device=DEV), kc, vc,
                        torch.zeros(1, dtype=torch.int64, device=DEV))
    with pytest.raises(ValueError):
        kv_paged_append(torch.zeros(1, 3, 8, dtype=torch.bfloat16, device=DEV), torch.zeros(1, 3, 8, dtype=torch.bfloat16, device=DEV),
                        kc, vc, torch.zeros(1, dtype=torch.int64, device=DEV))


@pytest.mark.parametrize("bs", [1, 8, 16])
def test_lookup_page_boundaries(native, bs):
    """Lengths 0, 1, bs-1, bs, bs+1, ... against the oracle; K and V tails are zero."""
    H, D, nb = 3, 16, 64
    lens = sorted({0, 1, max(bs - 1, 0), bs, bs + 1, 3 * bs - 1, 3 * bs, 3 * bs + 1})
    B, max_ctx = len(lens), 3 * bs + 5
    kc, vc = golden_io.pattern((nb, H, bs, D), torch.bfloat16, 9), golden_io.pattern((nb, H, bs, D), torch.bfloat16, 10)
    bt = gc._perm(nb, 11)[: B * 4].view(B, 4)
    ctx = torch.tensor(lens, dtype=torch.int32)
    ko, vo = oracle.kv_paged_lookup(kc, vc, bt, ctx, max_ctx)
    gk, gv = kv_paged_lookup(kc.to(DEV), vc.to(DEV), bt.to(DEV), ctx.to(DEV), max_ctx)
    assert torch.equal(gk.cpu(), ko) and torch.equal(gv.cpu(), vo)
    for b, n in enumerate(lens):
        assert not gk[b, :, n:].any() and not gv[b, :, n:].any()


def test_roundtrip_append_then_lookup_large(native):
    """Size-independent property at a realistic size: append every token of a batch through
    a permuted page table, look it up, and get the inputs back."""
    H, D, bs, B, ctx = 8, 128, 16, 16, 1000
    nb = B * ((ctx + bs - 1) // bs)
    g = torch.Generator(device=DEV); g.manual_seed(0)
    perm = torch.randperm(nb, device=DEV, generator=g)
    bt = perm.view(B, -1)
    k = torch.randn(B, ctx, H, D, device=DEV, generator=g).to(torch.bfloat16)
    v = torch.randn(B, ctx, H, D, device=DEV, generator=g).to(torch.bfloat16)
    t = torch.arange(ctx, device=DEV)
    slots = (bt[:, t // bs] * bs + t % bs).reshape(-1)
    kc = torch.zeros(nb, H, bs, D, dtype=torch.bfloat16, device=DEV)
    vc = torch.zeros_like(kc)
    kv_paged_append(k.reshape(-1, H, D), v.reshape(-1, H, D), kc, vc, slots)
    lens = torch.full((B,), ctx, dtype=torch.int32, device=DEV)
    ko, vo = kv_paged_lookup(kc, vc, bt, lens, ctx)
    assert torch.equal(ko, k.permute(0, 2, 1, 3)) and torch.equal(vo, v.permute(0, 2, 1, 3))
