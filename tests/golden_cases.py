"""Inputs of the golden cases, rebuilt identically by the fixture generator
(``tests/golden/make_golden.py``, which runs the reference on them) and by the tests (which
run the oracle and the CUDA library on them). Shapes follow the reference's own tests
(``tests/test_kv_cache.py``, ``test_rope.py``, ``test_softmax.py``, ``test_attention_parity.py``)
and small versions of the benchmark configurations."""
from __future__ import annotations

import torch

from golden_io import pattern

F16, BF16, F32 = torch.float16, torch.bfloat16, torch.float32
_TAG = {F16: "f16", BF16: "bf16", F32: "f32"}


def _perm(n: int, seed: int) -> torch.Tensor:
    """Deterministic permutation of range(n) from the integer pattern."""
    keys = pattern((n,), torch.float64, seed) + torch.arange(n, dtype=torch.float64) * 1e-9
    return torch.argsort(keys, stable=True)


def kv_write_cases() -> dict:
    cases = {}
    N, H, D, bs, nb = 32, 8, 64, 16, 8  # tests/test_kv_cache.py:33-53
    for i, dt in enumerate((F16, BF16, F32)):
        cases[f"kv_append_{_TAG[dt]}"] = dict(
            op="append", k_in=pattern((N, H, D), dt, 100 + i), v_in=pattern((N, H, D), dt, 110 + i),
            slots=torch.arange(N, dtype=torch.int64) * 2,
            k_cache0=pattern((nb, H, bs, D), dt, 120 + i), v_cache0=pattern((nb, H, bs, D), dt, 130 + i))
    N, H, D, bs, nb = 37, 3, 40, 8, 11  # odd sizes, random distinct slots, scatter entry (tests/test_kv_cache.py:125-145)
    cases["kv_scatter_odd_bf16"] = dict(
        op="scatter", k_in=pattern((N, H, D), BF16, 140), v_in=pattern((N, H, D), BF16, 141),
        slots=_perm(nb * bs, 142)[:N].to(torch.int64),
        k_cache0=torch.zeros(nb, H, bs, D, dtype=BF16), v_cache0=torch.zeros(nb, H, bs, D, dtype=BF16))
    return cases


def kv_lookup_cases() -> dict:
    cases = {}
    B, H, D, bs, ctx = 4, 8, 64, 16, 96  # tests/test_kv_cache.py:56-87
    nblk = ctx // bs
    cases["kv_lookup_f16"] = dict(
        k_cache=pattern((B * nblk, H, bs, D), F16, 200), v_cache=pattern((B * nblk, H, bs, D), F16, 201),
        block_table=torch.arange(B * nblk, dtype=torch.int64).view(B, nblk),
        context_lens=torch.full((B,), ctx, dtype=torch.int32), max_ctx=ctx)
    B, H, D, bs, max_ctx, nb = 3, 4, 32, 8, 64, 40  # zero tail, empty request, permuted pages (:90-122)
    cases["kv_lookup_ragged_bf16"] = dict(
        k_cache=pattern((nb, H, bs, D), BF16, 210), v_cache=pattern((nb, H, bs, D), BF16, 211),
        block_table=_perm(nb, 212)[: B * 8].view(B, 8).to(torch.int64),
        context_lens=torch.tensor([16, 40, 0], dtype=torch.int32), max_ctx=max_ctx)
    cases["kv_lookup_edges_f32"] = dict(  # lengths around page boundaries: 0, 1, bs-1, bs, bs+1
        k_cache=pattern((12, 2, 4, 8), F32, 220), v_cache=pattern((12, 2, 4, 8), F32, 221),
        block_table=_perm(12, 222)[:10].view(5, 2).to(torch.int64),
        context_lens=torch.tensor([0, 1, 3, 4, 5], dtype=torch.int32), max_ctx=7)
    return cases


def rope_cases() -> dict:
    cases = {}
    i = 0
    for dt in (F16, BF16, F32):
        for inter in (False, True):  # tests/test_rope.py:17-34
            cases[f"rope_{_TAG[dt]}_{'inter' if inter else 'half'}"] = dict(
                x=pattern((2, 64, 4, 64), dt, 300 + i), table_rows=64, D=64, base=1e4, dtype=dt, interleaved=inter,
                layout="bshd", pos=None)
            i += 1
    cases["rope_bhsd_f16"] = dict(x=pattern((1, 2, 16, 64), F16, 320), table_rows=16, D=64, base=1e4, dtype=F16,
                                  interleaved=False, layout="bhsd", pos=None)  # tests/test_rope.py:53-65
    pos = torch.tensor([0, 1, 511, 4095, 8191, 20000, 32767])
    cases["rope_bf16_bigpos"] = dict(x=pattern((1, 7, 5, 128), BF16, 321), table_rows=32768, D=128, base=1e6,
                                     dtype=BF16, interleaved=False, layout="bshd", pos=pos)
    return cases


def rope_table_cases() -> dict:
    return {
        "rope_tables_f32_1e4": dict(seq_len=257, D=64, base=1e4, dtype=F32, interleaved=False,
                                    rows=torch.tensor([0, 1, 2, 17, 128, 255, 256])),
        "rope_tables_bf16_1e6": dict(seq_len=8193, D=128, base=1e6, dtype=BF16, interleaved=False,
                                     rows=torch.tensor([0, 1, 255, 4097, 8192])),
        "rope_tables_f32_1e6_inter": dict(seq_len=32769, D=128, base=1e6, dtype=F32, interleaved=True,
                                          rows=torch.tensor([0, 1, 2, 255, 256, 4097, 8192, 16385, 32768])),
    }


def softmax_cases() -> dict:
    cases = {}
    i = 0
    for dt in (F32, BF16, F16):
        for n in (64, 1000):  # tests/test_softmax.py:17-45
            cases[f"softmax_{_TAG[dt]}_{n}"] = dict(x=pattern((8, n), dt, 400 + i, scale=2.0), causal=False)
            i += 1
    cases["softmax_causal_f32"] = dict(x=pattern((2, 3, 16, 16), F32, 420), causal=True)  # :63-84
    cases["softmax_large_f32"] = dict(x=pattern((4, 128), F32, 421) + 1000.0, causal=False)  # :48-60
    return cases


def attention_cases() -> dict:
    cases = {}
    i = 0
    for dt in (F32, BF16, F16):
        for causal in (False, True):  # tests/test_attention_parity.py:18-34 (smaller batch)
            cases[f"attn_mha_{_TAG[dt]}_{'causal' if causal else 'full'}"] = dict(
                q=pattern((1, 4, 64, 64), dt, 500 + i), k=pattern((1, 4, 64, 64), dt, 520 + i),
                v=pattern((1, 4, 64, 64), dt, 540 + i), causal=causal, mask=None, sm_scale=None)
            i += 1
    cases["attn_decode_f32"] = dict(q=pattern((1, 4, 1, 64), F32, 560), k=pattern((1, 4, 300, 64), F32, 561),
                                    v=pattern((1, 4, 300, 64), F32, 562), causal=False, mask=None, sm_scale=None)
    cases["attn_gqa_bf16_causal"] = dict(q=pattern((1, 8, 48, 128), BF16, 563), k=pattern((1, 2, 48, 128), BF16, 564),
                                         v=pattern((1, 2, 48, 128), BF16, 565), causal=True, mask=None, sm_scale=None)
    mask = pattern((2, 2, 10, 20), F32, 566)
    mask[:, :, :, 15:] = float("-inf")
    cases["attn_mask_scale_f32"] = dict(q=pattern((2, 2, 10, 32), F32, 567), k=pattern((2, 2, 20, 32), F32, 568),
                                        v=pattern((2, 2, 20, 32), F32, 569), causal=False, mask=mask, sm_scale=0.37)
    return cases


def _step(seed, *, Hq, Hkv, D, bs, lens, theta, dt, contiguous=False):
    B = len(lens)
    lens_t = torch.tensor(lens, dtype=torch.int64)
    pages = (lens_t + 1 + bs - 1) // bs
    nb = int(pages.sum()) + (0 if contiguous else 3)
    perm = torch.arange(nb) if contiguous else _perm(nb, seed)
    bt = torch.full((B, int(pages.max())), -1, dtype=torch.int64)
    o = 0
    for b in range(B):
        bt[b, : pages[b]] = perm[o:o + int(pages[b])]
        o += int(pages[b])
    pos = lens_t.clone()
    slots = bt[torch.arange(B), pos // bs] * bs + pos % bs
    return dict(q=pattern((B, Hq, D), dt, seed + 1), k=pattern((B, Hkv, D), dt, seed + 2),
                v=pattern((B, Hkv, D), dt, seed + 3),
                k_cache0=pattern((nb, Hkv, bs, D), dt, seed + 4), v_cache0=pattern((nb, Hkv, bs, D), dt, seed + 5),
                block_table=bt, old_lens=lens_t.to(torch.int32), context_lens=(lens_t + 1).to(torch.int32),
                positions=pos.to(torch.int32), slots=slots, table_rows=int(lens_t.max()) + 1, D=D, theta=theta,
                dtype=dt, block_size=bs)


def step_cases() -> dict:
    return {
        # configuration 1 as stated: fp32 MHA, 16 heads, D=64, 256 keys in contiguous pages of 16 + 1 new, theta 1e4
        "step_cfg1_f32": _step(600, Hq=16, Hkv=16, D=64, bs=16, lens=[256], theta=1e4, dt=F32, contiguous=True),
        # configuration-2-like: bf16 GQA 16/2, D=128, pages of 16, theta 1e6, lengths on page edges, one empty
        "step_cfg2_small_bf16": _step(610, Hq=16, Hkv=2, D=128, bs=16, lens=[0, 15, 16, 17, 200, 333], theta=1e6, dt=BF16),
        # configuration-4-like: 64/8 heads, pages of 32
        "step_cfg4_small_bf16": _step(620, Hq=64, Hkv=8, D=128, bs=32, lens=[31, 64, 257], theta=1e6, dt=BF16),
        # configuration-5-like head ratio (28/4: group of 7), pages of 16
        "step_cfg5_small_bf16": _step(630, Hq=28, Hkv=4, D=128, bs=16, lens=[5, 100, 48], theta=1e6, dt=BF16),
    }


def linear_norm_cases() -> dict:
    """Small shapes of the reference's fused linear + norm (tests/test_fused_linear_norm.py and the
    bench shapes of benchmark/bench_fused_linear_norm.py:24-29 scaled down): both norms, the three
    dtypes, optional bias / gamma / beta, row counts off the 128-row tile and widths off the
    256-column tile."""
    cases = {}
    spec = [("rms_bf16", BF16, 200, 256, 512, "rms", True, True),
            ("rms_bf16_nobias", BF16, 64, 128, 264, "rms", False, True),
            ("rms_f16_nogamma", F16, 130, 192, 256, "rms", True, False),
            ("layer_f16", F16, 96, 256, 768, "layer", True, True),
            ("layer_bf16_plain", BF16, 33, 64, 128, "layer", False, False),
            ("rms_f32", F32, 40, 72, 100, "rms", True, True),
            ("layer_f32", F32, 17, 50, 96, "layer", True, True),
            ("rms_bf16_odd", BF16, 10, 60, 70, "rms", True, True)]
    for i, (name, dt, M, K, N, norm, has_bias, has_gamma) in enumerate(spec):
        c = dict(x=pattern((M, K), dt, 700 + 10 * i), weight=pattern((N, K), dt, 701 + 10 * i, scale=0.25),
                 bias=pattern((N,), dt, 702 + 10 * i) if has_bias else None,
                 gamma=(pattern((N,), dt, 703 + 10 * i) + 1.0).to(dt) if has_gamma else None,
                 beta=pattern((N,), dt, 704 + 10 * i) if (norm == "layer" and has_gamma) else None,
                 norm=norm, eps=1e-5)
        cases[f"linear_norm_{name}"] = c
    return cases
