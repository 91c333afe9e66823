"""GPU parity of dense fused_attention through the C ABI (fp32 1e-5, bf16 2e-2, fp16 5e-3 as
the reference's tests use, tests/test_attention_parity.py)."""
from __future__ import annotations

import pytest
import torch

import golden_cases as gc
import golden_io
import oracle
from kernels.attention import fused_attention

pytestmark = [pytest.mark.gpu]
DEV = "cuda"
TOL = {torch.float32: 1e-5, torch.bfloat16: 2e-2, torch.float16: 5e-3}


@pytest.mark.parametrize("name", sorted(gc.attention_cases()))
def test_golden(name, native):
    c = gc.attention_cases()[name]
    t, _ = golden_io.load(name)
    tol = TOL[c["q"].dtype]
    mask = None if c["mask"] is None else c["mask"].to(DEV)
    o = fused_attention(c["q"].to(DEV), c["k"].to(DEV), c["v"].to(DEV), is_causal=c["causal"], attn_mask=mask,
                        sm_scale=c["sm_scale"])
    assert o.shape == c["q"].shape and o.dtype == c["q"].dtype
    torch.testing.assert_close(o.cpu().float(), t["out"].float(), atol=tol, rtol=tol)


@pytest.mark.parametrize("shape", [(1, 4, 128, 128, True), (1, 4, 1, 2048, False), (1, 4, 37, 500, False)])
def test_shapes_fp32_vs_oracle(native, shape):  # reference tests/test_attention_parity.py:37-56
    B, H, Sq, Sk, causal = shape
    q = golden_io.pattern((B, H, Sq, 64), torch.float32, 1)
    k, v = golden_io.pattern((B, H, Sk, 64), torch.float32, 2), golden_io.pattern((B, H, Sk, 64), torch.float32, 3)
    o = fused_attention(q.to(DEV), k.to(DEV), v.to(DEV), is_causal=causal)
    torch.testing.assert_close(o.cpu(), oracle.attention(q, k, v, is_causal=causal), atol=1e-5, rtol=1e-5)


def test_gqa_matches_expansion(native):  # reference tests/test_attention_parity.py:59-78
    q = golden_io.pattern((1, 32, 256, 64), torch.float16, 4)
    k, v = golden_io.pattern((1, 4, 256, 64), torch.float16, 5), golden_io.pattern((1, 4, 256, 64), torch.float16, 6)
    o = fused_attention(q.to(DEV), k.to(DEV), v.to(DEV), is_causal=True)
    ref = oracle.naive_attention_f64(q, k, v, mask=torch.triu(torch.full((256, 256), float("-inf")), 1))
    torch.testing.assert_close(o.cpu().double(), ref, atol=5e-3, rtol=5e-3)


def test_errors(native):
    q = torch.zeros(1, 6, 4, 8, device=DEV)
    with pytest.raises(ValueError, match="GQA requires"):
        fused_attention(q, torch.zeros(1, 4, 4, 8, device=DEV), torch.zeros(1, 4, 4, 8, device=DEV))
    with pytest.raises(ValueError, match="shape mismatch"):
        fused_attention(q, torch.zeros(1, 6, 4, 16, device=DEV), torch.zeros(1, 6, 4, 16, device=DEV))
    with pytest.raises(ValueError, match="attn_mask must be"):
        fused_attention(q, q, q, attn_mask=torch.zeros(1, 6, 4, 5, device=DEV))
    with pytest.raises(RuntimeError, match="CUDA"):
        fused_attention(q.cpu(), q.cpu(), q.cpu())
