"""GPU parity of RoPE through the C ABI. The torch path of the reference rounds after each
op, and so do the kernels: outputs are compared bit for bit in every dtype."""
from __future__ import annotations

import pytest
import torch

import golden_cases as gc
import golden_io
import oracle
from kernels.rope import apply_rope, apply_rope_, build_rope_tables

pytestmark = [pytest.mark.gpu]
DEV = "cuda"


@pytest.mark.parametrize("name", sorted(gc.rope_cases()))
def test_apply_golden(name, native):
    c = gc.rope_cases()[name]
    t, meta = golden_io.load(name)
    y = apply_rope(c["x"].to(DEV), t["cos"].to(DEV), t["sin"].to(DEV), interleaved=c["interleaved"], layout=c["layout"])
    assert y.is_contiguous() and y.shape == c["x"].shape
    assert golden_io.digest(y) == meta["y_digest"], f"max diff {(y.cpu().float() - t['y'].float()).abs().max()}"


def test_inplace_equals_out_of_place(native):  # reference tests/test_rope.py:37-50
    x = golden_io.pattern((1, 32, 2, 64), torch.float16, 1).to(DEV)
    cos, sin = (t.to(DEV) for t in oracle.build_rope_tables(32, 64, dtype=torch.float16))
    y = apply_rope(x, cos, sin)
    x2 = x.clone()
    r = apply_rope_(x2, cos, sin)
    assert r is x2 and torch.equal(x2, y)


def test_position_zero_is_identity(native):  # reference tests/test_rope.py:68-77
    x = golden_io.pattern((2, 1, 3, 32), torch.float32, 2).to(DEV)
    cos, sin = build_rope_tables(1, 32, device=DEV)
    assert torch.equal(apply_rope(x, cos, sin), x)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("inter", [False, True])
def test_strided_views_and_odd_widths(native, dtype, inter):
    """In place on a slice of a fused QKV buffer (strided, offset), head_dim 6 and 80."""
    for D in (6, 80):
        B, S, H = 2, 5, 3
        qkv = golden_io.pattern((B, S, 3 * H, D), dtype, 3)
        cos, sin = oracle.build_rope_tables(S, D, dtype=dtype, interleaved=inter)
        want = qkv.clone()
        want[:, :, H:2 * H] = oracle.apply_rope(qkv[:, :, H:2 * H], cos, sin, interleaved=inter)
        g = qkv.to(DEV)
        apply_rope_(g[:, :, H:2 * H], cos.to(DEV), sin.to(DEV), interleaved=inter)
        assert torch.equal(g.cpu(), want)
        y = apply_rope(qkv.to(DEV)[:, :, :H], cos.to(DEV), sin.to(DEV), interleaved=inter)
        assert torch.equal(y.cpu(), oracle.apply_rope(qkv[:, :, :H], cos, sin, interleaved=inter))


@pytest.mark.parametrize("name", sorted(gc.rope_table_cases()))
def test_tables_golden(name, native):
    """Device-built tables vs the reference's host-built ones: fp32 within 1e-5 (they differ
    by at most one fp32 ulp where torch's vectorised cos/sin is not correctly rounded)."""
    c = gc.rope_table_cases()[name]
    t, _ = golden_io.load(name)
    cos, sin = build_rope_tables(c["seq_len"], c["D"], base=c["base"], device=DEV, dtype=c["dtype"], interleaved=c["interleaved"])
    assert cos.shape == (c["seq_len"], c["D"]) and cos.dtype == c["dtype"]
    ref_cos, ref_sin = oracle.build_rope_tables(c["seq_len"], c["D"], base=c["base"], dtype=c["dtype"], interleaved=c["interleaved"])
    tol = 1e-5 if c["dtype"] == torch.float32 else 8e-3  # one bf16 ulp near 1.0
    torch.testing.assert_close(cos.cpu().float(), ref_cos.float(), atol=tol, rtol=0)
    torch.testing.assert_close(sin.cpu().float(), ref_sin.float(), atol=tol, rtol=0)
    torch.testing.assert_close(cos.cpu()[c["rows"]].float(), t["cos"].float(), atol=tol, rtol=0)
    if c["dtype"] == torch.float32:
        ulp = (cos.cpu() - ref_cos).abs().max().item()
        assert ulp <= 1.2e-7, ulp
    else:
        frac = (cos.cpu() != ref_cos).float().mean().item()
        assert frac < 1e-4, f"{frac:.2e} of bf16 cos entries differ"


def test_errors(native):
    x = torch.zeros(1, 2, 2, 8, device=DEV)
    cos = torch.zeros(2, 8, device=DEV)
    with pytest.raises(ValueError, match="unknown layout"):
        apply_rope(x, cos, cos, layout="hbsd")
    with pytest.raises(ValueError, match="cos/sin must be"):
        apply_rope(x, cos[:1], cos[:1])
    with pytest.raises(ValueError, match="even"):
        build_rope_tables(4, 9, device=DEV)
