"""GPU parity of online_softmax through the C ABI (tolerances: the reference's
kernels/_common/dtype.py:47-52 -- fp32 1e-5, bf16 2e-2, fp16 1e-3)."""
from __future__ import annotations

import pytest
import torch

import golden_cases as gc
import golden_io
import oracle
from kernels.softmax import online_softmax

pytestmark = [pytest.mark.gpu]
DEV = "cuda"
TOL = {torch.float32: 1e-5, torch.bfloat16: 2e-2, torch.float16: 1e-3}


@pytest.mark.parametrize("name", sorted(gc.softmax_cases()))
def test_golden(name, native):
    c = gc.softmax_cases()[name]
    t, _ = golden_io.load(name)
    tol = TOL[c["x"].dtype]
    y = online_softmax(c["x"].to(DEV), is_causal=c["causal"])
    ylog = online_softmax(c["x"].to(DEV), is_causal=c["causal"], log=True)
    torch.testing.assert_close(y.cpu().float(), t["y"].float(), atol=tol, rtol=tol)
    finite = torch.isfinite(t["ylog"])
    assert torch.equal(torch.isfinite(ylog.cpu()), finite)
    torch.testing.assert_close(ylog.cpu().float()[finite], t["ylog"].float()[finite], atol=tol * 10, rtol=tol)
    assert y.dtype == c["x"].dtype and y.shape == c["x"].shape


@pytest.mark.parametrize("n", [4096, 8192])
def test_long_fp32_rows_many_per_cta(native, n):
    """fp32 rows of four or eight vectors per thread: the grid is one wave of CTAs, each walking
    several rows with the next row's loads already in flight; plain and causal (ragged lengths)."""
    x = torch.randn(1500, n, device=DEV, generator=torch.Generator(device=DEV).manual_seed(n))
    torch.testing.assert_close(online_softmax(x).cpu(), oracle.online_softmax(x.cpu()), atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(online_softmax(x, log=True).cpu(), oracle.online_softmax(x.cpu(), log=True), atol=1e-4, rtol=1e-5)
    sq = torch.randn(1, 1, n, n, device=DEV, generator=torch.Generator(device=DEV).manual_seed(n + 1))
    y = online_softmax(sq, is_causal=True)
    rows = torch.tensor([0, 1, 7, 8, 1023, 1024, n // 2, n - 2, n - 1])
    ref = oracle.online_softmax(sq.cpu(), is_causal=True)
    torch.testing.assert_close(y.cpu()[0, 0, rows], ref[0, 0, rows], atol=1e-5, rtol=1e-5)
    assert not torch.triu(y[0, 0], diagonal=1).any()
    torch.testing.assert_close(y[0, 0].sum(-1), torch.ones(n, device=DEV), atol=1e-4, rtol=0)


@pytest.mark.parametrize("n", [1, 33, 4096, 50257, 60000])
def test_rows_sum_to_one(native, n):  # reference tests/test_softmax.py:17-33; 60000 takes the unstaged path
    x = torch.randn(6, n, device=DEV, generator=torch.Generator(device=DEV).manual_seed(n))
    y = online_softmax(x)
    torch.testing.assert_close(y.sum(-1), torch.ones(6, device=DEV), atol=1e-4, rtol=0)
    torch.testing.assert_close(y.cpu(), oracle.online_softmax(x.cpu()), atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(online_softmax(x, log=True).cpu(), oracle.online_softmax(x.cpu(), log=True), atol=1e-4, rtol=1e-5)


def test_batched_causal_and_errors(native):  # reference tests/test_softmax.py:63-97
    x = golden_io.pattern((2, 2, 33, 33), torch.float32, 5).to(DEV)
    y = online_softmax(x, is_causal=True)
    torch.testing.assert_close(y.cpu(), oracle.online_softmax(x.cpu(), is_causal=True), atol=1e-5, rtol=1e-5)
    assert not torch.triu(y, diagonal=1).any()
    with pytest.raises(ValueError, match="causal mode requires square"):
        online_softmax(torch.zeros(4, 8, device=DEV), is_causal=True)
    with pytest.raises(ValueError, match="backend="):
        online_softmax(x, backend="rocm")
