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


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("n", [512, 2048, 4096, 8192, 16384])
def test_16bit_rows_held_raw_in_registers(native, dtype, n):
    """16-bit rows stay in registers in their own type: a warp per row (up to 2048 elements), 128 threads
    (up to 4096), a CTA of 256 (up to 16 384). Plain, log and causal, against the oracle."""
    tol = TOL[dtype]
    x = (torch.randn(600, n, device=DEV, generator=torch.Generator(device=DEV).manual_seed(n)) * 3).to(dtype)
    torch.testing.assert_close(online_softmax(x).cpu().float(), oracle.online_softmax(x.cpu()).float(), atol=tol, rtol=tol)
    torch.testing.assert_close(online_softmax(x, log=True).cpu().float(), oracle.online_softmax(x.cpu(), log=True).float(),
                               atol=tol * 10, rtol=tol)
    if n <= 2048:
        sq = (torch.randn(2, n, n, device=DEV, generator=torch.Generator(device=DEV).manual_seed(n + 1)) * 3).to(dtype)
        y = online_softmax(sq, is_causal=True)
        torch.testing.assert_close(y.cpu().float(), oracle.online_softmax(sq.cpu(), is_causal=True).float(), atol=tol, rtol=tol)
        assert not torch.triu(y[0], diagonal=1).any()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_odd_16bit_rows_staged_in_shared_memory(native, dtype):
    """16-bit rows of an odd length below 64 KB: staged in shared memory in their own type, every row at
    another alignment, the exponentials kept in place of the inputs. Plain and log against the oracle."""
    tol = TOL[dtype]
    x = (torch.randn(400, 20001, device=DEV, generator=torch.Generator(device=DEV).manual_seed(6)) * 3).to(dtype)
    torch.testing.assert_close(online_softmax(x).cpu().float(), oracle.online_softmax(x.cpu()).float(), atol=tol, rtol=tol)
    torch.testing.assert_close(online_softmax(x, log=True).cpu().float(), oracle.online_softmax(x.cpu(), log=True).float(),
                               atol=tol * 10, rtol=tol)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_long_rows_in_two_passes(native, dtype):
    """Vocabulary-sized rows (64 KB and more): two passes over global memory with a running (maximum,
    sum) per thread, nothing staged; odd length, so every row starts at another alignment. Plain, log
    and in place against the oracle; causal rows (a 16 392-square for the 16-bit types' 64 KB) against
    the oracle on the visible part of sampled rows."""
    tol = TOL[dtype]
    x = (torch.randn(400, 50257, device=DEV, generator=torch.Generator(device=DEV).manual_seed(7)) * 3).to(dtype)
    ref = oracle.online_softmax(x.cpu()).float()
    torch.testing.assert_close(online_softmax(x).cpu().float(), ref, atol=tol, rtol=tol)
    torch.testing.assert_close(online_softmax(x, log=True).cpu().float(), oracle.online_softmax(x.cpu(), log=True).float(),
                               atol=tol * 10, rtol=tol)
    n = 16392 if dtype == torch.float32 else 32776  # rows of just over 64 KB
    sq = (torch.randn(1, n, n, device=DEV, generator=torch.Generator(device=DEV).manual_seed(8)) * 3).to(dtype)
    y = online_softmax(sq, is_causal=True)
    assert not torch.triu(y[0], diagonal=1).any()
    for r in (0, 1, 7, 8, 4097, n // 2, n - 2, n - 1):
        rr = oracle.online_softmax(sq[0, r:r + 1, :r + 1].cpu())
        torch.testing.assert_close(y[0, r:r + 1, :r + 1].cpu().float(), rr.float(), atol=tol, rtol=tol)


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
