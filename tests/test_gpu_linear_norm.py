"""Fused linear + norm through the C ABI against the reference's outputs (golden fixtures made by
its torch path) and the oracle: the tcgen05 GEMM and the plain one, both norms, three dtypes."""
import pytest
import torch

import golden_cases as gc
import golden_io
import oracle
from kernels.fused_linear_norm import LinearNormWorkspace, fused_linear_layernorm, fused_linear_rmsnorm

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0)
# The reference's own tests of this op (tests/test_fused_linear_norm.py:41,61,81) allow 5e-2 in bf16
# and 5e-3 in fp16 and fp32. Tighter here: 2e-2 / 5e-3 for the 16-bit types (the path's general
# tolerances, kernels/_common/dtype.py:47-52) and 1e-4 in fp32 -- not the 1e-5 of dtype.py, because
# a K-long fp32 dot product summed in another order than torch's GEMM moves the result by a few
# 1e-6 relative, and the norm then divides by a standard deviation that can be small.
TOL = {torch.float32: 1e-4, torch.bfloat16: 2e-2, torch.float16: 5e-3}


def _run(c, **kw):
    d = lambda t: None if t is None else t.to(DEV)  # noqa: E731
    if c["norm"] == "rms":
        return fused_linear_rmsnorm(d(c["x"]), d(c["weight"]), bias=d(c["bias"]), gamma=d(c["gamma"]), eps=c["eps"], **kw)
    return fused_linear_layernorm(d(c["x"]), d(c["weight"]), bias=d(c["bias"]), gamma=d(c["gamma"]), beta=d(c["beta"]),
                                  eps=c["eps"], **kw)


@pytest.mark.parametrize("force_generic", [False, True])
@pytest.mark.parametrize("name", sorted(gc.linear_norm_cases()))
def test_golden(name, force_generic, native):
    c = gc.linear_norm_cases()[name]
    want, _ = golden_io.load(name)
    ws = LinearNormWorkspace(DEV)
    got = _run(c, workspace=ws, force_generic=force_generic)
    assert ws.status() == 0
    tol = TOL[c["x"].dtype]
    torch.testing.assert_close(got.cpu().float(), want["y"].float(), atol=tol, rtol=tol)


def test_tensor_core_gemm_is_selected(native):
    import ctypes as C
    from kernels import _native as N
    def kind(dtype, K, Nn, M=4):
        a = N.LinearNormArgs(x=256, weight=256, out=256, M=M, K=K, N=Nn, eps=1e-5, norm_type=1, dtype=N._DTYPE_CODE[dtype])
        return N.lib().rfx_fused_linear_norm_kernel_kind(C.byref(a))
    assert kind(torch.bfloat16, 4096, 4096) == 2      # 4 rows: the weight-streaming kernel
    assert kind(torch.bfloat16, 4096, 4096, M=512) == 1
    assert kind(torch.float16, 768, 3072, M=100) == 1
    assert kind(torch.float32, 4096, 4096) == 0
    assert kind(torch.bfloat16, 60, 70) == 0


@pytest.mark.parametrize("M,K,N,norm", [(1, 4096, 4096, "rms"), (7, 512, 1000, "layer"), (300, 1024, 1792, "rms"),
                                        (257, 768, 3072, "layer")])
def test_larger_shapes_vs_oracle(M, K, N, norm, native):
    """Row counts off the tile, many K steps (the ring wraps), several N tiles per row (the row
    statistics come from more than one CTA), a 3-D input."""
    g = torch.Generator().manual_seed(M + N)
    dt = torch.bfloat16
    x = torch.randn(1, M, K, generator=g).to(dt)
    w = (torch.randn(N, K, generator=g) * K ** -0.5).to(dt)
    bias, gamma = torch.randn(N, generator=g).to(dt), (1 + 0.1 * torch.randn(N, generator=g)).to(dt)
    beta = torch.randn(N, generator=g).to(dt) if norm == "layer" else None
    want = oracle.fused_linear_norm(x, w, bias=bias, gamma=gamma, beta=beta, norm_type=norm)
    fn = fused_linear_rmsnorm if norm == "rms" else fused_linear_layernorm
    kw = dict(bias=bias.to(DEV), gamma=gamma.to(DEV))
    if beta is not None:
        kw["beta"] = beta.to(DEV)
    got = fn(x.to(DEV), w.to(DEV), **kw)
    assert got.shape == (1, M, N)
    # 3e-2: random weights with K up to 4096 and a bias and gamma of order one put outputs near +-4,
    # where one bf16 ulp is 3.1e-2 -- the oracle and the kernel may round the same value to neighbours;
    # the reference's tolerance for this op in bf16 is 5e-2 (tests/test_fused_linear_norm.py:41)
    torch.testing.assert_close(got.cpu().float(), want.float(), atol=3e-2, rtol=3e-2)


def test_errors(native):
    x = torch.zeros(4, 8, device=DEV, dtype=torch.bfloat16)
    w = torch.zeros(16, 8, device=DEV, dtype=torch.bfloat16)
    with pytest.raises(ValueError):
        fused_linear_rmsnorm(x, torch.zeros(16, 9, device=DEV, dtype=torch.bfloat16))
    with pytest.raises(ValueError):
        fused_linear_rmsnorm(x, w, gamma=torch.zeros(15, device=DEV, dtype=torch.bfloat16))
    with pytest.raises(RuntimeError):
        fused_linear_rmsnorm(x.cpu(), w.cpu())
    with pytest.raises(ValueError):
        fused_linear_rmsnorm(x, w, backend="metal")
    assert fused_linear_rmsnorm(x[:0], w).shape == (0, 16)
