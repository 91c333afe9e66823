"""Fused linear + LayerNorm / RMSNorm; same surface as the reference's
``kernels/fused_linear_norm/__init__.py:27-73``."""
from __future__ import annotations

from typing import Optional

import torch

from .. import _native as N


class LinearNormWorkspace:
    """Row statistics of the norm (and a status word); grows on demand, reused across calls."""

    def __init__(self, device):
        self.device = torch.device(device)
        self.buf: Optional[torch.Tensor] = None

    def ensure(self, nbytes: int) -> torch.Tensor:
        if self.buf is None or self.buf.numel() < nbytes:
            self.buf = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
        return self.buf

    def status(self) -> int:
        return 0 if self.buf is None else int(self.buf[:4].view(torch.int32).item())


class LinearNormCall:
    """A validated, ready-to-launch fused linear + norm over fixed buffers: argument checks and
    workspace sizing happen once, ``run()`` is one foreign call (what a serving loop that reuses
    its buffers wants, and what a CUDA graph captures)."""

    def __init__(self, x, weight, *, bias=None, gamma=None, beta=None, eps=1e-5, norm_type="rms", out=None,
                 workspace=None, force_generic=False, name="fused_linear_norm"):
        import ctypes as C
        dev = N.require_cuda(name, x, weight, bias, gamma, beta, out)
        if weight.dim() != 2:
            raise ValueError(f"{name}: weight must be [D_out, D_in], got {tuple(weight.shape)}")
        n, k = weight.shape
        if x.shape[-1] != k:
            raise ValueError(f"{name}: x has {x.shape[-1]} input features, weight expects {k}")
        for t, what in ((bias, "bias"), (gamma, "gamma"), (beta, "beta")):
            if t is not None and t.shape != (n,):
                raise ValueError(f"{name}: {what} must be [{n}], got {tuple(t.shape)}")
        for t in (weight, bias, gamma, beta):
            if t is not None and t.dtype != x.dtype:
                raise RuntimeError(f"{name}: all tensors must share x's dtype {x.dtype}")
        if norm_type not in ("layer", "rms"):
            raise ValueError(f"{name}: norm_type must be 'layer' or 'rms'")
        x2 = x.reshape(-1, k).contiguous()
        if out is None:
            out = torch.empty((x2.shape[0], n), dtype=x.dtype, device=dev)
        elif out.shape != (x2.shape[0], n) or out.dtype != x.dtype or not out.is_contiguous():
            raise ValueError(f"{name}: out must be a contiguous [{x2.shape[0]}, {n}] tensor of x's dtype")
        cont = lambda t: None if t is None else t.contiguous()  # noqa: E731
        weight, bias, gamma, beta = weight.contiguous(), cont(bias), cont(gamma), cont(beta)
        a = N.LinearNormArgs(x=N.ptr(x2), weight=N.ptr(weight), bias=N.ptr(bias), gamma=N.ptr(gamma), beta=N.ptr(beta),
                             out=N.ptr(out), M=x2.shape[0], K=k, N=n, eps=float(eps),
                             norm_type=0 if norm_type == "layer" else 1, dtype=N.dtype_code(x2),
                             force_generic=int(bool(force_generic)), workspace=None, workspace_bytes=0, stream=None)
        lib = N.lib()
        need = int(lib.rfx_fused_linear_norm_workspace_bytes(C.byref(a)))
        if workspace is None:
            workspace = LinearNormWorkspace(dev)
        buf = workspace.ensure(max(need, 256))
        a.workspace, a.workspace_bytes = buf.data_ptr(), buf.numel()
        self.kernel_kind = int(lib.rfx_fused_linear_norm_kernel_kind(C.byref(a)))  # 1 tcgen05, 2 small-M, 0 plain
        self.out = out.reshape(*x.shape[:-1], n)
        self.workspace = workspace
        self.device = dev
        self._args, self._ref, self._lib = a, C.byref(a), lib
        self._keep = (x2, weight, bias, gamma, beta, out, buf)

    def run(self) -> torch.Tensor:
        self._args.stream = N.stream_handle(self.device)
        with torch.cuda.device(self.device):
            N.check(self._lib.rfx_fused_linear_norm(self._ref))
        return self.out


def _fused_linear_norm(name, x, weight, bias, gamma, beta, eps, norm_type, backend, workspace, force_generic):
    N.check_backend(backend)
    return LinearNormCall(x, weight, bias=bias, gamma=gamma, beta=beta, eps=eps,
                          norm_type="layer" if norm_type == 0 else "rms", workspace=workspace,
                          force_generic=force_generic, name=name).run()


def fused_linear_layernorm(
    x: torch.Tensor,
    weight: torch.Tensor,
    *,
    bias: Optional[torch.Tensor] = None,
    gamma: Optional[torch.Tensor] = None,
    beta: Optional[torch.Tensor] = None,
    eps: float = 1e-5,
    backend: Optional[str] = None,
    workspace: Optional[LinearNormWorkspace] = None,
    force_generic: bool = False,
) -> torch.Tensor:
    """``layer_norm(x @ weight.T + bias) * gamma + beta`` over the last dim
    (``kernels/fused_linear_norm/__init__.py:27-50``)."""
    return _fused_linear_norm("fused_linear_layernorm", x, weight, bias, gamma, beta, eps, 0, backend, workspace,
                              force_generic)


def fused_linear_rmsnorm(
    x: torch.Tensor,
    weight: torch.Tensor,
    *,
    bias: Optional[torch.Tensor] = None,
    gamma: Optional[torch.Tensor] = None,
    eps: float = 1e-5,
    backend: Optional[str] = None,
    workspace: Optional[LinearNormWorkspace] = None,
    force_generic: bool = False,
) -> torch.Tensor:
    """``rmsnorm(x @ weight.T + bias) * gamma`` (``kernels/fused_linear_norm/__init__.py:53-73``)."""
    return _fused_linear_norm("fused_linear_rmsnorm", x, weight, bias, gamma, None, eps, 1, backend, workspace,
                              force_generic)


__all__ = ["fused_linear_layernorm", "fused_linear_rmsnorm", "LinearNormWorkspace", "LinearNormCall"]
