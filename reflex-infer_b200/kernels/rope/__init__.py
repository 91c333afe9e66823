"""RoPE; same surface as the reference's ``kernels/rope/__init__.py``.

``apply_rope`` returns a new tensor, ``apply_rope_`` rotates in place, and
``build_rope_tables`` builds the cos/sin tables on the device. Rounding follows the
reference's torch path: each multiply / add is rounded to the activation dtype
(``kernels/rope/triton_rope.py:230-240``), so 16-bit outputs match it bit for bit when
the tables carry the activation dtype (the way every reference test builds them,
``tests/test_rope.py:25-27``).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .. import _native as N


def _resolve_layout(x: torch.Tensor, layout: str):
    if x.dim() != 4:
        raise ValueError(f"x must be 4-D, got {tuple(x.shape)}")
    if layout == "bshd":
        B, S, H, D = x.shape
        sb, ss, sh, sd = x.stride()
    elif layout == "bhsd":
        B, H, S, D = x.shape
        sb, sh, ss, sd = x.stride()
    else:
        raise ValueError(f"unknown layout {layout!r}; want 'bshd' or 'bhsd'")
    return (B, S, H, D), (sb, ss, sh, sd)


def _tables_for(x, cos, sin, S, D):
    if cos.shape != (S, D) or sin.shape != (S, D):
        raise ValueError(f"cos/sin must be [{S}, {D}], got {tuple(cos.shape)} and {tuple(sin.shape)}")
    # The kernels work in the activation dtype (see module docstring).
    if cos.dtype != x.dtype:
        cos = cos.to(x.dtype)
    if sin.dtype != x.dtype:
        sin = sin.to(x.dtype)
    if cos.stride(1) != 1:
        cos = cos.contiguous()
    if sin.stride() != cos.stride():
        sin = sin.contiguous()
        cos = cos.contiguous()
    return cos, sin


def _launch(x, y, cos, sin, interleaved, layout):
    dev = N.require_cuda("apply_rope", x, y, cos, sin)
    (B, S, H, D), (xsb, xss, xsh, _) = _resolve_layout(x, layout)
    _, (ysb, yss, ysh, _) = _resolve_layout(y, layout)
    if D % 2 != 0:
        raise ValueError("head_dim must be even for RoPE")
    cos, sin = _tables_for(x, cos, sin, S, D)
    a = N.RopeArgs(
        x=N.ptr(x), y=N.ptr(y), cos=N.ptr(cos), sin=N.ptr(sin),
        batch=B, seq=S, heads=H, head_dim=D,
        x_stride_b=xsb, x_stride_s=xss, x_stride_h=xsh,
        y_stride_b=ysb, y_stride_s=yss, y_stride_h=ysh,
        table_stride_s=cos.stride(0),
        interleaved=int(bool(interleaved)), dtype=N.dtype_code(x), stream=N.stream_handle(dev),
    )
    N.call("rfx_rope_apply", a, dev)


def apply_rope(
    x: torch.Tensor,
    cos: torch.Tensor,
    sin: torch.Tensor,
    *,
    interleaved: bool = False,
    layout: str = "bshd",
    backend: Optional[str] = None,
) -> torch.Tensor:
    """Apply RoPE to ``x``; returns a new contiguous tensor.

    ``x``: ``[B, S, H, D]`` (``bshd``) or ``[B, H, S, D]`` (``bhsd``); ``cos``/``sin``: ``[S, D]``;
    row ``s`` rotates sequence index ``s``. ``interleaved`` pairs ``(2i, 2i+1)``, otherwise
    ``(i, i + D/2)``.
    """
    N.check_backend(backend)
    _resolve_layout(x, layout)
    if x.stride(-1) != 1:
        x = x.contiguous()
    y = torch.empty(x.shape, dtype=x.dtype, device=x.device)
    _launch(x, y, cos, sin, interleaved, layout)
    return y


def apply_rope_(
    x: torch.Tensor,
    cos: torch.Tensor,
    sin: torch.Tensor,
    *,
    interleaved: bool = False,
    layout: str = "bshd",
    backend: Optional[str] = None,
) -> torch.Tensor:
    """In-place RoPE. Returns the (mutated) input tensor.

    ``x`` may be any strided view whose last axis is contiguous; a view that is not
    raises instead of silently rotating a copy (the reference's Triton path does the
    latter, ``kernels/rope/triton_rope.py:172-173``).
    """
    N.check_backend(backend)
    _resolve_layout(x, layout)
    if x.stride(-1) != 1:
        raise ValueError("apply_rope_: the head_dim axis must be contiguous to rotate in place")
    _launch(x, x, cos, sin, interleaved, layout)
    return x


def build_rope_tables(
    seq_len: int,
    head_dim: int,
    *,
    base: float = 10000.0,
    device: Optional[torch.device] = None,
    dtype: torch.dtype = torch.float32,
    interleaved: bool = False,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Build the cos/sin tables ``[seq_len, head_dim]`` on the device.

    Same recipe as the reference (``kernels/rope/triton_rope.py:247-285``): inverse
    frequencies ``1/base**(i/half)`` in fp32, angle = position * frequency in fp32,
    cos/sin, duplicated to width ``head_dim`` (concatenated halves, or repeated pairs when
    ``interleaved``), cast to ``dtype``. The ``half``-long frequency vector is formed with
    the very torch expression the reference uses and handed to the kernel, so the angles
    are bit-identical; cos/sin are correctly rounded on the device, within 1 fp32 ulp of
    torch's CPU values.
    """
    if head_dim % 2 != 0:
        raise ValueError("head_dim must be even for RoPE")
    dev = torch.device("cuda" if device is None else device)
    if dev.type != "cuda":
        raise RuntimeError(f"build_rope_tables builds on a CUDA device (got {dev}); there is no CPU path")
    if dev.index is None:
        dev = torch.device("cuda", torch.cuda.current_device())
    half = head_dim // 2
    inv_freq = (1.0 / (base ** (torch.arange(0, half, dtype=torch.float32) / half))).to(dev)
    cos = torch.empty((seq_len, head_dim), dtype=dtype, device=dev)
    sin = torch.empty_like(cos)
    a = N.RopeTableArgs(cos=N.ptr(cos), sin=N.ptr(sin), inv_freq=N.ptr(inv_freq), seq_len=seq_len,
                        head_dim=head_dim, base=float(base), interleaved=int(bool(interleaved)),
                        dtype=N.dtype_code(cos), stream=N.stream_handle(dev))
    N.call("rfx_rope_build_tables", a, dev)
    return cos, sin


__all__ = [
    "apply_rope",
    "apply_rope_",
    "build_rope_tables",
]
