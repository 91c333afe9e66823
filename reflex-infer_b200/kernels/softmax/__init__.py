"""Row softmax; same surface as the reference's ``kernels/softmax/__init__.py:15-35``."""
from __future__ import annotations

from typing import Optional

import torch

from .. import _native as N


def online_softmax(
    x: torch.Tensor,
    *,
    is_causal: bool = False,
    log: bool = False,
    backend: Optional[str] = None,
) -> torch.Tensor:
    """Softmax (or log-softmax) along the last dim of ``x``, any leading shape.

    ``is_causal`` treats the last two dims as a square score matrix and masks
    ``col > row``; non-square input raises ``ValueError`` as in the reference
    (``kernels/softmax/triton_softmax.py:146-164,190-195``).
    """
    N.check_backend(backend)
    if is_causal:
        if x.dim() < 2 or x.shape[-2] != x.shape[-1]:
            raise ValueError(
                "causal mode requires square input (last two dims equal); "
                f"got {tuple(x.shape)}."
            )
    dev = N.require_cuda("online_softmax", x)
    n = x.shape[-1]
    x2 = x.reshape(-1, n).contiguous()
    y = torch.empty_like(x2)
    a = N.SoftmaxArgs(x=N.ptr(x2), y=N.ptr(y), rows=x2.shape[0], n=n, is_causal=int(is_causal), log=int(log),
                      dtype=N.dtype_code(x2), stream=N.stream_handle(dev))
    N.call("rfx_online_softmax", a, dev)
    return y.reshape(x.shape)


__all__ = ["online_softmax"]
