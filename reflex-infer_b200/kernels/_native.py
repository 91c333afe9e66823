"""ctypes binding of ``libreflex_b200.so`` (the C ABI declared in ``include/reflex_b200.h``).

This module is the only place where Python touches the native library. It loads the
shared object built in-tree by ``build.py``, mirrors the C argument structs, and turns a
non-zero status into the exception type the reference raises for the same mistake
(``ValueError`` for argument problems, ``RuntimeError`` otherwise; reference:
``kernels/attention/triton_fused_attention.py:275-286``, ``kernels/_common/launch.py:109-111``).

There is deliberately no fallback: if the library is missing or the tensors are not on a
CUDA device the call fails.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path
from typing import Optional

import torch

_LIB_PATH = Path(__file__).resolve().parent.parent / "lib" / "libreflex_b200.so"
_lib: Optional[C.CDLL] = None

RFX_SUCCESS = 0
RFX_UNSUPPORTED_DEVICE = 1
RFX_INVALID_ARGUMENT = 4
RFX_NOT_IMPLEMENTED = 5
RFX_CUDA_ERROR = 6
RFX_TIMEOUT = 7
RFX_WORKSPACE_TOO_SMALL = 8

_DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}

_VALID_BACKENDS = {None, "triton", "cuda", "torch"}

i64 = C.c_int64
vp = C.c_void_p


class KvAppendArgs(C.Structure):
    _fields_ = [
        ("k_in", vp), ("v_in", vp), ("k_cache", vp), ("v_cache", vp), ("slot_mapping", vp),
        ("n_tokens", i64), ("num_kv_heads", i64), ("head_dim", i64), ("num_blocks", i64), ("block_size", i64),
        ("in_stride_n", i64), ("in_stride_h", i64),
        ("cache_stride_blk", i64), ("cache_stride_h", i64), ("cache_stride_pos", i64),
        ("dtype", C.c_int), ("stream", vp),
    ]


class KvLookupArgs(C.Structure):
    _fields_ = [
        ("k_cache", vp), ("v_cache", vp), ("k_out", vp), ("v_out", vp), ("block_table", vp), ("context_lens", vp),
        ("batch", i64), ("num_kv_heads", i64), ("head_dim", i64), ("num_blocks", i64), ("block_size", i64),
        ("max_ctx", i64), ("max_blocks", i64),
        ("cache_stride_blk", i64), ("cache_stride_h", i64), ("cache_stride_pos", i64),
        ("bt_stride_b", i64),
        ("dtype", C.c_int), ("stream", vp),
    ]


class RopeArgs(C.Structure):
    _fields_ = [
        ("x", vp), ("y", vp), ("cos", vp), ("sin", vp),
        ("batch", i64), ("seq", i64), ("heads", i64), ("head_dim", i64),
        ("x_stride_b", i64), ("x_stride_s", i64), ("x_stride_h", i64),
        ("y_stride_b", i64), ("y_stride_s", i64), ("y_stride_h", i64),
        ("table_stride_s", i64),
        ("interleaved", C.c_int), ("dtype", C.c_int), ("stream", vp),
    ]


class RopeTableArgs(C.Structure):
    _fields_ = [
        ("cos", vp), ("sin", vp), ("inv_freq", vp),
        ("seq_len", i64), ("head_dim", i64), ("base", C.c_double),
        ("interleaved", C.c_int), ("dtype", C.c_int), ("stream", vp),
    ]


class RopeAppendArgs(C.Structure):
    _fields_ = [
        ("k_in", vp), ("v_in", vp), ("q_in", vp), ("q_out", vp), ("k_cache", vp), ("v_cache", vp),
        ("slot_mapping", vp), ("positions", vp), ("cos", vp), ("sin", vp),
        ("n_tokens", i64), ("num_q_heads", i64), ("num_kv_heads", i64), ("head_dim", i64),
        ("num_blocks", i64), ("block_size", i64), ("table_rows", i64),
        ("cache_stride_blk", i64), ("cache_stride_h", i64), ("cache_stride_pos", i64),
        ("interleaved", C.c_int), ("dtype", C.c_int), ("stream", vp),
        ("kv_int8", C.c_int), ("k_scales", vp), ("v_scales", vp),
    ]


class SoftmaxArgs(C.Structure):
    _fields_ = [
        ("x", vp), ("y", vp), ("rows", i64), ("n", i64),
        ("is_causal", C.c_int), ("log", C.c_int), ("dtype", C.c_int), ("stream", vp),
    ]


class AttentionArgs(C.Structure):
    _fields_ = [
        ("q", vp), ("k", vp), ("v", vp), ("out", vp), ("attn_mask", vp),
        ("batch", i64), ("num_q_heads", i64), ("num_kv_heads", i64), ("seq_q", i64), ("seq_k", i64),
        ("head_dim", i64),
        ("sm_scale", C.c_float), ("is_causal", C.c_int), ("dtype", C.c_int),
        ("workspace", vp), ("workspace_bytes", C.c_size_t), ("stream", vp),
    ]


class PagedAttentionArgs(C.Structure):
    _fields_ = [
        ("q", vp), ("out", vp), ("k_cache", vp), ("v_cache", vp), ("block_table", vp), ("context_lens", vp),
        ("q_start", vp), ("rope_cos", vp), ("rope_sin", vp), ("rope_positions", vp),
        ("n_q", i64), ("batch", i64), ("num_q_heads", i64), ("num_kv_heads", i64), ("head_dim", i64),
        ("num_blocks", i64), ("block_size", i64), ("max_blocks", i64), ("bt_stride_b", i64), ("table_rows", i64),
        ("max_q_len", i64),
        ("sm_scale", C.c_float), ("is_causal", C.c_int), ("rope_interleaved", C.c_int), ("dtype", C.c_int),
        ("reuse_plan", C.c_int), ("force_generic", C.c_int),
        ("target_chunk", i64),
        ("workspace", vp), ("workspace_bytes", C.c_size_t), ("stream", vp),
        ("kv_int8", C.c_int), ("k_scales", vp), ("v_scales", vp),
    ]


class CombineArgs(C.Structure):
    _fields_ = [
        ("acc", vp), ("m", vp), ("l", vp), ("split_begin", vp), ("out", vp),
        ("rows", i64), ("head_dim", i64), ("dtype", C.c_int), ("stream", vp),
    ]


class LinearNormArgs(C.Structure):
    _fields_ = [
        ("x", vp), ("weight", vp), ("bias", vp), ("gamma", vp), ("beta", vp), ("out", vp),
        ("M", i64), ("K", i64), ("N", i64),
        ("eps", C.c_float), ("norm_type", C.c_int), ("dtype", C.c_int), ("force_generic", C.c_int),
        ("workspace", vp), ("workspace_bytes", C.c_size_t), ("stream", vp),
    ]


RFX_MAX_PEERS = 16


class HeadGatherArgs(C.Structure):
    _fields_ = [
        ("world", C.c_int), ("rank", C.c_int),
        ("peer_out", vp * RFX_MAX_PEERS), ("peer_flags", vp * RFX_MAX_PEERS),
        ("arrival_counter", vp), ("epoch", C.c_uint32), ("wait", C.c_int), ("spin_limit", i64),
        ("epoch_word", vp), ("out_alt_offset", i64),
    ]


class PeerHandle(C.Structure):
    _fields_ = [("handle", C.c_ubyte * 64), ("offset", i64)]


# Every symbol include/reflex_b200.h declares: (name, restype, argtypes).
EXPORTS = {
    "rfx_abi_version": (C.c_int, []),
    "rfx_debug_set_flags": (C.c_int, [C.c_char_p]),
    "rfx_args_size": (C.c_size_t, [C.c_int]),
    "rfx_status_string": (C.c_char_p, [C.c_int]),
    "rfx_last_error": (C.c_char_p, []),
    "rfx_kv_paged_append": (C.c_int, [C.POINTER(KvAppendArgs)]),
    "rfx_kv_paged_scatter": (C.c_int, [C.POINTER(KvAppendArgs)]),
    "rfx_kv_paged_lookup": (C.c_int, [C.POINTER(KvLookupArgs)]),
    "rfx_rope_apply": (C.c_int, [C.POINTER(RopeArgs)]),
    "rfx_rope_build_tables": (C.c_int, [C.POINTER(RopeTableArgs)]),
    "rfx_rope_append": (C.c_int, [C.POINTER(RopeAppendArgs)]),
    "rfx_online_softmax": (C.c_int, [C.POINTER(SoftmaxArgs)]),
    "rfx_fused_attention_workspace_bytes": (C.c_size_t, [C.POINTER(AttentionArgs)]),
    "rfx_fused_attention": (C.c_int, [C.POINTER(AttentionArgs)]),
    "rfx_paged_attention_workspace_bytes": (C.c_size_t, [C.POINTER(PagedAttentionArgs)]),
    "rfx_paged_attention_plan": (C.c_int, [C.POINTER(PagedAttentionArgs)]),
    "rfx_paged_attention": (C.c_int, [C.POINTER(PagedAttentionArgs)]),
    "rfx_paged_attention_partials": (C.c_int, [C.POINTER(PagedAttentionArgs)]),
    "rfx_paged_attention_partials_final": (C.c_int, [C.POINTER(PagedAttentionArgs)]),
    "rfx_paged_attention_combine": (C.c_int, [C.POINTER(PagedAttentionArgs)]),
    "rfx_paged_attention_kernel_kind": (C.c_int, [C.POINTER(PagedAttentionArgs)]),
    "rfx_fused_attention_kernel_kind": (C.c_int, [C.POINTER(AttentionArgs)]),
    "rfx_paged_attention_static_capacity": (C.c_size_t, []),
    "rfx_paged_attention_static": (C.c_int, [C.POINTER(PagedAttentionArgs)]),
    "rfx_splitk_combine": (C.c_int, [C.POINTER(CombineArgs)]),
    "rfx_paged_attention_status": (C.c_int, [vp, vp, C.POINTER(C.c_int)]),
    "rfx_paged_attention_combine_gather": (C.c_int, [C.POINTER(PagedAttentionArgs), C.POINTER(HeadGatherArgs)]),
    "rfx_paged_attention_gather": (C.c_int, [C.POINTER(PagedAttentionArgs), C.POINTER(HeadGatherArgs)]),
    "rfx_peer_export": (C.c_int, [vp, C.POINTER(PeerHandle)]),
    "rfx_peer_open": (C.c_int, [C.POINTER(PeerHandle), C.POINTER(vp), C.POINTER(vp)]),
    "rfx_peer_close": (C.c_int, [vp]),
    "rfx_fused_linear_norm_workspace_bytes": (C.c_size_t, [C.POINTER(LinearNormArgs)]),
    "rfx_fused_linear_norm": (C.c_int, [C.POINTER(LinearNormArgs)]),
    "rfx_fused_linear_norm_kernel_kind": (C.c_int, [C.POINTER(LinearNormArgs)]),
}


# Index of each mirror in rfx_args_size().
ARG_STRUCTS = [KvAppendArgs, KvLookupArgs, RopeArgs, RopeTableArgs, RopeAppendArgs, SoftmaxArgs,
               AttentionArgs, PagedAttentionArgs, CombineArgs, HeadGatherArgs, PeerHandle, LinearNormArgs]


def library_path() -> Path:
    return Path(os.environ.get("REFLEX_B200_LIB", str(_LIB_PATH)))


def lib() -> C.CDLL:
    """Load the shared library once. Raises ``RuntimeError`` if it has not been built."""
    global _lib
    if _lib is None:
        path = library_path()
        if not path.exists():
            raise RuntimeError(
                f"{path} not found: build it with `python reflex-infer_b200/build.py` "
                "(there is no fallback implementation)"
            )
        handle = C.CDLL(str(path))
        for name, (restype, argtypes) in EXPORTS.items():
            fn = getattr(handle, name)
            fn.restype = restype
            fn.argtypes = argtypes
        for idx, mirror in enumerate(ARG_STRUCTS):
            if handle.rfx_args_size(idx) != C.sizeof(mirror):
                raise RuntimeError(
                    f"ABI mismatch: {mirror.__name__} is {C.sizeof(mirror)} B here, "
                    f"{handle.rfx_args_size(idx)} B in {path}"
                )
        _lib = handle
    return _lib


def check_backend(backend: Optional[str]) -> None:
    """``backend=`` is kept in every signature for drop-in compatibility; every accepted
    value runs the native library (reference validation: ``kernels/_common/launch.py:107-111``)."""
    if backend not in _VALID_BACKENDS:
        raise ValueError(f"backend={backend!r}; expected triton|cuda|torch")


def dtype_code(t: torch.Tensor) -> int:
    try:
        return _DTYPE_CODE[t.dtype]
    except KeyError:
        raise ValueError(f"unsupported dtype {t.dtype}; expected float32, bfloat16 or float16") from None


def require_cuda(name: str, *tensors: torch.Tensor) -> torch.device:
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError(f"{name} requires CUDA tensors (got a tensor on {t.device}); there is no CPU path")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise RuntimeError(f"{name}: tensors on different devices ({dev} and {t.device})")
    if dev is None:
        raise RuntimeError(f"{name}: no tensor arguments")
    return dev


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def stream_handle(dev: torch.device) -> int:
    return torch.cuda.current_stream(dev).cuda_stream


def check(status: int) -> None:
    if status == RFX_SUCCESS:
        return
    handle = lib()
    msg = handle.rfx_last_error().decode("utf-8", "replace")
    kind = handle.rfx_status_string(status).decode()
    if status == RFX_INVALID_ARGUMENT:
        raise ValueError(msg)
    raise RuntimeError(f"{kind}: {msg}")


def call(name: str, args: C.Structure, dev: torch.device) -> None:
    """Invoke an ``int f(const Args*)`` entry point with ``dev`` current."""
    fn = getattr(lib(), name)
    with torch.cuda.device(dev):
        check(fn(C.byref(args)))


def peer_export(device_ptr: int, dev: torch.device) -> bytes:
    """Handle (bytes, picklable) under which another process can map the allocation holding
    ``device_ptr``; see ``peer_open``."""
    h = PeerHandle()
    with torch.cuda.device(dev):
        check(lib().rfx_peer_export(device_ptr, C.byref(h)))
    return bytes(h)


def peer_open(handle: bytes, dev: torch.device):
    """Maps a buffer exported by another process. Returns ``(pointer, base)``; ``base`` goes to
    ``peer_close``."""
    h = PeerHandle.from_buffer_copy(handle)
    mapped, base = vp(), vp()
    with torch.cuda.device(dev):
        check(lib().rfx_peer_open(C.byref(h), C.byref(mapped), C.byref(base)))
    return int(mapped.value), int(base.value)


def peer_close(base: int, dev: torch.device) -> None:
    with torch.cuda.device(dev):
        check(lib().rfx_peer_close(base))
