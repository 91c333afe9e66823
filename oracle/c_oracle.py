"""ctypes loader of the plain-C oracle (``paged_oracle.c``). Test infrastructure only."""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIB = HERE / "_build" / "libpaged_oracle.so"


def build() -> Path:
    subprocess.run(["make", "-s", "-C", str(HERE)], check=True)
    return LIB


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not LIB.exists():
            build()
        _lib = C.CDLL(str(LIB))
        _lib.oracle_kv_append.restype = C.c_int
        _lib.oracle_kv_lookup.restype = C.c_int
    return _lib


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def kv_append(k_in, v_in, k_cache, v_cache, slots) -> int:
    """numpy arrays of any 2- or 4-byte dtype; caches mutated in place."""
    n, heads, dim = k_in.shape
    nb, _, bs, _ = k_cache.shape
    slots = np.ascontiguousarray(slots, dtype=np.int64)
    return lib().oracle_kv_append(_p(np.ascontiguousarray(k_in)), _p(np.ascontiguousarray(v_in)), _p(k_cache),
                                  _p(v_cache), _p(slots), C.c_int64(n), C.c_int64(heads), C.c_int64(dim),
                                  C.c_int64(nb), C.c_int64(bs), C.c_int64(k_in.dtype.itemsize))


def kv_lookup(k_cache, v_cache, block_table, ctx, max_ctx):
    nb, heads, bs, dim = k_cache.shape
    B = ctx.shape[0]
    bt = np.ascontiguousarray(block_table, dtype=np.int64)
    cl = np.ascontiguousarray(ctx, dtype=np.int32)
    k_out = np.empty((B, heads, max_ctx, dim), dtype=k_cache.dtype)
    v_out = np.empty_like(k_out)
    rc = lib().oracle_kv_lookup(_p(k_cache), _p(v_cache), _p(k_out), _p(v_out), _p(bt), _p(cl), C.c_int64(B),
                                C.c_int64(heads), C.c_int64(dim), C.c_int64(nb), C.c_int64(bs), C.c_int64(max_ctx),
                                C.c_int64(bt.shape[1]), C.c_int64(k_cache.dtype.itemsize))
    if rc != 0:
        raise IndexError("page or position out of range")
    return k_out, v_out


def rope_bf16(x_bits, cos_bits, sin_bits, pos, interleaved=False):
    """x_bits [rows, dim] uint16 bf16 patterns; tables [T, dim] uint16; pos [rows] int32."""
    x_bits = np.ascontiguousarray(x_bits, dtype=np.uint16)
    y = np.empty_like(x_bits)
    pos = np.ascontiguousarray(pos, dtype=np.int32)
    lib().oracle_rope_bf16(_p(x_bits), _p(y), _p(np.ascontiguousarray(cos_bits, dtype=np.uint16)),
                           _p(np.ascontiguousarray(sin_bits, dtype=np.uint16)), _p(pos), C.c_int64(x_bits.shape[0]),
                           C.c_int64(x_bits.shape[1]), C.c_int(int(interleaved)))
    return y


def attention_row_f64(q, k, v, scale):
    q = np.ascontiguousarray(q, dtype=np.float32)
    k = np.ascontiguousarray(k, dtype=np.float32)
    v = np.ascontiguousarray(v, dtype=np.float32)
    out = np.empty(q.shape[0], dtype=np.float64)
    lib().oracle_attention_row_f64(_p(q), _p(k), _p(v), C.c_int64(k.shape[0]), C.c_int64(q.shape[0]),
                                   C.c_double(scale), _p(out))
    return out
