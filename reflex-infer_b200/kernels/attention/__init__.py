"""Attention; ``fused_attention`` keeps the reference's surface
(``kernels/attention/__init__.py:86-123``) and the paged entry points fuse the
composition the reference spells as lookup -> attention.

Dense:
    ``fused_attention(q, k, v, *, is_causal, attn_mask, sm_scale, backend)``

Paged (additive; none of them changes the functions above):
    ``rope_append``        RoPE on new K (and optionally Q) + write K, V into the pool
    ``paged_attention``    split-K attention straight from the pool, ragged query chunks,
                           bottom-right causal, optional RoPE fused into the Q load
    ``paged_decode``       the one-row-per-request case of ``paged_attention``
    ``paged_decode_step``  ``rope_append`` + ``paged_decode`` for one decode step
    ``PagedWorkspace``     caller-owned scratch for the split-K plan and partials
    ``splitk_combine``     merge caller-provided (m, l, acc) partials

int8 KV: a pool whose caches are ``torch.int8`` with fp32 scales ``[num_blocks, H_kv, block_size]``
(one per position and kv head, the reference's ``kv_int8`` / ``k_scales`` / ``v_scales`` of
``include/reflex/infer.h:189-203`` on pages). ``rope_append`` quantises on the way in
(``scale = max|row| / 127``, ``q = round(row / scale)``), the paged entry points take
``k_scales=`` / ``v_scales=``; ``int8_pool`` allocates such a pool.
"""
from __future__ import annotations

import ctypes as C
import math
from typing import Optional

import torch

from .. import _native as N


def _resolve_head_repeat(num_heads_q: int, num_heads_kv: int) -> int:
    if num_heads_q % num_heads_kv != 0:
        raise ValueError(
            f"GQA requires num_heads_q ({num_heads_q}) divisible by "
            f"num_heads_kv ({num_heads_kv})"
        )
    return num_heads_q // num_heads_kv


def fused_attention(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    *,
    is_causal: bool = False,
    attn_mask: Optional[torch.Tensor] = None,
    sm_scale: Optional[float] = None,
    backend: Optional[str] = None,
) -> torch.Tensor:
    """``softmax(q k^T * sm_scale + attn_mask) v`` with in-kernel GQA.

    ``q``: ``[B, H, S_q, D]``; ``k``, ``v``: ``[B, H_kv, S_k, D]`` with ``H % H_kv == 0`` (query
    head ``h`` reads kv head ``h // (H/H_kv)``, ``triton_fused_attention.py:130-132``);
    ``is_causal`` masks ``key > query`` (top-left aligned, ``:185-187``); ``attn_mask`` is an
    additive ``[B, H, S_q, S_k]`` bias (bool masks and broadcastable shapes are expanded);
    ``sm_scale`` defaults to ``1/sqrt(D)``. Output ``[B, H, S_q, D]`` in ``q``'s dtype.
    """
    N.check_backend(backend)
    if q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
        raise ValueError(f"shape mismatch q={tuple(q.shape)} k={tuple(k.shape)} v={tuple(v.shape)}")
    if not q.is_cuda:
        raise RuntimeError("fused_attention requires a CUDA tensor")
    dev = N.require_cuda("fused_attention", q, k, v, attn_mask)
    B, H, S_q, D = q.shape
    Bk, Hk, S_k, Dk = k.shape
    Bv, Hv, S_v, Dv = v.shape
    if (B, S_k, D) != (Bk, S_k, Dk) or (B, S_k, D) != (Bv, S_v, Dv):
        raise ValueError(f"shape mismatch q={q.shape} k={k.shape} v={v.shape}")
    if Hk != Hv:
        raise ValueError(f"K/V head count mismatch: {Hk} vs {Hv}")
    _resolve_head_repeat(H, Hk)
    if k.dtype != q.dtype or v.dtype != q.dtype:
        raise RuntimeError(f"q, k, v dtypes differ: {q.dtype}, {k.dtype}, {v.dtype}")
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(D)
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    if attn_mask is not None:
        if attn_mask.dtype == torch.bool:
            attn_mask = torch.zeros(attn_mask.shape, dtype=q.dtype, device=dev).masked_fill_(~attn_mask, float("-inf"))
        try:
            attn_mask = attn_mask.expand(B, H, S_q, S_k)
        except RuntimeError:
            raise ValueError(
                f"attn_mask must be [{B},{H},{S_q},{S_k}], got {tuple(attn_mask.shape)}"
            ) from None
        attn_mask = attn_mask.to(q.dtype).contiguous()
    out = torch.empty_like(q)
    a = N.AttentionArgs(
        q=N.ptr(q), k=N.ptr(k), v=N.ptr(v), out=N.ptr(out), attn_mask=N.ptr(attn_mask),
        batch=B, num_q_heads=H, num_kv_heads=Hk, seq_q=S_q, seq_k=S_k, head_dim=D,
        sm_scale=float(sm_scale), is_causal=int(bool(is_causal)), dtype=N.dtype_code(q),
        workspace=None, workspace_bytes=0, stream=N.stream_handle(dev),
    )
    global last_dense_kernel_kind
    last_dense_kernel_kind = int(N.lib().rfx_fused_attention_kernel_kind(C.byref(a)))
    N.call("rfx_fused_attention", a, dev)
    return out


#: Which kernel the last ``fused_attention`` call selected: 1 = tcgen05 kernel, 0 = scalar kernel.
last_dense_kernel_kind = -1


# ---------------------------------------------------------------------------- paged ----

class PagedWorkspace:
    """Caller-owned scratch of one paged-attention problem size (plan + split-K partials).

    The native library never allocates; this object asks it for the size and keeps a
    ``torch.uint8`` buffer. Reuse it across steps and layers of the same shape.
    """

    def __init__(self, device: torch.device):
        self.device = torch.device(device)
        self.buffer: Optional[torch.Tensor] = None

    def ensure(self, nbytes: int) -> torch.Tensor:
        if self.buffer is None or self.buffer.numel() < nbytes:
            self.buffer = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
        return self.buffer

    def status(self) -> int:
        """Device status word of the last launch (0 = clean). Synchronises the stream."""
        import ctypes as C
        if self.buffer is None:
            return 0
        word = C.c_int(0)
        with torch.cuda.device(self.device):
            st = N.lib().rfx_paged_attention_status(self.buffer.data_ptr(), N.stream_handle(self.device), C.byref(word))
        if st not in (N.RFX_SUCCESS, N.RFX_TIMEOUT):
            N.check(st)
        return int(word.value)


class PagedAttentionCall:
    """A validated, ready-to-launch paged attention over fixed buffers.

    Construction does all argument checking, dtype/stride normalisation and workspace
    sizing once; ``run()`` (plan + partials + combine) and the single stages then cost one
    foreign call each, which is what a serving loop that reuses its buffers every step
    wants. The tensors are referenced, not copied: refill them in place between calls.
    """

    def __init__(self, q, k_cache, v_cache, block_table, context_lens, *, q_start=None, max_q_len=None,
                 is_causal=True, sm_scale=None, rope_cos=None, rope_sin=None, rope_positions=None,
                 rope_interleaved=False, workspace=None, out=None, force_generic=False, target_chunk=0,
                 k_scales=None, v_scales=None):
        import ctypes as C
        name = "paged_attention"
        dev = N.require_cuda(name, q, k_cache, v_cache, block_table, context_lens, q_start, rope_cos, rope_sin,
                             rope_positions, out, k_scales, v_scales)
        if q.dim() != 3:
            raise ValueError(f"{name}: q must be [N_q, H_q, D], got {tuple(q.shape)}")
        if k_cache.dim() != 4 or v_cache.shape != k_cache.shape:
            raise ValueError(f"{name}: caches must both be [num_blocks, H_kv, block_size, D]")
        n_q, Hq, D = q.shape
        nb, Hkv, bs, Dc = k_cache.shape
        if Dc != D:
            raise ValueError(f"{name}: head_dim of q ({D}) and cache ({Dc}) differ")
        _resolve_head_repeat(Hq, Hkv)
        kv_int8 = k_cache.dtype == torch.int8
        if kv_int8:
            if v_cache.dtype != torch.int8 or k_scales is None or v_scales is None:
                raise ValueError(f"{name}: an int8 pool needs int8 k_cache and v_cache and k_scales, v_scales")
            for t in (k_scales, v_scales):
                if t.dtype != torch.float32 or tuple(t.shape) != (nb, Hkv, bs) or not t.is_contiguous():
                    raise ValueError(f"{name}: scales must be contiguous float32 [{nb}, {Hkv}, {bs}]")
        elif k_cache.dtype != q.dtype or v_cache.dtype != q.dtype:
            raise RuntimeError(f"{name}: q dtype {q.dtype} differs from the cache dtype {k_cache.dtype}")
        if not (k_cache.is_contiguous() and v_cache.is_contiguous()):
            raise ValueError(f"{name}: the caches must be contiguous")
        q = q.contiguous()
        if block_table.dtype != torch.int64:
            block_table = block_table.to(torch.int64)
        if block_table.dim() != 2 or block_table.stride(1) != 1:
            block_table = block_table.contiguous()
        if context_lens.dtype != torch.int32:
            context_lens = context_lens.to(torch.int32)
        context_lens = context_lens.contiguous()
        B = context_lens.shape[0]
        if block_table.shape[0] != B:
            raise ValueError(f"{name}: block_table has {block_table.shape[0]} rows, context_lens {B}")
        if q_start is not None:
            if q_start.shape != (B + 1,):
                raise ValueError(f"{name}: q_start must be [B+1]={B + 1}, got {tuple(q_start.shape)}")
            q_start = q_start.to(torch.int32).contiguous()
        elif n_q != B:
            raise ValueError(f"{name}: without q_start q needs one row per request ({B}), got {n_q}")
        if (rope_cos is None) != (rope_sin is None):
            raise ValueError(f"{name}: rope_cos and rope_sin go together")
        if rope_cos is not None:
            if rope_positions is None or rope_positions.shape != (n_q,):
                raise ValueError(f"{name}: rope_positions must be [N_q]={n_q}")
            rope_positions = rope_positions.to(torch.int32).contiguous()
            rope_cos = rope_cos.to(q.dtype).contiguous()
            rope_sin = rope_sin.to(q.dtype).contiguous()
            if rope_cos.dim() != 2 or rope_cos.shape[1] != D or rope_sin.shape != rope_cos.shape:
                raise ValueError(f"{name}: rope tables must be [rows, {D}]")
        if max_q_len is None:
            # No request can own more rows than there are: a safe bound that needs no device read.
            max_q_len = max(1, n_q) if q_start is not None else 1
        if int(max_q_len) < 1:
            raise ValueError(f"{name}: max_q_len must be >= 1, got {max_q_len}")
        if sm_scale is None:
            sm_scale = 1.0 / math.sqrt(D)
        if out is None:
            out = torch.empty_like(q)
        elif out.shape != q.shape or out.dtype != q.dtype or not out.is_contiguous():
            raise ValueError(f"{name}: out must be a contiguous tensor shaped like q")
        if workspace is None:
            workspace = PagedWorkspace(dev)
        a = N.PagedAttentionArgs(
            q=N.ptr(q), out=N.ptr(out), k_cache=N.ptr(k_cache), v_cache=N.ptr(v_cache),
            block_table=N.ptr(block_table), context_lens=N.ptr(context_lens), q_start=N.ptr(q_start),
            rope_cos=N.ptr(rope_cos), rope_sin=N.ptr(rope_sin), rope_positions=N.ptr(rope_positions),
            n_q=n_q, batch=B, num_q_heads=Hq, num_kv_heads=Hkv, head_dim=D,
            num_blocks=nb, block_size=bs, max_blocks=block_table.shape[1], bt_stride_b=block_table.stride(0),
            table_rows=0 if rope_cos is None else rope_cos.shape[0],
            max_q_len=int(max_q_len),
            sm_scale=float(sm_scale), is_causal=int(bool(is_causal)), rope_interleaved=int(bool(rope_interleaved)),
            dtype=N.dtype_code(q), reuse_plan=0, force_generic=int(bool(force_generic)),
            target_chunk=int(target_chunk), workspace=None, workspace_bytes=0, stream=None,
            kv_int8=int(kv_int8), k_scales=N.ptr(k_scales) if kv_int8 else None,
            v_scales=N.ptr(v_scales) if kv_int8 else None,
        )
        lib = N.lib()
        need = lib.rfx_paged_attention_workspace_bytes(C.byref(a))
        if need == 0 and n_q > 0:
            N.check(N.RFX_INVALID_ARGUMENT)
        buf = workspace.ensure(max(int(need), 256))
        a.workspace = buf.data_ptr()
        a.workspace_bytes = buf.numel()
        self.kernel_kind = int(lib.rfx_paged_attention_kernel_kind(C.byref(a)))  # 3/2 tcgen05 (3: one-row requests on the decode kernel), 1 TMA/MMA decode, 0 scalar
        self.out = out
        self.workspace = workspace
        self.device = dev
        self._args = a
        self._ref = C.byref(a)
        self._lib = lib
        self._keep = (q, k_cache, v_cache, block_table, context_lens, q_start, rope_cos, rope_sin, rope_positions, buf,
                      k_scales, v_scales)

    def _call(self, fn):
        self._args.stream = N.stream_handle(self.device)
        with torch.cuda.device(self.device):
            N.check(fn(self._ref))

    def run(self, reuse_plan: bool = False) -> torch.Tensor:
        """plan (unless ``reuse_plan``) + split-K partials + combine."""
        self._args.reuse_plan = int(bool(reuse_plan))
        self._call(self._lib.rfx_paged_attention)
        return self.out

    def run_static(self) -> torch.Tensor:
        """Same result as ``run()``, but the plan and the split-K partials go to the 8 MiB
        scratch array built into the library instead of this call's workspace, and nothing
        is allocated. For hosts that may not allocate device memory when they run attention
        (memory handed out up front, a foreign memory pool, a latency-critical thread).
        Raises ``RuntimeError`` (WorkspaceTooSmall) when the problem needs more than the
        array holds. All callers on a GPU share the array, so calls must not overlap there."""
        self._call(self._lib.rfx_paged_attention_static)
        return self.out

    def plan(self) -> None:
        self._call(self._lib.rfx_paged_attention_plan)

    def partials(self) -> None:
        self._call(self._lib.rfx_paged_attention_partials)

    def partials_final(self) -> torch.Tensor:
        """The decode kernel alone (``kernel_kind == 1``) over the existing plan, finishing its rows
        itself: no ``combine()`` follows. This is what ``run()`` launches after the plan."""
        self._call(self._lib.rfx_paged_attention_partials_final)
        return self.out

    def combine(self) -> torch.Tensor:
        self._call(self._lib.rfx_paged_attention_combine)
        return self.out

    def run_gather(self, gather, reuse_plan: bool = False) -> torch.Tensor:
        """``run()`` for a rank that holds a slice of the heads: the combine kernel stores this
        rank's heads into every rank's full output and the ranks meet inside the kernel
        (``gather``: a ``sharding.FusedHeadGather``). Returns this rank's full ``[N, H_q_total, D]``
        output of the step; it stays valid until the step after the next one."""
        import ctypes as C
        g, full = gather.next_args()
        self._args.reuse_plan = int(bool(reuse_plan))
        self._args.stream = N.stream_handle(self.device)
        with torch.cuda.device(self.device):
            N.check(self._lib.rfx_paged_attention_gather(self._ref, C.byref(g)))
        return full

    def run_gather_replayable(self, gather) -> None:
        """``run_gather`` in the form a CUDA graph can replay: nothing in the launch arguments changes
        from step to step (``gather.replayable_args()``); the n-th launch leaves its result in
        ``gather.output_of(n)``."""
        import ctypes as C
        g = gather.replayable_args()
        self._args.reuse_plan = 0
        self._args.stream = N.stream_handle(self.device)
        with torch.cuda.device(self.device):
            N.check(self._lib.rfx_paged_attention_gather(self._ref, C.byref(g)))

    def combine_gather(self, gather) -> torch.Tensor:
        """The combine stage alone, with the gather (after ``plan()`` and ``partials()``)."""
        import ctypes as C
        g, full = gather.next_args()
        self._args.stream = N.stream_handle(self.device)
        with torch.cuda.device(self.device):
            N.check(self._lib.rfx_paged_attention_combine_gather(self._ref, C.byref(g)))
        return full


def paged_attention(
    q: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    block_table: torch.Tensor,
    context_lens: torch.Tensor,
    *,
    q_start: Optional[torch.Tensor] = None,
    max_q_len: Optional[int] = None,
    is_causal: bool = True,
    sm_scale: Optional[float] = None,
    rope_cos: Optional[torch.Tensor] = None,
    rope_sin: Optional[torch.Tensor] = None,
    rope_positions: Optional[torch.Tensor] = None,
    rope_interleaved: bool = False,
    workspace: Optional[PagedWorkspace] = None,
    out: Optional[torch.Tensor] = None,
    reuse_plan: bool = False,
    force_generic: bool = False,
    target_chunk: int = 0,
    k_scales: Optional[torch.Tensor] = None,
    v_scales: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """Attention of ragged query chunks over the paged pool.

    ``q``: ``[N_q, H_q, D]``; request ``b`` owns rows ``q_start[b]:q_start[b+1]`` (one row per
    request when ``q_start`` is None) and keys ``0..context_lens[b]-1``, which include the
    request's new tokens (append first). With ``is_causal`` row ``i`` of ``n_b`` sees keys
    ``0..context_lens[b]-n_b+i`` (bottom-right aligned). Equals, per request,
    ``fused_attention(q_b, *kv_paged_lookup(..., max_ctx=context_lens[b]))`` with GQA
    expansion. ``max_q_len`` is a host-side upper bound of any request's row count (sizes
    the workspace and the grid; default: ``N_q`` when ``q_start`` is given, else 1). If a
    request turns out to own more rows than that, or ``q_start[B] - q_start[0] != N_q``, nothing is
    computed, the output rows are zero or left as they were, and bit 2 of the workspace status
    word is set. Pass ``rope_cos/rope_sin/rope_positions`` to rotate Q on load.
    """
    call = PagedAttentionCall(q, k_cache, v_cache, block_table, context_lens, q_start=q_start, max_q_len=max_q_len,
                              is_causal=is_causal, sm_scale=sm_scale, rope_cos=rope_cos, rope_sin=rope_sin,
                              rope_positions=rope_positions, rope_interleaved=rope_interleaved, workspace=workspace,
                              out=out, force_generic=force_generic, target_chunk=target_chunk,
                              k_scales=k_scales, v_scales=v_scales)
    return call.run(reuse_plan=reuse_plan)


def paged_decode(q, k_cache, v_cache, block_table, context_lens, **kw) -> torch.Tensor:
    """One query row per request (``q``: ``[B, H_q, D]``): the decode case of ``paged_attention``."""
    kw.pop("q_start", None)
    kw.setdefault("max_q_len", 1)
    return paged_attention(q, k_cache, v_cache, block_table, context_lens, q_start=None, **kw)


class RopeAppendCall:
    """A validated, ready-to-launch fused RoPE + append over fixed buffers (see ``rope_append``)."""

    def __init__(self, k_new, v_new, k_cache, v_cache, slot_mapping, positions, cos, sin, *, q=None, q_out=None,
                 interleaved=False, k_scales=None, v_scales=None):
        import ctypes as C
        name = "rope_append"
        dev = N.require_cuda(name, k_new, v_new, k_cache, v_cache, slot_mapping, positions, cos, sin, q, q_out,
                             k_scales, v_scales)
        if k_new.dim() != 3 or v_new.shape != k_new.shape:
            raise ValueError(f"{name}: k_new and v_new must both be [N, H_kv, D]")
        n, Hkv, D = k_new.shape
        if k_cache.dim() != 4 or v_cache.shape != k_cache.shape or k_cache.stride() != v_cache.stride():
            raise ValueError(f"{name}: caches must both be [num_blocks, H_kv, block_size, D] with one stride pattern")
        nb, ch, bs, cd = k_cache.shape
        if (Hkv, D) != (ch, cd):
            raise ValueError(f"{name}: input heads/head_dim {(Hkv, D)} do not match the cache {(ch, cd)}")
        if k_cache.stride(3) != 1:
            raise ValueError(f"{name}: the head_dim axis of the caches must be contiguous")
        if D % 2 != 0:
            raise ValueError("head_dim must be even for RoPE")
        kv_int8 = k_cache.dtype == torch.int8
        if kv_int8:
            if v_cache.dtype != torch.int8 or k_scales is None or v_scales is None:
                raise ValueError(f"{name}: an int8 pool needs int8 k_cache and v_cache and k_scales, v_scales")
            if not (k_cache.is_contiguous() and v_cache.is_contiguous()):
                raise ValueError(f"{name}: an int8 pool must be contiguous")
            for t in (k_scales, v_scales):
                if t.dtype != torch.float32 or tuple(t.shape) != (nb, ch, bs) or not t.is_contiguous():
                    raise ValueError(f"{name}: scales must be contiguous float32 [{nb}, {ch}, {bs}]")
            if v_new.dtype != k_new.dtype:
                raise RuntimeError(f"{name}: k_new and v_new dtypes differ")
        elif k_new.dtype != k_cache.dtype or v_new.dtype != k_cache.dtype:
            raise RuntimeError(f"{name}: input dtype {k_new.dtype} does not match cache dtype {k_cache.dtype}")
        k_new, v_new = k_new.contiguous(), v_new.contiguous()
        slot_mapping = slot_mapping.to(torch.int64).contiguous()
        positions = positions.to(torch.int32).contiguous()
        if slot_mapping.shape != (n,) or positions.shape != (n,):
            raise ValueError(f"{name}: slot_mapping and positions must be [N]={n}")
        cos = cos.to(k_new.dtype).contiguous()
        sin = sin.to(k_new.dtype).contiguous()
        if cos.dim() != 2 or cos.shape[1] != D or sin.shape != cos.shape:
            raise ValueError(f"{name}: rope tables must be [rows, {D}]")
        Hq = 0
        if q is not None:
            if q.dim() != 3 or q.shape[0] != n or q.shape[2] != D or q.dtype != k_new.dtype:
                raise ValueError(f"{name}: q must be [N, H_q, D] in the activation dtype")
            q = q.contiguous()
            Hq = q.shape[1]
            if q_out is None:
                q_out = torch.empty_like(q)
            elif q_out.shape != q.shape or q_out.dtype != q.dtype or not q_out.is_contiguous():
                raise ValueError(f"{name}: q_out must be a contiguous tensor shaped like q")
        else:
            q_out = None
        self._args = N.RopeAppendArgs(
            k_in=N.ptr(k_new), v_in=N.ptr(v_new), q_in=N.ptr(q), q_out=N.ptr(q_out),
            k_cache=N.ptr(k_cache), v_cache=N.ptr(v_cache), slot_mapping=N.ptr(slot_mapping),
            positions=N.ptr(positions), cos=N.ptr(cos), sin=N.ptr(sin),
            n_tokens=n, num_q_heads=Hq, num_kv_heads=Hkv, head_dim=D, num_blocks=nb, block_size=bs,
            table_rows=cos.shape[0],
            cache_stride_blk=k_cache.stride(0), cache_stride_h=k_cache.stride(1), cache_stride_pos=k_cache.stride(2),
            interleaved=int(bool(interleaved)), dtype=N.dtype_code(k_new), stream=None,
            kv_int8=int(kv_int8), k_scales=N.ptr(k_scales) if kv_int8 else None,
            v_scales=N.ptr(v_scales) if kv_int8 else None,
        )
        self._ref = C.byref(self._args)
        self._fn = N.lib().rfx_rope_append
        self.device = dev
        self.q_out = q_out
        self._keep = (k_new, v_new, q, k_cache, v_cache, slot_mapping, positions, cos, sin, k_scales, v_scales)

    def run(self) -> Optional[torch.Tensor]:
        self._args.stream = N.stream_handle(self.device)
        with torch.cuda.device(self.device):
            N.check(self._fn(self._ref))
        return self.q_out


def rope_append(
    k_new: torch.Tensor,
    v_new: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    slot_mapping: torch.Tensor,
    positions: torch.Tensor,
    cos: torch.Tensor,
    sin: torch.Tensor,
    *,
    q: Optional[torch.Tensor] = None,
    q_out: Optional[torch.Tensor] = None,
    interleaved: bool = False,
    k_scales: Optional[torch.Tensor] = None,
    v_scales: Optional[torch.Tensor] = None,
) -> Optional[torch.Tensor]:
    """Rotate ``k_new`` with table rows ``positions`` and write it and ``v_new`` into the
    pool at ``slot_mapping`` in one launch; with ``q`` also returns the rotated queries.

    Pool contents equal ``kv_paged_append(apply_rope(k_new...), v_new, ...)`` of the
    reference bit for bit (tables in the activation dtype). With an int8 pool (``torch.int8``
    caches plus ``k_scales`` / ``v_scales``) the rotated K rows and the V rows are quantised
    row by row: ``scale = max|row| / 127`` (1 for an all-zero row), ``q = round(row / scale)``.
    """
    return RopeAppendCall(k_new, v_new, k_cache, v_cache, slot_mapping, positions, cos, sin, q=q, q_out=q_out,
                          interleaved=interleaved, k_scales=k_scales, v_scales=v_scales).run()


def int8_pool(num_blocks: int, num_kv_heads: int, block_size: int, head_dim: int, device):
    """An empty int8 KV pool: ``(k_cache, v_cache, k_scales, v_scales)``, caches
    ``[num_blocks, H_kv, block_size, D]`` int8, scales ``[num_blocks, H_kv, block_size]`` float32."""
    k = torch.zeros((num_blocks, num_kv_heads, block_size, head_dim), dtype=torch.int8, device=device)
    ks = torch.ones((num_blocks, num_kv_heads, block_size), dtype=torch.float32, device=device)
    return k, torch.zeros_like(k), ks, torch.ones_like(ks)


def paged_decode_step(
    q_new: torch.Tensor,
    k_new: torch.Tensor,
    v_new: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    block_table: torch.Tensor,
    context_lens: torch.Tensor,
    slot_mapping: torch.Tensor,
    positions: torch.Tensor,
    cos: torch.Tensor,
    sin: torch.Tensor,
    *,
    sm_scale: Optional[float] = None,
    interleaved: bool = False,
    workspace: Optional[PagedWorkspace] = None,
    out: Optional[torch.Tensor] = None,
    k_scales: Optional[torch.Tensor] = None,
    v_scales: Optional[torch.Tensor] = None,
    **kw,
) -> torch.Tensor:
    """One decode step of one layer: append the new token's rotated K and its V to the
    pool, then attend the rotated query over ``context_lens`` keys (which count the new
    token). Three launches on top of the plan: RoPE+append, split-K partials with RoPE
    fused into the Q load, combine."""
    rope_append(k_new, v_new, k_cache, v_cache, slot_mapping, positions, cos, sin, interleaved=interleaved,
                k_scales=k_scales, v_scales=v_scales)
    return paged_decode(q_new, k_cache, v_cache, block_table, context_lens, sm_scale=sm_scale,
                        rope_cos=cos, rope_sin=sin, rope_positions=positions, rope_interleaved=interleaved,
                        workspace=workspace, out=out, k_scales=k_scales, v_scales=v_scales, **kw)


def splitk_combine(acc: torch.Tensor, m: torch.Tensor, l: torch.Tensor, split_begin: torch.Tensor,
                   *, dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """Merge split-K partials: rows ``r`` own partials ``split_begin[r]:split_begin[r+1]``;
    ``acc`` ``[P, D]`` fp32 un-normalised, ``m`` ``[P]`` maxima (natural-log domain), ``l`` ``[P]``
    sums. Returns ``[rows, D]`` in ``dtype``. The running-max recurrence of the reference
    (``kernels/softmax/triton_softmax.py:84-89``) applied across splits."""
    dev = N.require_cuda("splitk_combine", acc, m, l, split_begin)
    if acc.dim() != 2 or acc.dtype != torch.float32 or m.dtype != torch.float32 or l.dtype != torch.float32:
        raise ValueError("splitk_combine: acc [P, D], m [P], l [P] must be float32")
    acc, m, l = acc.contiguous(), m.contiguous(), l.contiguous()
    split_begin = split_begin.to(torch.int32).contiguous()
    rows = split_begin.shape[0] - 1
    out = torch.empty((rows, acc.shape[1]), dtype=dtype, device=dev)
    a = N.CombineArgs(acc=N.ptr(acc), m=N.ptr(m), l=N.ptr(l), split_begin=N.ptr(split_begin), out=N.ptr(out),
                      rows=rows, head_dim=acc.shape[1], dtype=N.dtype_code(out), stream=N.stream_handle(dev))
    N.call("rfx_splitk_combine", a, dev)
    return out


__all__ = [
    "fused_attention",
    "paged_attention",
    "paged_decode",
    "paged_decode_step",
    "rope_append",
    "splitk_combine",
    "int8_pool",
    "PagedWorkspace",
    "PagedAttentionCall",
    "RopeAppendCall",
]
