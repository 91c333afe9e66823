"""The entry point that allocates nothing: ``rfx_paged_attention_static`` keeps its split-K
plan and partials in an array built into the library, for hosts that may not allocate
device memory when they run attention (all memory reserved up front, a foreign memory
pool, a latency-critical thread). Called through the C ABI twice in a row and compared
with the workspace-taking entry point on the same inputs. Collected last on purpose."""
from __future__ import annotations

import ctypes as C

import pytest
import torch

import workloads
from kernels import _native as N
from kernels.attention import PagedAttentionCall

pytestmark = [pytest.mark.gpu]
DEV = "cuda"


def _batch(seed):
    # the shape of the 32-request GQA decode configuration, shortened contexts
    return workloads.make_paged_batch("noalloc", B=32, Hq=16, Hkv=2, D=128, block_size=16, ctx_range=(64, 1500),
                                      num_blocks=4096, device=DEV, seed=seed)


def test_static_scratch_matches_workspace_path_twice(native):
    lib = native.lib()
    assert lib.rfx_paged_attention_static_capacity() == 8 << 20
    for seed in (21, 22):  # two calls in a row on different data: the second sees the first one's leftovers
        b = _batch(seed)
        ref_call = PagedAttentionCall(b.q_new, b.k_cache, b.v_cache, b.block_table, b.context_lens,
                                      rope_cos=b.cos, rope_sin=b.sin, rope_positions=b.positions)
        want = ref_call.run().clone()
        out = torch.full_like(want, float("nan"))
        call = PagedAttentionCall(b.q_new, b.k_cache, b.v_cache, b.block_table, b.context_lens,
                                  rope_cos=b.cos, rope_sin=b.sin, rope_positions=b.positions, out=out)
        args = call._args
        args.workspace = None          # the entry point must not need it
        args.workspace_bytes = 0
        args.stream = N.stream_handle(torch.device(DEV, torch.cuda.current_device()))
        status = lib.rfx_paged_attention_static(C.byref(args))
        torch.cuda.synchronize()
        assert status == N.RFX_SUCCESS, lib.rfx_last_error()
        assert torch.isfinite(out).all()
        torch.testing.assert_close(out.float(), want.float(), atol=2e-2, rtol=2e-2)
        first = out.clone()
        # Once the array's address is known (the very first call on a device makes the
        # driver load it), a call leaves the amount of free device memory untouched.
        out.fill_(float("nan"))
        free_before = torch.cuda.mem_get_info()[0]
        status = lib.rfx_paged_attention_static(C.byref(args))
        torch.cuda.synchronize()
        assert status == N.RFX_SUCCESS, lib.rfx_last_error()
        assert torch.cuda.mem_get_info()[0] == free_before, "the call changed the amount of free device memory"
        assert torch.equal(out, first)
        assert torch.equal(call.run_static(), first)
        # the status word of the built-in array (bad page, expired wait, capacity): a NULL workspace asks for it
        word = C.c_int(-1)
        assert lib.rfx_paged_attention_status(None, args.stream, C.byref(word)) == N.RFX_SUCCESS
        assert word.value == 0


def test_static_scratch_rejects_oversized_problems(native):
    lib = native.lib()
    b = workloads.make_paged_batch("big", B=512, Hq=64, Hkv=8, D=128, block_size=32, ctx_range=(1, 40),
                                   num_blocks=1024, device=DEV, seed=3)
    call = PagedAttentionCall(b.q_new, b.k_cache, b.v_cache, b.block_table, b.context_lens)
    with pytest.raises(RuntimeError, match="WorkspaceTooSmall.*built-in array"):
        call.run_static()
    call.run()  # the same problem is fine with a caller workspace
