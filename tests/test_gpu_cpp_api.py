"""The C++ face of the library (include/reflex_b200.hpp, in the style of the reference's
include/reflex/infer.h:189-203,270-282) driven on the GPU: a small translation unit compiled with
g++ calls reflex::b200::paged_flash_attention_decode on device buffers this test wrote, for a
16-bit and for an int8 pool, and the result is compared with the CPU oracle. The compiled code is
loaded into this process (a shared object with one extern "C" shim) so that it can be handed the
device pointers."""
from __future__ import annotations

import ctypes as C
import shutil
import subprocess
from pathlib import Path

import pytest
import torch

import oracle
import workloads
from kernels.attention import rope_append

pytestmark = [pytest.mark.gpu]
DEV = "cuda"
ROOT = Path(__file__).resolve().parent.parent

SHIM = r'''
#include "reflex_b200.hpp"
namespace rb = reflex::b200;
extern "C" int run_decode(void* out, const void* q, const void* kc, const void* vc, const long long* bt,
                          const int* lens, int batch, int heads, int kv_heads, long long num_blocks, int block_size,
                          int max_blocks, float scale, const float* ks, const float* vs, void* ws, size_t ws_bytes,
                          void* stream, size_t* need) {
    if (!rb::kernel_support().paged_decode_attention || !rb::kernel_support().kv_convert) return -1;
    rb::PagedAttentionDecodeArgs a;
    a.output = out; a.q = q; a.k_cache = kc; a.v_cache = vc;
    a.block_table = reinterpret_cast<const std::int64_t*>(bt); a.context_lens = lens;
    a.batch = batch; a.n_heads = heads; a.n_kv_heads = kv_heads; a.head_dim = 128;
    a.num_blocks = num_blocks; a.block_size = block_size; a.max_blocks = max_blocks; a.scale = scale;
    a.dtype = rb::DType::BF16;
    a.kv_int8 = ks != nullptr; a.k_scales = ks; a.v_scales = vs;
    a.stream = stream;
    *need = rb::paged_decode_workspace_bytes(a);
    if (*need > ws_bytes) return static_cast<int>(rb::Status::WorkspaceTooSmall);
    a.workspace = ws; a.workspace_bytes = ws_bytes;
    return static_cast<int>(rb::paged_flash_attention_decode(a));
}
'''


@pytest.fixture(scope="module")
def shim(tmp_path_factory):
    if shutil.which("g++") is None:
        pytest.skip("no g++")
    d = tmp_path_factory.mktemp("cpp")
    src = d / "shim.cpp"
    src.write_text(SHIM)
    lib = ROOT / "reflex-infer_b200" / "lib"
    so = d / "libshim.so"
    subprocess.check_call(["g++", "-std=c++17", "-shared", "-fPIC", f"-I{ROOT / 'include'}", str(src), f"-L{lib}",
                           "-lreflex_b200", f"-Wl,-rpath,{lib}", "-o", str(so)])
    h = C.CDLL(str(so))
    h.run_decode.restype = C.c_int
    h.run_decode.argtypes = [C.c_void_p] * 6 + [C.c_int, C.c_int, C.c_int, C.c_longlong, C.c_int, C.c_int, C.c_float,
                                                C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p,
                                                C.POINTER(C.c_size_t)]
    return h


@pytest.mark.parametrize("int8", [False, True])
def test_cpp_paged_decode_against_oracle(int8, shim, native):
    cos, sin = oracle.build_rope_tables(700, 128, base=1e6, dtype=torch.bfloat16)
    cpu = workloads.make_paged_batch("cpp", B=5, Hq=16, Hkv=2, D=128, block_size=16, ctx_range=(30, 600),
                                     num_blocks=256, seed=17, tables=(cos, sin))
    pos = cpu.positions.long()
    q_rot = oracle.apply_rope(cpu.q_new.unsqueeze(0), cos[pos], sin[pos])[0]
    k_rot = oracle.apply_rope(cpu.k_new.unsqueeze(0), cos[pos], sin[pos])[0]
    g = cpu.to(DEV)
    if int8:
        kq, ks = oracle.kv_quantize_rows(cpu.k_cache)
        vq, vs = oracle.kv_quantize_rows(cpu.v_cache)
        oracle.kv_paged_append_q8(k_rot, cpu.v_new, kq, vq, ks, vs, cpu.slot_mapping)
        ref = oracle.paged_attention_composed(q_rot.float(), oracle.kv_dequantize(kq, ks), oracle.kv_dequantize(vq, vs),
                                              cpu.block_table, cpu.context_lens)
        kc, vc, ksg, vsg = kq.to(DEV), vq.to(DEV), ks.to(DEV), vs.to(DEV)
    else:
        kc, vc = g.k_cache, g.v_cache
        rope_append(g.k_new, g.v_new, kc, vc, g.slot_mapping, g.positions, g.cos, g.sin)
        kcpu, vcpu = cpu.k_cache.clone(), cpu.v_cache.clone()
        oracle.kv_paged_append(k_rot, cpu.v_new, kcpu, vcpu, cpu.slot_mapping)
        ref = oracle.paged_attention_composed(q_rot, kcpu, vcpu, cpu.block_table, cpu.context_lens).float()
        ksg = vsg = None
    q = q_rot.to(DEV)
    out = torch.full_like(q, float("nan"))
    ws = torch.empty(8 << 20, dtype=torch.uint8, device=DEV)
    need = C.c_size_t(0)
    stream = torch.cuda.current_stream().cuda_stream
    st = shim.run_decode(out.data_ptr(), q.data_ptr(), kc.data_ptr(), vc.data_ptr(), g.block_table.data_ptr(),
                         g.context_lens.data_ptr(), cpu.B, 16, 2, cpu.num_blocks, 16, g.block_table.shape[1],
                         128 ** -0.5, ksg.data_ptr() if int8 else None, vsg.data_ptr() if int8 else None,
                         ws.data_ptr(), ws.numel(), stream, C.byref(need))
    torch.cuda.synchronize()
    assert st == 0, native.lib().rfx_last_error()
    assert 0 < need.value <= ws.numel()
    torch.testing.assert_close(out.cpu().float(), ref, atol=2e-2, rtol=2e-2)
