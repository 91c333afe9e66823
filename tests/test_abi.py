"""The C-ABI boundary without a GPU: the library builds/loads, exports every symbol the
header declares, the ctypes mirrors have the C sizes, and argument errors come back as
status codes with messages (no compute is launched)."""
from __future__ import annotations

import ctypes as C
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "reflex_b200.h"


def declared_symbols():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(rfx_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_all_exported(native):
    lib = native.lib()
    names = declared_symbols()
    assert len(names) >= 17
    for name in names:
        assert hasattr(lib, name), f"{name} declared in the header but not exported"
    assert set(names) == set(native.EXPORTS), "binding table and header disagree"


def test_struct_sizes_match(native):
    lib = native.lib()
    for i, mirror in enumerate(native.ARG_STRUCTS):
        assert lib.rfx_args_size(i) == C.sizeof(mirror), mirror.__name__
    assert lib.rfx_args_size(99) == 0
    assert lib.rfx_abi_version() == 2


def test_status_strings(native):
    lib = native.lib()
    want = ["Success", "UnsupportedDevice", "UnsupportedModel", "UnsupportedQuantFormat", "InvalidArgument",
            "NotImplemented", "CudaError", "Timeout", "WorkspaceTooSmall"]  # include/reflex/infer.h:16-23 + 3
    assert [lib.rfx_status_string(i).decode() for i in range(9)] == want


def test_invalid_arguments_are_status_codes(native):
    lib = native.lib()
    assert lib.rfx_kv_paged_append(None) == native.RFX_INVALID_ARGUMENT
    a = native.RopeArgs(head_dim=63, batch=1, seq=1, heads=1, dtype=1)
    assert lib.rfx_rope_apply(C.byref(a)) == native.RFX_INVALID_ARGUMENT
    assert b"head_dim must be even" in lib.rfx_last_error()
    s = native.SoftmaxArgs(rows=6, n=4, is_causal=1, dtype=0)
    assert lib.rfx_online_softmax(C.byref(s)) == native.RFX_INVALID_ARGUMENT
    assert b"causal mode requires square" in lib.rfx_last_error()
    f = native.AttentionArgs(batch=1, num_q_heads=6, num_kv_heads=4, seq_q=1, seq_k=1, head_dim=8, dtype=0)
    assert lib.rfx_fused_attention(C.byref(f)) == native.RFX_INVALID_ARGUMENT
    assert b"GQA requires" in lib.rfx_last_error()
    p = native.PagedAttentionArgs(batch=2, n_q=3, num_q_heads=4, num_kv_heads=2, head_dim=64, num_blocks=4,
                                  block_size=16, max_blocks=2, dtype=1)
    assert lib.rfx_paged_attention(C.byref(p)) == native.RFX_INVALID_ARGUMENT
    # empty problems succeed without touching a device
    e = native.KvAppendArgs(n_tokens=0, num_kv_heads=2, head_dim=8, num_blocks=1, block_size=4, dtype=1)
    assert lib.rfx_kv_paged_append(C.byref(e)) == native.RFX_SUCCESS


def test_workspace_size_query(native):
    lib = native.lib()
    p = native.PagedAttentionArgs(batch=32, n_q=32, num_q_heads=16, num_kv_heads=2, head_dim=128, num_blocks=64,
                                  block_size=16, max_blocks=8, max_q_len=1, dtype=1)
    n1 = lib.rfx_paged_attention_workspace_bytes(C.byref(p))
    assert n1 > 0 and n1 % 256 == 0
    p.batch = p.n_q = 64
    assert lib.rfx_paged_attention_workspace_bytes(C.byref(p)) > n1


def test_workspace_capacity_rule(native):
    """The partial rows the workspace holds: G * (Hkv * n_q + runs * max_q_len), runs = 8 per SM
    (148 SMs assumed where no device answers). The plan kernel refuses, on the device, any q_start
    whose requests exceed max_q_len or whose total differs from n_q, so this host-side size is a
    bound the kernels never write past."""
    lib = native.lib()
    Hq, Hkv, D, n_q, B = 28, 4, 128, 900, 64
    def size(mq):
        p = native.PagedAttentionArgs(batch=B, n_q=n_q, num_q_heads=Hq, num_kv_heads=Hkv, head_dim=D, num_blocks=64,
                                      block_size=16, max_blocks=8, max_q_len=mq, dtype=1)
        p.q_start = 256  # any non-null pointer: the query only looks at sizes
        return lib.rfx_paged_attention_workspace_bytes(C.byref(p))
    G = Hq // Hkv
    s1, s64 = size(1), size(64)
    per_row = (D + 2) * 4 + 8 / 128  # m, l, acc of a partial row; one 8-byte entry of the unit list per 128 rows
    sms = round((s64 - s1) / (G * 8 * 63 * per_row))
    assert sms >= 100, sms
    assert abs((s64 - s1) - G * 8 * sms * 63 * per_row) <= 4 * 256
    rows1 = G * (Hkv * n_q + 8 * sms)
    assert s1 >= rows1 * (D + 2) * 4
    assert size(0) == s1  # a bound below one row per request is read as one


def test_cpp_header_compiles_and_links(native, tmp_path):
    """The header-only C++ face (reference-style `Status`, args structs, `const Args&` calls)
    compiles as C++17, links against the library and reports an argument error as a status."""
    import shutil
    import subprocess
    from pathlib import Path
    if shutil.which("g++") is None:
        pytest.skip("no g++")
    root = Path(__file__).resolve().parent.parent
    lib = root / "reflex-infer_b200" / "lib"
    src = tmp_path / "t.cpp"
    src.write_text(
        '#include "reflex_b200.hpp"\n'
        "int main() {\n"
        "    namespace rb = reflex::b200;\n"
        "    rb::PagedAttentionDecodeArgs a;\n"
        "    a.batch = 1; a.n_heads = 3; a.n_kv_heads = 2; a.head_dim = 64; a.num_blocks = 1; a.block_size = 16;\n"
        "    if (rb::paged_decode_workspace_bytes(a) != 0) return 2;   // 3 heads over 2 kv heads: rejected\n"
        "    if (rb::paged_flash_attention_decode(a) != rb::Status::InvalidArgument) return 3;\n"
        "    return rb::kernel_support().paged_decode_attention ? 0 : 1;\n"
        "}\n")
    exe = tmp_path / "t"
    subprocess.check_call(["g++", "-std=c++17", f"-I{root / 'include'}", str(src), f"-L{lib}", "-lreflex_b200",
                           f"-Wl,-rpath,{lib}", "-o", str(exe)])
    assert subprocess.call([str(exe)]) == 0
