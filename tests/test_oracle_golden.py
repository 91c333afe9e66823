"""Pins the CPU oracle to the reference: every golden fixture (outputs of the reference's
own torch path, tests/golden/make_golden.py) must be reproduced by oracle/ on the same
inputs -- bit for bit where the fixture stores a digest."""
from __future__ import annotations

import numpy as np
import pytest
import torch

import golden_cases as gc
import golden_io
import oracle
from oracle import c_oracle

TOL = {torch.float32: 1e-6, torch.bfloat16: 0.0, torch.float16: 0.0}


@pytest.mark.parametrize("name", sorted(gc.kv_write_cases()))
def test_kv_write(name):
    c = gc.kv_write_cases()[name]
    _, meta = golden_io.load(name)
    kc, vc = c["k_cache0"].clone(), c["v_cache0"].clone()
    (oracle.kv_paged_scatter if c["op"] == "scatter" else oracle.kv_paged_append)(c["k_in"], c["v_in"], kc, vc, c["slots"])
    assert golden_io.digest(kc) == meta["k_digest"]
    assert golden_io.digest(vc) == meta["v_digest"]
    # the plain-C statement of the same indexing
    view = torch.int16 if kc.element_size() == 2 else torch.int32
    kn, vn = c["k_cache0"].clone().view(view).numpy(), c["v_cache0"].clone().view(view).numpy()
    assert c_oracle.kv_append(c["k_in"].view(view).numpy(), c["v_in"].view(view).numpy(), kn, vn, c["slots"].numpy()) == 0
    assert np.array_equal(kn, kc.view(view).numpy()) and np.array_equal(vn, vc.view(view).numpy())


@pytest.mark.parametrize("name", sorted(gc.kv_lookup_cases()))
def test_kv_lookup(name):
    c = gc.kv_lookup_cases()[name]
    _, meta = golden_io.load(name)
    args = (c["k_cache"], c["v_cache"], c["block_table"], c["context_lens"], c["max_ctx"])
    ko, vo = oracle.kv_paged_lookup(*args)
    assert golden_io.digest(ko) == meta["k_digest"] and golden_io.digest(vo) == meta["v_digest"]
    kw, vw = oracle.kv_paged_lookup_as_written(*args)
    assert torch.equal(kw, ko) and torch.equal(vw, vo)
    view = torch.int16 if ko.element_size() == 2 else torch.int32
    kn, vn = c_oracle.kv_lookup(c["k_cache"].view(view).numpy(), c["v_cache"].view(view).numpy(),
                                c["block_table"].numpy(), c["context_lens"].numpy(), c["max_ctx"])
    assert np.array_equal(kn, ko.view(view).numpy()) and np.array_equal(vn, vo.view(view).numpy())


@pytest.mark.parametrize("name", sorted(gc.rope_cases()))
def test_rope(name):
    c = gc.rope_cases()[name]
    t, meta = golden_io.load(name)
    cos, sin = oracle.build_rope_tables(c["table_rows"], c["D"], base=c["base"], dtype=c["dtype"], interleaved=c["interleaved"])
    if c["pos"] is not None:
        cos, sin = cos[c["pos"]], sin[c["pos"]]
    assert torch.equal(cos, t["cos"]) and torch.equal(sin, t["sin"])
    y = oracle.apply_rope(c["x"], cos, sin, interleaved=c["interleaved"], layout=c["layout"])
    assert golden_io.digest(y) == meta["y_digest"]
    if c["dtype"] == torch.bfloat16 and c["layout"] == "bshd":
        # independent scalar statement of the per-op rounding
        B, S, H, D = c["x"].shape
        x2 = c["x"].reshape(B * S * H, D).view(torch.int16).numpy().view(np.uint16)
        pos = np.repeat(np.tile(np.arange(S), B), H).astype(np.int32)
        yc = c_oracle.rope_bf16(x2, cos.view(torch.int16).numpy().view(np.uint16),
                                sin.view(torch.int16).numpy().view(np.uint16), pos, c["interleaved"])
        assert np.array_equal(yc, y.reshape(B * S * H, D).view(torch.int16).numpy().view(np.uint16))


@pytest.mark.parametrize("name", sorted(gc.rope_table_cases()))
def test_rope_tables(name):
    c = gc.rope_table_cases()[name]
    t, meta = golden_io.load(name)
    cos, sin = oracle.build_rope_tables(c["seq_len"], c["D"], base=c["base"], dtype=c["dtype"], interleaved=c["interleaved"])
    assert golden_io.digest(cos) == meta["cos_digest"] and golden_io.digest(sin) == meta["sin_digest"]
    assert torch.equal(cos[c["rows"]], t["cos"])


def test_rope_position_zero_is_identity():
    # the reference's one analytic known answer, tests/test_rope.py:68-77
    x = golden_io.pattern((1, 1, 3, 32), torch.float32, 7)
    cos, sin = oracle.build_rope_tables(1, 32)
    assert torch.equal(oracle.apply_rope(x, cos, sin), x)


@pytest.mark.parametrize("name", sorted(gc.softmax_cases()))
def test_softmax(name):
    c = gc.softmax_cases()[name]
    t, _ = golden_io.load(name)
    assert torch.equal(oracle.online_softmax(c["x"], is_causal=c["causal"]), t["y"])
    assert torch.equal(oracle.online_softmax(c["x"], is_causal=c["causal"], log=True), t["ylog"])


def test_softmax_causal_needs_square():
    with pytest.raises(ValueError, match="causal mode requires square"):  # tests/test_softmax.py:87-97
        oracle.online_softmax(torch.zeros(4, 8), is_causal=True)


@pytest.mark.parametrize("name", sorted(gc.attention_cases()))
def test_attention(name):
    c = gc.attention_cases()[name]
    t, _ = golden_io.load(name)
    o = oracle.attention(c["q"], c["k"], c["v"], is_causal=c["causal"], attn_mask=c["mask"], sm_scale=c["sm_scale"])
    assert torch.equal(o, t["out"])
    if c["mask"] is None and not c["causal"]:
        ref64 = oracle.naive_attention_f64(c["q"], c["k"], c["v"], sm_scale=c["sm_scale"])
        tol = 1e-5 if c["q"].dtype == torch.float32 else 2e-2
        torch.testing.assert_close(o.double(), ref64, atol=tol, rtol=tol)


@pytest.mark.parametrize("name", sorted(gc.step_cases()))
def test_decode_step(name):
    c = gc.step_cases()[name]
    t, meta = golden_io.load(name)
    cos, sin = oracle.build_rope_tables(c["table_rows"], c["D"], base=c["theta"], dtype=c["dtype"])
    pos = c["positions"].long()
    q_rot = oracle.apply_rope(c["q"].unsqueeze(0), cos[pos], sin[pos])[0]
    k_rot = oracle.apply_rope(c["k"].unsqueeze(0), cos[pos], sin[pos])[0]
    assert torch.equal(q_rot, t["q_rot"]) and torch.equal(k_rot, t["k_rot"])
    kc, vc = c["k_cache0"].clone(), c["v_cache0"].clone()
    oracle.kv_paged_append(k_rot, c["v"], kc, vc, c["slots"])
    assert golden_io.digest(kc) == meta["k_digest"] and golden_io.digest(vc) == meta["v_digest"]
    out = oracle.paged_attention_composed(q_rot, kc, vc, c["block_table"], c["context_lens"])
    assert torch.equal(out, t["out"])
    if name == "step_cfg1_f32":
        # known answer of the first benchmark configuration: naive softmax(QK^T/sqrt(d))V
        kd, vd = oracle.kv_paged_lookup(kc, vc, c["block_table"], c["context_lens"], 257)
        ref = oracle.naive_attention_f64(q_rot.view(1, 16, 1, 64), kd, vd).view(1, 16, 64)
        torch.testing.assert_close(out.double(), ref, atol=1e-5, rtol=1e-5)
        row = c_oracle.attention_row_f64(q_rot[0, 3].numpy(), kd[0, 3].numpy(), vd[0, 3].numpy(), 1.0 / 8.0)
        np.testing.assert_allclose(row, ref[0, 3].numpy(), atol=1e-12)


def test_composed_chunk_matches_naive():
    # bottom-right causal chunk: row i of n sees keys 0..ctx-n+i
    g = golden_io.pattern
    Hq, Hkv, D, bs = 4, 2, 32, 8
    kc, vc = g((6, Hkv, bs, D), torch.float32, 1), g((6, Hkv, bs, D), torch.float32, 2)
    bt = torch.tensor([[4, 1, 3], [0, 2, 5]])
    ctx = torch.tensor([19, 9], dtype=torch.int32)
    q_start = [0, 5, 8]
    q = g((8, Hq, D), torch.float32, 3)
    out = oracle.paged_attention_composed(q, kc, vc, bt, ctx, q_start=q_start)
    for b in range(2):
        n_q, c = q_start[b + 1] - q_start[b], int(ctx[b])
        kd, vd = oracle.kv_paged_lookup(kc, vc, bt[b:b + 1], ctx[b:b + 1], c)
        mask = oracle.bottom_right_mask(n_q, c)
        ref = oracle.naive_attention_f64(q[q_start[b]:q_start[b + 1]].transpose(0, 1)[None], kd, vd, mask=mask)
        torch.testing.assert_close(out[q_start[b]:q_start[b + 1]].transpose(0, 1)[None].double(), ref, atol=1e-5, rtol=1e-5)


def test_merge_partials_equals_unsplit():
    g = golden_io.pattern
    s = g((50,), torch.float32, 11, scale=3.0)
    v = g((50, 16), torch.float32, 12)
    full = (torch.softmax(s.double(), 0)[:, None] * v.double()).sum(0)
    ms, ls, accs = [], [], []
    for lo, hi in ((0, 7), (7, 7), (7, 33), (33, 50)):
        if hi == lo:
            ms.append(torch.tensor(float("-inf"))); ls.append(torch.tensor(0.0)); accs.append(torch.zeros(16))
            continue
        m = s[lo:hi].max()
        p = torch.exp(s[lo:hi] - m)
        ms.append(m); ls.append(p.sum()); accs.append((p[:, None] * v[lo:hi]).sum(0))
    out = oracle.merge_partials(torch.stack(ms), torch.stack(ls), torch.stack(accs))
    torch.testing.assert_close(out, full, atol=1e-6, rtol=1e-6)


@pytest.mark.parametrize("name", sorted(gc.linear_norm_cases()))
def test_fused_linear_norm(name):
    c = gc.linear_norm_cases()[name]
    want, _ = golden_io.load(name)
    got = oracle.fused_linear_norm(c["x"], c["weight"], bias=c["bias"], gamma=c["gamma"], beta=c["beta"], eps=c["eps"],
                                   norm_type=c["norm"])
    tol = {torch.float32: 1e-5, torch.bfloat16: 2e-2, torch.float16: 5e-3}[c["x"].dtype]
    torch.testing.assert_close(got.float(), want["y"].float(), atol=tol, rtol=tol)
