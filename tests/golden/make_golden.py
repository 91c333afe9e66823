"""Generates the golden fixtures in this directory by running the REFERENCE's own torch
path (``backend="torch"``, CPU tensors) on small deterministic inputs.

Run where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/reference

It imports ``kernels`` from the reference tree only (this repository's package of the same
name is not on ``sys.path`` in this process). Inputs come from ``golden_io.pattern`` (pure
integer arithmetic, reproducible anywhere) and are not stored; each ``.npz`` holds the
reference's outputs -- in full where a tolerance applies, as a sha256 digest where the
result must match bit for bit (plus a few sampled rows for diagnosis). The tests never
need the reference afterwards. ``tests/golden_cases.py`` rebuilds the same inputs.
"""
from __future__ import annotations

import sys
from pathlib import Path

if len(sys.argv) < 2:
    raise SystemExit("usage: make_golden.py /path/to/reference")
REF = Path(sys.argv[1])
HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(REF))
sys.path.insert(1, str(HERE.parent))

import torch  # noqa: E402

from kernels.attention import fused_attention  # noqa: E402  (reference)
from kernels.kv_cache import kv_paged_append, kv_paged_lookup, kv_paged_scatter  # noqa: E402
from kernels.rope import apply_rope, build_rope_tables  # noqa: E402
from kernels.softmax import online_softmax  # noqa: E402
from kernels.fused_linear_norm import fused_linear_layernorm, fused_linear_rmsnorm  # noqa: E402

import golden_cases as gc  # noqa: E402
import golden_io  # noqa: E402

assert Path(sys.modules["kernels"].__file__).resolve().is_relative_to(REF.resolve()), "wrong `kernels` imported"
META = {"torch_version": torch.__version__}
BK = "torch"


def exact(t):
    """digest + first/last rows for diagnosis"""
    flat = t.reshape(-1, t.shape[-1])
    return golden_io.digest(t), torch.cat((flat[:2], flat[-2:]))


def main():
    n = 0
    for name, c in gc.kv_write_cases().items():
        kc, vc = c["k_cache0"].clone(), c["v_cache0"].clone()
        fn = kv_paged_scatter if c["op"] == "scatter" else kv_paged_append
        fn(c["k_in"], c["v_in"], kc, vc, c["slots"], backend=BK)
        (dk, sk), (dv, sv) = exact(kc), exact(vc)
        golden_io.save(name, dict(k_rows=sk, v_rows=sv), {**META, "k_digest": dk, "v_digest": dv}); n += 1
    for name, c in gc.kv_lookup_cases().items():
        ko, vo = kv_paged_lookup(c["k_cache"], c["v_cache"], c["block_table"], c["context_lens"], c["max_ctx"], backend=BK)
        (dk, sk), (dv, sv) = exact(ko), exact(vo)
        golden_io.save(name, dict(k_rows=sk, v_rows=sv), {**META, "k_digest": dk, "v_digest": dv}); n += 1
    for name, c in gc.rope_cases().items():
        cos, sin = build_rope_tables(c["table_rows"], c["D"], base=c["base"], dtype=c["dtype"], interleaved=c["interleaved"])
        if c["pos"] is not None:
            cos, sin = cos[c["pos"]], sin[c["pos"]]
        y = apply_rope(c["x"], cos, sin, interleaved=c["interleaved"], layout=c["layout"], backend=BK)
        golden_io.save(name, dict(y=y, cos=cos, sin=sin), {**META, "y_digest": golden_io.digest(y)}); n += 1
    for name, c in gc.rope_table_cases().items():
        cos, sin = build_rope_tables(c["seq_len"], c["D"], base=c["base"], dtype=c["dtype"], interleaved=c["interleaved"])
        rows = c["rows"]
        golden_io.save(name, dict(cos=cos[rows], sin=sin[rows]),
                       {**META, "cos_digest": golden_io.digest(cos), "sin_digest": golden_io.digest(sin)}); n += 1
    for name, c in gc.softmax_cases().items():
        golden_io.save(name, dict(y=online_softmax(c["x"], is_causal=c["causal"], backend=BK),
                                  ylog=online_softmax(c["x"], is_causal=c["causal"], log=True, backend=BK)), META); n += 1
    for name, c in gc.attention_cases().items():
        k, v = c["k"], c["v"]
        rep = c["q"].shape[1] // k.shape[1]
        if rep > 1:  # the reference's torch path has no GQA; its tests expand first (tests/test_attention_parity.py:72-76)
            k, v = k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)
        o = fused_attention(c["q"], k, v, is_causal=c["causal"], attn_mask=c["mask"], sm_scale=c["sm_scale"], backend=BK)
        golden_io.save(name, dict(out=o), META); n += 1
    for name, c in gc.step_cases().items():
        # The decode step as the reference spells it: tables -> apply_rope(q), apply_rope(k) -> kv_paged_append
        # -> per-request kv_paged_lookup(max_ctx = ctx_b) -> GQA expansion -> fused_attention.
        cos, sin = build_rope_tables(c["table_rows"], c["D"], base=c["theta"], dtype=c["dtype"])
        pos = c["positions"].long()
        q_rot = apply_rope(c["q"].unsqueeze(0), cos[pos], sin[pos], backend=BK)[0]
        k_rot = apply_rope(c["k"].unsqueeze(0), cos[pos], sin[pos], backend=BK)[0]
        kc, vc = c["k_cache0"].clone(), c["v_cache0"].clone()
        kv_paged_append(k_rot, c["v"], kc, vc, c["slots"], backend=BK)
        B, Hq, D = c["q"].shape
        rep = Hq // c["k"].shape[1]
        out = torch.zeros(B, Hq, D, dtype=c["dtype"])
        for b in range(B):
            ctx = int(c["context_lens"][b])
            kd, vd = kv_paged_lookup(kc, vc, c["block_table"][b:b + 1], c["context_lens"][b:b + 1], ctx, backend=BK)
            ob = fused_attention(q_rot[b].view(1, Hq, 1, D), kd.repeat_interleave(rep, 1), vd.repeat_interleave(rep, 1),
                                 is_causal=False, backend=BK)
            out[b] = ob.view(Hq, D)
        golden_io.save(name, dict(out=out, q_rot=q_rot, k_rot=k_rot),
                       {**META, "k_digest": golden_io.digest(kc), "v_digest": golden_io.digest(vc)}); n += 1
    for name, c in gc.linear_norm_cases().items():
        if c["norm"] == "rms":
            y = fused_linear_rmsnorm(c["x"], c["weight"], bias=c["bias"], gamma=c["gamma"], eps=c["eps"], backend=BK)
        else:
            y = fused_linear_layernorm(c["x"], c["weight"], bias=c["bias"], gamma=c["gamma"], beta=c["beta"],
                                       eps=c["eps"], backend=BK)
        golden_io.save(name, dict(y=y), META); n += 1
    total = sum(p.stat().st_size for p in HERE.glob("*.npz"))
    print(f"wrote {n} fixtures, {total / 1e6:.2f} MB, torch {torch.__version__}")


if __name__ == "__main__":
    main()
