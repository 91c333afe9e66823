"""Host-side mirror of the reference interface, checked without a GPU: names, signatures,
argument validation and exception types (the parts of the contract that run before any
kernel), and the workload generators."""
from __future__ import annotations

import inspect

import pytest
import torch

import workloads
from kernels.attention import fused_attention, paged_attention, rope_append
from kernels.kv_cache import kv_paged_append, kv_paged_lookup, kv_paged_scatter
from kernels.rope import apply_rope, apply_rope_, build_rope_tables
from kernels.softmax import online_softmax


def test_public_names_match_reference():
    import kernels.attention, kernels.kv_cache, kernels.rope, kernels.softmax
    assert set(kernels.kv_cache.__all__) == {"kv_paged_append", "kv_paged_lookup", "kv_paged_scatter"}
    assert set(kernels.rope.__all__) == {"apply_rope", "apply_rope_", "build_rope_tables"}
    assert kernels.softmax.__all__ == ["online_softmax"]
    assert "fused_attention" in kernels.attention.__all__


@pytest.mark.parametrize("fn,params", [
    (kv_paged_append, ["k_in", "v_in", "k_cache", "v_cache", "slot_mapping", "backend"]),
    (kv_paged_scatter, ["k_updates", "v_updates", "k_cache", "v_cache", "slot_mapping", "backend"]),
    (kv_paged_lookup, ["k_cache", "v_cache", "block_table", "context_lens", "max_ctx", "backend"]),
    (apply_rope, ["x", "cos", "sin", "interleaved", "layout", "backend"]),
    (apply_rope_, ["x", "cos", "sin", "interleaved", "layout", "backend"]),
    (build_rope_tables, ["seq_len", "head_dim", "base", "device", "dtype", "interleaved"]),
    (online_softmax, ["x", "is_causal", "log", "backend"]),
    (fused_attention, ["q", "k", "v", "is_causal", "attn_mask", "sm_scale", "backend"]),
])
def test_signatures(fn, params):
    sig = inspect.signature(fn)
    assert list(sig.parameters) == params
    assert sig.parameters[params[-1]].kind is inspect.Parameter.KEYWORD_ONLY


def test_no_cpu_path():
    x = torch.zeros(2, 4)
    with pytest.raises(RuntimeError, match="CUDA"):
        online_softmax(x)
    with pytest.raises(RuntimeError, match="CUDA"):
        fused_attention(torch.zeros(1, 1, 2, 8), torch.zeros(1, 1, 2, 8), torch.zeros(1, 1, 2, 8))
    with pytest.raises(RuntimeError, match="CUDA"):
        build_rope_tables(4, 8, device="cpu")


def test_validation_errors_precede_device_checks():
    with pytest.raises(ValueError, match="backend="):
        online_softmax(torch.zeros(2, 2), backend="metal")
    with pytest.raises(ValueError, match="causal mode requires square"):
        online_softmax(torch.zeros(4, 8), is_causal=True)
    with pytest.raises(ValueError, match="head_dim must be even"):
        build_rope_tables(4, 7)
    with pytest.raises(ValueError, match="unknown layout"):
        apply_rope(torch.zeros(1, 1, 1, 4), torch.zeros(1, 4), torch.zeros(1, 4), layout="sbhd")


def test_workload_generators_are_consistent():
    b = workloads.cfg2(scale=0.05)
    assert b.q_new.shape == (b.B, 16, 128) and b.k_new.shape == (b.B, 2, 128)
    assert torch.equal(b.context_lens, b.old_lens + b.n_new)
    # every new token's slot lies in a page its request owns, at its position
    for n in range(b.n_tokens):
        req = n  # one token per request
        pos = int(b.positions[n])
        assert pos == int(b.old_lens[req])
        page = int(b.block_table[req, pos // b.block_size])
        assert int(b.slot_mapping[n]) == page * b.block_size + pos % b.block_size
    used = b.block_table[b.block_table >= 0]
    assert used.numel() == used.unique().numel(), "a page was handed to two requests"
    # same seed, same batch
    b2 = workloads.cfg2(scale=0.05)
    assert torch.equal(b.block_table, b2.block_table) and torch.equal(b.q_new, b2.q_new)


def test_workload_fragmented_pool_uses_only_free_pages():
    b = workloads.cfg5(scale=0.02)
    free = b.extra["free_mask"]
    used = b.block_table[b.block_table >= 0]
    assert bool(free[used].all())
    assert int(b.q_start[-1]) == b.n_tokens and b.max_q_len == int(b.n_new.max())
    assert b.Hq // b.Hkv == 7
