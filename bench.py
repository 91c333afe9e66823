#!/usr/bin/env python
"""Benchmark of the paged-KV decode step on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cfg4|cfg2]
                    [--impl ours|reference] [--shard request|replica|head]

One "step" is one decode step of one layer over one synthetic batch of the named
configuration: fused RoPE + append of the new token's K/V, split-K plan, paged GQA
attention partials (the HBM-bound kernel), combine. Rank 0 prints ONE JSON line.

  value      decode tokens/s of the whole job, inputs already in HBM, timed with CUDA
             events per step, max over ranks;
  e2e        the same step driven from pinned HOST buffers: H2D of q/k/v/slots/positions,
             the kernels, D2H of the output, all inside the timed region;
  roofline   algorithmic K+V bytes of the batch / mean duration of the partial kernel
             (events around that launch inside the timed steps) vs the measured HBM peak;
  cpu_baseline  the CPU oracle (a port of the reference's torch path) timed on this box's
             host cores on a bounded sample of the same workload (rank 0, N=1 only).

``--impl reference`` times the reference's own torch path on CPU (its ``kernels`` package from
``baseline/_ref`` when that copy exists, else the oracle port of it), on the same configuration,
and prints the same line with ``"impl": "reference"``.

Multi-GPU: one process per GPU (torchrun). ``--shard request`` (default, strong scaling): the ONE
batch of the configuration is split by request across the ranks with a greedy balance on context
length, no collective. ``--shard head`` (strong): ranks own kv-head slices of the pool and the
output heads are assembled inside the combine kernel (peer stores) or by one NCCL all-gather.
``--shard replica`` (weak): every rank decodes its own batch of the configuration. Without
``--shard`` a multi-GPU run measures the request split for the headline and then the other three
modes, reported under ``other_shards``.

The secondary blocks (the other decode configuration, prefill, the mixed batch, fused linear + norm,
the small ops) are printed as their own JSON lines BEFORE the result line, which is the last line
of stdout and repeats their headline figures under ``secondary``.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
PKG = ROOT / "reflex-infer_b200"
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def use_package():
    """Puts this repository's package (kernels, workloads, sharding) on the import path. Not done in
    the reference arm, where ``kernels`` must be the reference's own package."""
    if str(PKG) not in sys.path:
        sys.path.insert(0, str(PKG))


def load_workloads():
    """The synthetic workload generators, loaded by file so that the reference arm need not put this
    repository's ``kernels`` package on the path."""
    if "workloads" in sys.modules:
        return sys.modules["workloads"]
    import importlib.util
    spec = importlib.util.spec_from_file_location("workloads", PKG / "workloads.py")
    mod = importlib.util.module_from_spec(spec)
    sys.modules["workloads"] = mod
    spec.loader.exec_module(mod)
    return mod

import torch  # noqa: E402

METRIC = "paged_decode_attn_tokens_per_s"
UNIT = "tokens/s"
FALLBACK_HBM_GBS = 6650.0


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg4", choices=["cfg4", "cfg2"])
    ap.add_argument("--gather", default="fused", choices=["fused", "nccl"],
                    help="--shard head: assemble the heads inside the combine kernel (peer stores) or with an "
                         "NCCL all-gather")
    ap.add_argument("--shard", default=None, choices=["replica", "request", "head"],
                    help="default: request (strong scaling); a multi-GPU run without this flag also measures "
                         "the other modes and reports them under other_shards")
    ap.add_argument("--pool-pages", type=int, default=0,
                    help="with --only cfg5: pages in the pool instead of 1,048,576 (a small case for ncu; >= 65536)")
    ap.add_argument("--small-filter", default=None,
                    help="with --only small_ops: time only the ops whose label contains this text (small cases for ncu)")
    ap.add_argument("--only", default=None, choices=["cfg3", "cfg5", "linear_norm", "small_ops", "int8_kv", "clocks"],
                    help="run just that secondary block on one GPU and print it (small profiling cases: "
                         "--only cfg3 --requests 2)")
    ap.add_argument("--cpu-sample", type=int, default=0, help="requests in the CPU-baseline sample (0 = auto)")
    ap.add_argument("--cpu-budget", type=float, default=120.0,
                    help="--impl reference: seconds of CPU work the warm-up and timed steps may take in total")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extra", action="store_true", help="skip the secondary configuration block")
    ap.add_argument("--chunk", type=int, default=0, help="keys per split (0 = planner's choice)")
    ap.add_argument("--graph", action="store_true",
                    help="replay the step from a CUDA graph in the step-timing pass (launch overhead off the clock)")
    ap.add_argument("--requests", type=int, default=0,
                    help="profiling aid: shrink the batch to this many requests (0 = the configuration's own)")
    return ap.parse_args()


REFERENCE_SAMPLE_NOTE = ("the reference arm (--impl reference) times a bounded sample of the requests per step "
                         "on the host cores and is normalised per token")


def line_config(workload: str, shard: str, extra: dict = None) -> dict:
    """The `config` object of the result line; the same for both arms of a run."""
    kv_small = workload == "cfg2"
    return {**workload_desc(workload), "shard": shard,
            "l2": ("512 MiB memset between timed steps flushes L2 (outside the timed events)" if kv_small else
                   "K+V read per step exceeds L2 (126 MB) many times over; no flush"),
            "timing": "CUDA events per step on the launch stream, max over ranks",
            "reference_arm_sample": REFERENCE_SAMPLE_NOTE, **(extra or {})}


def workload_desc(name: str) -> dict:
    if name == "cfg4":
        return {"workload": "cfg4: bf16 paged GQA decode, 256 requests, ctx U[8192,32768], 64q/8kv heads, D=128, "
                            "page 32, permuted pages, theta 1e6, 1 new token per request",
                "batch": 256, "q_heads": 64, "kv_heads": 8, "head_dim": 128, "page_size": 32}
    return {"workload": "cfg2: bf16 paged GQA decode, 32 requests, ctx U[512,8192], 16q/2kv heads, D=128, "
                        "page 16, permuted 32768-page pool, theta 1e6, 1 new token per request",
            "batch": 32, "q_heads": 16, "kv_heads": 2, "head_dim": 128, "page_size": 16}


def measured_peak():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


# ---- clocks -----------------------------------------------------------------------------

class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons every 50 ms while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.proc = None
        self.lines = []   # (arrival time, text)
        self.gpu = gpu_index
        self.window = [None, None]  # wall-clock bounds of the timed regions

    def mark_begin(self):
        if self.window[0] is None:
            self.window[0] = time.time()

    def mark_end(self):
        self.window[1] = time.time()

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50",
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, mx, pw, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        lo, hi = self.window
        inside = [ln for t, ln in self.lines if lo is not None and hi is not None and lo <= t <= hi + 0.06]
        for ln in (inside if inside else [ln for _, ln in self.lines]):
            parts = [x.strip() for x in ln.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1])); pw.append(float(parts[2]))
            except ValueError:
                continue
            for nm, v in zip(names, parts[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_median": statistics.median(pw) if pw else None, "power_w_max": max(pw) if pw else None,
                "samples": len(sm), "samples_inside_timed_regions": len(inside), "reasons": sorted(reasons)}


# ---- CPU legs (the reference arm; the only place besides tests that may import the oracle) --------

class ReferenceOps:
    """The four ops of the path as the reference arm calls them: the reference's own ``kernels``
    package (torch backend, CPU tensors) when a copy sits under baseline/_ref, else the oracle's
    restatement of that path. `kind` says which ("reference" / "port")."""

    def __init__(self):
        root = ROOT / "baseline" / "_ref"
        self.kind = "port"
        if (root / "kernels" / "attention" / "__init__.py").exists() and "kernels" not in sys.modules:
            sys.path.insert(0, str(root))
            try:
                from kernels.attention import fused_attention
                from kernels.kv_cache import kv_paged_append, kv_paged_lookup
                from kernels.rope import apply_rope
                assert Path(sys.modules["kernels"].__file__).resolve().is_relative_to(root.resolve())
                bk = dict(backend="torch")
                self.apply_rope = lambda x, c, s_: apply_rope(x, c, s_, **bk)
                self.append = lambda k, v, kc, vc, sl: kv_paged_append(k, v, kc, vc, sl, **bk)
                self.lookup = lambda kc, vc, bt, cl, mx: kv_paged_lookup(kc, vc, bt, cl, mx, **bk)
                self.attention = lambda q, k, v: fused_attention(q, k, v, **bk)
                self.kind = "reference"
            except Exception as e:  # an unusable copy: say so and fall back to the port
                print(f"bench.py: baseline/_ref is not importable ({e}); using the oracle port", file=sys.stderr)
                sys.path.remove(str(root))
        import oracle
        self.oracle = oracle
        if self.kind == "port":
            self.apply_rope = oracle.apply_rope
            self.append = oracle.kv_paged_append
            self.lookup = oracle.kv_paged_lookup_as_written
            self.attention = lambda q, k, v: oracle.attention(q, k, v)

    def decode_step(self, batch, vectorised: bool = False) -> float:
        """One decode step of `batch` (CPU tensors) the way the reference composes it: tables rows ->
        apply_rope -> kv_paged_append -> per request kv_paged_lookup, GQA expansion, fused_attention.
        `vectorised` swaps the per-token Python loop of the reference's lookup for one gather (same
        result), so that the baseline is not a Python loop alone. Seconds."""
        t0 = time.perf_counter()
        pos = batch.positions.long()
        q_rot = self.apply_rope(batch.q_new.unsqueeze(0), batch.cos[pos], batch.sin[pos])[0]
        k_rot = self.apply_rope(batch.k_new.unsqueeze(0), batch.cos[pos], batch.sin[pos])[0]
        self.append(k_rot, batch.v_new, batch.k_cache, batch.v_cache, batch.slot_mapping)
        lookup = self.oracle.kv_paged_lookup if vectorised else self.lookup
        g = batch.Hq // batch.Hkv
        out = torch.zeros_like(q_rot)
        for r in range(batch.B):
            ctx = int(batch.context_lens[r])
            kd, vd = lookup(batch.k_cache, batch.v_cache, batch.block_table[r:r + 1], batch.context_lens[r:r + 1], ctx)
            qb = q_rot[r:r + 1].transpose(0, 1).unsqueeze(0)  # [1, H, 1, D]
            ob = self.attention(qb, kd.repeat_interleave(g, dim=1), vd.repeat_interleave(g, dim=1))
            out[r] = ob[0, :, 0]
        self.last_out = out
        return time.perf_counter() - t0


def make_cpu_batch(workload: str, n_req: int, seed: int):
    import oracle
    workloads = load_workloads()
    if workload == "cfg4":
        cos, sin = oracle.build_rope_tables(32770, 128, base=1e6, dtype=torch.bfloat16)
        return workloads.cfg4(device="cpu", seed=seed, B=n_req, tables=(cos, sin))
    cos, sin = oracle.build_rope_tables(8194, 128, base=1e6, dtype=torch.bfloat16)
    b = workloads.make_paged_batch("cfg2", B=n_req, Hq=16, Hkv=2, D=128, block_size=16, ctx_range=(512, 8192),
                                   theta=1e6, device="cpu", seed=seed, tables=(cos, sin))
    return b


def cpu_baseline(workload: str, sample: int, budget_s: float = 20.0) -> dict:
    """The reference arm run as its own process (its `kernels` package cannot share a process with
    this repository's package of the same name) on a bounded sample; its `cpu_baseline` object."""
    cmd = [sys.executable, str(Path(__file__).resolve()), "--impl", "reference", "--workload", workload, "--steps", "2",
           "--warmup", "1", "--cpu-budget", str(budget_s)] + (["--cpu-sample", str(sample)] if sample else [])
    try:
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
        line = json.loads(r.stdout.strip().splitlines()[-1])
        return line["cpu_baseline"]
    except Exception as e:
        return {"value": None, "unit": UNIT, "cores": os.cpu_count(), "kind": "port", "sample": f"failed: {e}"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    torch.set_num_threads(os.cpu_count() or 1)
    cores = torch.get_num_threads()
    ops = ReferenceOps()
    n = args.cpu_sample or 2
    batch = make_cpu_batch(args.workload, n, seed=100)
    t = ops.decode_step(batch)
    if not args.cpu_sample:
        # size the per-step sample so that warm-up + steps end within the budget (about two minutes
        # for the driver's run, 20 s for the in-line baseline of the GPU arm)
        per_req = t / n
        n = max(1, min(64, workload_desc(args.workload)["batch"],
                       int(args.cpu_budget / max(args.steps + args.warmup, 1) / max(per_req, 1e-3))))
        batch = make_cpu_batch(args.workload, n, seed=101)
    for _ in range(args.warmup):
        ops.decode_step(batch)
    times = [ops.decode_step(batch) for _ in range(args.steps)]
    total = sum(times)
    value = n * args.steps / total
    t_vec = min(ops.decode_step(batch, vectorised=True) for _ in range(2))
    what = ("the reference's own kernels package (baseline/_ref), backend='torch', CPU tensors" if ops.kind == "reference"
            else "CPU oracle port of the reference's torch path")
    sample = (f"{n} of {workload_desc(args.workload)['batch']} requests of {args.workload} per step (same generator and "
              f"distributions), {what}: apply_rope -> kv_paged_append -> per request kv_paged_lookup, GQA expansion, "
              f"fused_attention")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / args.steps,
        "higher_is_better": True, "scaling": "weak" if args.shard == "replica" else "strong", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": line_config(args.workload, args.shard or "request"),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": ops.kind, "sample": sample,
                         "vectorised_gather_value": n / t_vec,
                         "vectorised_gather_note": "same composition with the lookup's per-token Python loop replaced "
                                                   "by one gather (identical result), best of 2",
                         "torch": torch.__version__},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---- GPU legs -----------------------------------------------------------------------------

class DecodeStep:
    """Prepared launches of one decode step over fixed device buffers."""

    def __init__(self, batch, chunk: int = 0):
        from kernels.attention import PagedAttentionCall, PagedWorkspace, RopeAppendCall
        self.b = batch
        dev = batch.q_new.device
        self.ws = PagedWorkspace(dev)
        self.append = RopeAppendCall(batch.k_new, batch.v_new, batch.k_cache, batch.v_cache, batch.slot_mapping,
                                     batch.positions, batch.cos, batch.sin)
        self.attn = PagedAttentionCall(batch.q_new, batch.k_cache, batch.v_cache, batch.block_table,
                                       batch.context_lens, rope_cos=batch.cos, rope_sin=batch.sin,
                                       rope_positions=batch.positions, workspace=self.ws, target_chunk=chunk)
        self.out = self.attn.out
        self.gather = None  # a sharding.FusedHeadGather: the combine then writes every rank's full output
        self.fused = self.attn.kernel_kind == 1  # the decode kernel finishes its rows: no combine launch

    @property
    def kernel_launches(self):
        return 3 if self.fused and self.gather is None else 4

    def run(self, ev0=None, ev1=None):
        self.append.run()
        self.attn.plan()
        if ev0 is not None:
            ev0.record()
        if self.fused and self.gather is None:
            self.attn.partials_final()
            if ev1 is not None:
                ev1.record()
            return self.out
        self.attn.partials()
        if ev1 is not None:
            ev1.record()
        if self.gather is not None:
            return self.attn.combine_gather(self.gather)
        self.attn.combine()
        return self.out


def pack_step_inputs(batch):
    """Re-homes the per-step inputs (q, k, v, slots, positions) as views of ONE device buffer,
    so a host-driven step uploads them with a single copy. Returns (packed device buffer, batch)."""
    import dataclasses
    names = ["q_new", "k_new", "v_new", "slot_mapping", "positions"]
    offs, total = {}, 0
    for n in names:
        t = getattr(batch, n)
        offs[n] = total
        total += (t.numel() * t.element_size() + 255) // 256 * 256
    buf = torch.empty(total, dtype=torch.uint8, device=batch.q_new.device)
    views = {}
    for n in names:
        t = getattr(batch, n)
        nb = t.numel() * t.element_size()
        v = buf[offs[n]:offs[n] + nb].view(t.dtype).view(t.shape)
        v.copy_(t)
        views[n] = v
    return buf, dataclasses.replace(batch, **views)


class HostDrivenStep:
    """The same step fed from one pinned host buffer (all of the step's inputs), result read
    back to pinned host memory. With head sharding the step includes the gather (`post`: the
    NCCL variant; the fused variant is inside the step) and rank 0 alone reads back the
    assembled output, as a serving rank would."""

    def __init__(self, step: DecodeStep, packed: torch.Tensor, post=None, read_back: bool = True):
        self.step = step
        self.post = post
        self.dev = packed
        self.host = packed.cpu().pin_memory()
        shape = step.gather.shape if step.gather is not None else (post.full.shape if post is not None else step.out.shape)
        self.out_host = torch.empty(shape, dtype=step.out.dtype).pin_memory() if read_back else None
        self.h2d = self.host.numel()
        self.d2h = self.out_host.numel() * self.out_host.element_size() if read_back else 0

    def run(self):
        self.dev.copy_(self.host, non_blocking=True)
        out = self.step.run()
        if self.post is not None:
            out = self.post.run(out)
        if self.out_host is not None:
            self.out_host.copy_(out, non_blocking=True)


def timed_steps(fn, steps, warmup, flush=None, dist=None, with_kernel_events=False):
    """W warm-up steps, then K steps each bracketed by its own CUDA event pair (an untimed L2
    flush in between when `flush` is given); barrier + synchronize on both sides. Returns
    (total_ms, [per-kernel ms] or None)."""
    for _ in range(warmup):
        if flush is not None:
            flush()
        fn(None, None) if with_kernel_events else fn()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    se = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    ee = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    k0 = [torch.cuda.Event(enable_timing=True) for _ in range(steps)] if with_kernel_events else None
    k1 = [torch.cuda.Event(enable_timing=True) for _ in range(steps)] if with_kernel_events else None
    for i in range(steps):
        if flush is not None:
            flush()
        se[i].record()
        if with_kernel_events:
            fn(k0[i], k1[i])
        else:
            fn()
        ee[i].record()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    total = sum(s.elapsed_time(e) for s, e in zip(se, ee))
    kern = [a.elapsed_time(b) for a, b in zip(k0, k1)] if with_kernel_events else None
    return total, kern


def build_batch(workload, device, seed, shard, rank, world, requests=0):
    workloads = load_workloads()
    if workload == "cfg4":
        b = workloads.cfg4(device=device, seed=seed, B=requests or None)
    elif requests:
        b = workloads.make_paged_batch("cfg2", B=requests, Hq=16, Hkv=2, D=128, block_size=16, ctx_range=(512, 8192),
                                       num_blocks=32768, theta=1e6, device=device, seed=seed)
    else:
        b = workloads.cfg2(device=device, seed=seed)
    if world > 1 and shard == "request":
        from sharding import shard_batch_by_request
        b = shard_batch_by_request(b, rank, world)
    elif world > 1 and shard == "head":
        from sharding import shard_batch_by_kv_head
        b = shard_batch_by_kv_head(b, rank, world)
    return b


def measure(workload, args, device, rank, world, dist, want_e2e=True, sampler=None, shard="request", gather_kind="fused"):
    seed_base = {"cfg4": 3, "cfg2": 1}[workload]
    # replica: every rank draws its own batch; request/head: all ranks draw the same one, then cut it
    seed = seed_base + (1000 * rank if shard == "replica" else 0)
    batch = build_batch(workload, device, seed, shard, rank, world, args.requests if workload == args.workload else 0)
    packed, batch = pack_step_inputs(batch)
    step = DecodeStep(batch, chunk=args.chunk)
    kv_bytes = batch.kv_bytes()
    tokens = batch.n_tokens
    flush = None
    flush_note = "K+V read per step exceeds L2 (126 MB) many times over; no flush"
    if kv_bytes < 4 * 126e6:
        scratch = torch.empty(512 << 20, dtype=torch.uint8, device=device)
        flush = lambda: scratch.zero_()  # noqa: E731
        flush_note = "512 MiB memset between timed steps flushes L2 (outside the timed events)"

    gather = None
    gather_check = None
    if world > 1 and shard == "head":
        from sharding import FusedHeadGather, HeadGather
        gather = HeadGather(step.out, dist)
        if gather_kind == "fused":
            # same step twice: NCCL all-gather of the local heads (combine kernel, the arithmetic of the
            # gathering combine), then the gathering combine
            step.append.run(); step.attn.plan(); step.attn.partials()
            want = gather.run(step.attn.combine()).clone()
            step.gather = FusedHeadGather(step.out.shape[0], batch.Hq, batch.D, batch.dtype, device, dist)
            got = step.run()
            torch.cuda.synchronize()
            gather_check = "equal to the NCCL all-gather" if torch.equal(got, want) else "DIFFERS from the NCCL all-gather"
            gather = None

    def run(ev0=None, ev1=None):
        out = step.run(ev0, ev1)
        if gather is not None:
            gather.run(out)

    if sampler:
        sampler.mark_begin()
    # Two timed passes of K steps each: the first times whole steps with nothing between the
    # launches (an event record between two kernels would keep the second from being launched
    # programmatically behind the first); the second brackets the partial kernel with its own
    # event pair for the roofline.
    step_fn = lambda: run()  # noqa: E731
    if args.graph and gather is None:
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            run()
            torch.cuda.synchronize()
            cg = torch.cuda.CUDAGraph()
            with torch.cuda.graph(cg, stream=side):
                run()
        torch.cuda.synchronize()
        step_fn = cg.replay
    total_ms, _ = timed_steps(step_fn, args.steps, args.warmup, flush, dist)
    _, kern_ms = timed_steps(run, args.steps, 1, flush, dist, with_kernel_events=True)
    # the same step for the further layers of a model: the plan depends only on the lengths, so layers
    # 2..N of a decode step reuse it (reuse_plan): RoPE + append and the decode kernel, two launches
    reused_ms = None
    if gather is None and step.fused:
        def later_layer():
            step.append.run()
            step.attn.partials_final()
        reused_ms, _ = timed_steps(later_layer, args.steps, args.warmup, flush, dist)
    status = step.ws.status()
    res = {"tokens": tokens, "plan_reused_ms": reused_ms, "kv_bytes": kv_bytes, "total_ms": total_ms, "kernel_ms": statistics.mean(kern_ms),
           "kernel_ms_min": min(kern_ms), "status": status, "flush": flush_note, "kernel_kind": step.attn.kernel_kind,
           "launches": step.kernel_launches * args.steps, "gather_check": gather_check}
    if want_e2e:
        head_mode = world > 1 and shard == "head"
        host = HostDrivenStep(step, packed, post=gather, read_back=(rank == 0 or not head_mode))
        e2e_ms, _ = timed_steps(host.run, args.steps, args.warmup, flush, dist)
        res.update(e2e_ms=e2e_ms, h2d=host.h2d, d2h=host.d2h)
    if sampler:
        sampler.mark_end()
    res["batch"] = batch
    res["step"] = step
    return res


def whole_job(res, dist, device, shard, world):
    """Whole-job figures of one measurement: the tokens of all ranks over the slowest rank's time.
    Returns (total_ms, e2e_ms, kernel_ms, tokens, kv_bytes), the times as max over ranks."""
    t = torch.tensor([res["total_ms"], res.get("e2e_ms", 0.0), res["kernel_ms"]], dtype=torch.float64, device=device)
    toks = torch.tensor([float(res["tokens"]), float(res["kv_bytes"])], dtype=torch.float64, device=device)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(toks, op=dist.ReduceOp.SUM)
    total_ms, e2e_ms, kernel_ms = t.tolist()
    all_tokens, all_bytes = toks.tolist()
    if shard == "head" and world > 1:
        all_tokens = float(res["tokens"])  # every rank works on all requests; count them once
    return total_ms, e2e_ms, kernel_ms, all_tokens, all_bytes


def release(res):
    """Frees what a measurement holds on the device (peer mappings first)."""
    g = getattr(res.get("step"), "gather", None)
    if g is not None:
        g.close()
    res.clear()
    torch.cuda.empty_cache()


def measure_prefill(args, device):
    """Configuration 3 (causal paged prefill, 8 x 2048 new tokens, 32q/8kv heads, D=128, page 16):
    one step = fused RoPE + append of every new token (Q rotated too) + causal attention from
    the pool on the tcgen05 kernel. Tensor-pipe roofline on the attention kernel."""
    workloads = load_workloads()
    from kernels.attention import PagedAttentionCall, RopeAppendCall
    b = workloads.cfg3(device=device, scale=(args.requests / 8.0 if args.requests else 1.0), seq=2048)
    q_rot = torch.empty_like(b.q_new)
    ra = RopeAppendCall(b.k_new, b.v_new, b.k_cache, b.v_cache, b.slot_mapping, b.positions, b.cos, b.sin,
                        q=b.q_new, q_out=q_rot)
    attn = PagedAttentionCall(q_rot, b.k_cache, b.v_cache, b.block_table, b.context_lens, q_start=b.q_start,
                              max_q_len=b.max_q_len)

    def run(ev0=None, ev1=None):
        ra.run()
        if ev0 is not None:
            ev0.record()
        attn.run()
        if ev1 is not None:
            ev1.record()

    total_ms, kern_ms = timed_steps(run, args.steps, args.warmup, None, None, with_kernel_events=True)
    S = int(b.n_new[0])
    flops = 4.0 * b.B * b.Hq * b.D * S * (S + 1) / 2  # causal count; the reference's own count has no discount
    km = statistics.mean(kern_ms)
    peaks = {}
    try:
        peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text())
    except Exception:
        pass
    burst = float(peaks.get("bf16_tflops", 1590.0))
    return {"config": f"cfg3: bf16 causal paged prefill, {b.B} x 2048 new tokens on an empty cache, 32q/8kv heads, "
                      "D=128, page 16, theta 1e6",
            "value": b.n_tokens * args.steps / (total_ms * 1e-3), "unit": UNIT, "ms_per_step": total_ms / args.steps,
            "kernel": "prefill_tc_kernel" if attn.kernel_kind in (2, 3) else "scalar",
            "kernel_ms": km, "roofline": {"bound": "tensor", "achieved": flops / (km * 1e-3) / 1e12, "peak": burst,
                                          "unit": "TFLOP/s", "frac": flops / (km * 1e-3) / 1e12 / burst,
                                          "peak_sustained": peaks.get("bf16_tflops_sustained"),
                                          "flops_causal": flops, "flops_reference_count": 2 * flops * S / (S + 1)},
            "append_gigabytes_moved": 2.0 * b.n_tokens * (b.Hq + 2 * b.Hkv) * b.D * 2 / 1e9,
            "status": attn.workspace.status()}


def measure_mixed(args, device):
    """Configuration 5 (mixed batch: 64 requests with 1..64 new tokens each on contexts of 0..16384
    keys, 28q/4kv heads, page 16, 1 Mi-page pool with 40 % of the pages free, 10 % of the requests
    compacted onto fresh pages with kv_paged_scatter before the step). One step = fused RoPE +
    append of the new tokens + bottom-right-causal attention from the pool."""
    workloads = load_workloads()
    from kernels.attention import PagedAttentionCall, RopeAppendCall
    from kernels.kv_cache import kv_paged_scatter
    b = workloads.cfg5(device=device, pool_pages=(args.pool_pages or None))
    q_rot = torch.empty_like(b.q_new)
    ra = RopeAppendCall(b.k_new, b.v_new, b.k_cache, b.v_cache, b.slot_mapping, b.positions, b.cos, b.sin,
                        q=b.q_new, q_out=q_rot)
    # compaction: the chosen requests' rows are gathered and scattered to pages nobody uses
    bt = b.block_table.cpu()
    used = torch.zeros(b.num_blocks, dtype=torch.bool)
    used[bt[bt >= 0]] = True
    fresh = torch.nonzero(b.extra["free_mask"] & ~used).flatten()
    ctx = b.context_lens.cpu()
    move = torch.randperm(b.B, generator=torch.Generator().manual_seed(5))[:max(1, b.B // 10)].tolist()
    bs, o, moved = b.block_size, 0, 0
    rows_k = b.k_cache.permute(0, 2, 1, 3).reshape(-1, b.Hkv, b.D)  # [slot, head, D] view of the pool
    rows_v = b.v_cache.permute(0, 2, 1, 3).reshape(-1, b.Hkv, b.D)
    for r in move:
        n = int(ctx[r])
        if n == 0:
            continue
        npg = (n + bs - 1) // bs
        t = torch.arange(n)
        old = (bt[r, t // bs] * bs + t % bs).to(device)
        bt[r, :npg] = fresh[o:o + npg]
        o += npg
        kv_paged_scatter(rows_k[old], rows_v[old], b.k_cache, b.v_cache, (bt[r, t // bs] * bs + t % bs).to(device))
        moved += 2 * 2 * n * b.Hkv * b.D * 2  # K and V, read and write
    table = bt.to(device)
    attn = PagedAttentionCall(q_rot, b.k_cache, b.v_cache, table, b.context_lens, q_start=b.q_start,
                              max_q_len=b.max_q_len)

    def run(ev0=None, ev1=None):
        ra.run()
        if ev0 is not None:
            ev0.record()
        attn.run()
        if ev1 is not None:
            ev1.record()

    total_ms, kern_ms = timed_steps(run, args.steps, args.warmup, None, None, with_kernel_events=True)
    km = statistics.mean(kern_ms)
    qs = b.q_start.cpu().tolist()
    pairs = 0  # (query token, visible key) pairs under the bottom-right causal rule
    for r in range(b.B):
        n, c = qs[r + 1] - qs[r], int(ctx[r])
        pairs += n * (c - n) + n * (n + 1) // 2
    flops = 4.0 * b.Hq * b.D * pairs
    kv = float(b.kv_bytes())
    peak, _ = measured_peak()
    return {"config": "cfg5: bf16 mixed batch, 64 requests x U[1,64] new tokens on contexts U[0,16384], 28q/4kv "
                      f"heads, D=128, page 16, {b.num_blocks:,}-page pool (40 % free), 10 % of requests compacted",
            "value": b.n_tokens * args.steps / (total_ms * 1e-3), "unit": UNIT, "ms_per_step": total_ms / args.steps,
            "kernel": {3: "prefill_tc_kernel + decode_mma_kernel (one-row requests)", 2: "prefill_tc_kernel",
                       1: "decode_mma_kernel"}.get(attn.kernel_kind, "scalar"),
            "kernel_ms": km, "kv_gigabytes": kv / 1e9, "hbm_gbs": kv / (km * 1e-3) / 1e9,
            "hbm_frac": kv / (km * 1e-3) / 1e9 / peak, "tflops": flops / (km * 1e-3) / 1e12,
            "compaction_requests": len(move), "compaction_gigabytes_moved": moved / 1e9,
            "l2": "inputs larger than L2", "status": attn.workspace.status()}


def measure_int8_kv(args, device):
    """The headline decode configuration (cfg4) on an int8 pool with one fp32 scale per (position, kv
    head): the same step -- quantising RoPE + append, plan, the decode kernel's int8 instantiation,
    combine -- with the K+V bytes roughly halved. Algorithmic bytes: (D + 4) per key and kv head for
    K and for V."""
    workloads = load_workloads()
    from kernels.attention import PagedAttentionCall, PagedWorkspace, RopeAppendCall
    b = workloads.cfg4(device=device, seed=3, B=args.requests or None)

    def quantise(cache):  # row-wise absmax quantiser with torch ops, a slice of pages at a time
        q = torch.empty(cache.shape, dtype=torch.int8, device=device)
        sc = torch.empty(cache.shape[:3], dtype=torch.float32, device=device)
        step = 4096
        for i in range(0, cache.shape[0], step):
            x = cache[i:i + step].float()
            amax = x.abs().amax(dim=-1)
            s_ = torch.where(amax > 0, amax / 127.0, torch.ones_like(amax))
            q[i:i + step] = torch.round(x / s_.unsqueeze(-1)).clamp_(-127, 127).to(torch.int8)
            sc[i:i + step] = s_
        return q, sc

    kq, ks = quantise(b.k_cache)
    b.k_cache = None
    vq, vs = quantise(b.v_cache)
    b.v_cache = None
    torch.cuda.empty_cache()
    ws = PagedWorkspace(device)
    ra = RopeAppendCall(b.k_new, b.v_new, kq, vq, b.slot_mapping, b.positions, b.cos, b.sin, k_scales=ks, v_scales=vs)
    attn = PagedAttentionCall(b.q_new, kq, vq, b.block_table, b.context_lens, rope_cos=b.cos, rope_sin=b.sin,
                              rope_positions=b.positions, workspace=ws, k_scales=ks, v_scales=vs)

    def run(ev0=None, ev1=None):
        ra.run()
        attn.plan()
        if ev0 is not None:
            ev0.record()
        attn.partials_final()
        if ev1 is not None:
            ev1.record()

    total_ms, _ = timed_steps(lambda: run(), args.steps, args.warmup, None, None)
    _, kern_ms = timed_steps(run, args.steps, 1, None, None, with_kernel_events=True)
    km = statistics.mean(kern_ms)
    keys = int(b.context_lens.sum().item())
    nbytes = 2.0 * b.Hkv * keys * (b.D + 4)
    peak, _ = measured_peak()
    # sanity against the oracle on the first request (float32 attention over the dequantised pages)
    import oracle
    r, ctx = 0, int(b.context_lens[0])
    pages = b.block_table[r, :(ctx + b.block_size - 1) // b.block_size]
    kd = oracle.kv_dequantize(kq[pages].cpu(), ks[pages].cpu())
    vd = oracle.kv_dequantize(vq[pages].cpu(), vs[pages].cpu())
    pos = b.positions[r:r + 1].cpu().long()
    q_rot = oracle.apply_rope(b.q_new[r:r + 1].cpu().unsqueeze(0), b.cos.cpu()[pos], b.sin.cpu()[pos])[0]
    ref = oracle.paged_attention_composed(q_rot.float(), kd, vd, torch.arange(pages.numel()).view(1, -1),
                                          torch.tensor([ctx], dtype=torch.int32))
    err = (attn.out[r].cpu().float() - ref[0]).abs().max().item()
    return {"config": "cfg4 on an int8 pool: 256 requests, ctx U[8192,32768], 64q/8kv heads, D=128, page 32, int8 K and V "
                      "with one fp32 scale per (position, kv head)",
            "value": b.n_tokens * args.steps / (total_ms * 1e-3), "unit": UNIT, "ms_per_step": total_ms / args.steps,
            "kernel": "decode_mma_kernel (int8)" if attn.kernel_kind == 1 else "scalar", "kernel_ms": km,
            "kv_gigabytes": nbytes / 1e9, "hbm_gbs": nbytes / (km * 1e-3) / 1e9, "hbm_frac": nbytes / (km * 1e-3) / 1e9 / peak,
            "max_abs_err_vs_oracle": err, "status": ws.status()}


def measure_steps_vs_clocks(args, device):
    """The headline decode step timed over a short and a long run in one process, with the SM clock and
    the board power sampled during each: does the rate depend on how long the GPU has been under load
    (power cap, clocks)? `kernel_ms x MHz` is the kernel's length in SM cycles (millions)."""
    out = {}
    batch = build_batch("cfg4", device, 3, "request", 0, 1, args.requests)
    packed, batch = pack_step_inputs(batch)
    step = DecodeStep(batch)
    kv = batch.kv_bytes()
    for steps in (20, 400):
        sampler = ClockSampler(device.index or 0)
        sampler.start()
        time.sleep(0.3)
        sampler.mark_begin()
        _, kern = timed_steps(step.run, steps, 3, None, None, with_kernel_events=True)
        sampler.mark_end()
        c = sampler.stop()
        km = statistics.mean(kern)
        out[f"{steps}_steps"] = {"kernel_ms": km, "kernel_ms_first5": statistics.mean(kern[:5]), "kernel_ms_last5": statistics.mean(kern[-5:]),
                                 "gbs": kv / (km * 1e-3) / 1e9, "sm_mhz_median": c["sm_mhz"], "power_w_median": c.get("power_w_median"),
                                 "power_w_max": c.get("power_w_max"), "reasons": c["reasons"],
                                 "kernel_mcycles": km * 1e-3 * (c["sm_mhz"] or 0)}
        time.sleep(1.0)
    return out


def measure_linear_norm(args, device):
    """Fused linear + norm on the shapes of the reference's own benchmark
    (benchmark/bench_fused_linear_norm.py:24-29): one call = GEMM with the row statistics in its
    epilogue + the norm over the output. FLOPs counted as the reference does (2*M*K*N)."""
    from kernels.fused_linear_norm import LinearNormCall
    peak = 1590.0
    try:
        peak = float(json.loads((ROOT / "MEASURED_PEAKS.json").read_text()).get("bf16_tflops", peak))
    except Exception:
        pass
    shapes = [("llama8b_mlp_in", 1024, 4096, 14336, "rms", torch.bfloat16),
              ("llama8b_attn_out", 1024, 4096, 4096, "rms", torch.bfloat16),
              ("gpt2_mlp_in", 4096, 768, 3072, "layer", torch.float16),
              ("decode_small", 1, 4096, 4096, "rms", torch.bfloat16)]
    out = {}
    g = torch.Generator(device=device).manual_seed(9)
    flush_buf = torch.empty(512 << 20, dtype=torch.uint8, device=device)
    for name, M, K, N, norm, dt in shapes:
        x = torch.randn(M, K, device=device, generator=g).to(dt)
        w = (torch.randn(N, K, device=device, generator=g) * K ** -0.5).to(dt)
        bias = torch.randn(N, device=device, generator=g).to(dt)
        gamma = torch.randn(N, device=device, generator=g).to(dt)
        beta = torch.randn(N, device=device, generator=g).to(dt) if norm == "layer" else None
        call = LinearNormCall(x, w, bias=bias, gamma=gamma, beta=beta, norm_type=norm)
        # the call's launches (memset, GEMM, norm) replayed from a CUDA graph: these run for tens of
        # microseconds, less than the Python call path; L2 flushed between replays (weights > L2
        # only for the largest shape)
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            call.run()
            torch.cuda.synchronize()
            cg = torch.cuda.CUDAGraph()
            with torch.cuda.graph(cg, stream=side):
                call.run()
        torch.cuda.synchronize()
        total_ms, _ = timed_steps(cg.replay, args.steps, args.warmup, lambda: flush_buf.zero_(), None)
        ms = total_ms / args.steps
        flops = 2.0 * M * K * N
        moved = (M * K + N * K + M * N) * x.element_size()
        out[name] = {"M": M, "K": K, "N": N, "norm": norm, "dtype": str(dt).replace("torch.", ""),
                     "kernel": {1: "linear_stats_tc_kernel", 2: "linear_stats_small_m_kernel"}.get(call.kernel_kind, "generic"),
                     "ms": ms, "tflops": flops / (ms * 1e-3) / 1e12, "frac_of_bf16_peak": flops / (ms * 1e-3) / 1e12 / peak,
                     "gbs_min_traffic": moved / (ms * 1e-3) / 1e9, "l2": "512 MiB memset between timed replays",
                     "status": call.workspace.status()}
    return out


def measure_small_ops(args, device):
    """The bandwidth-bound ops of the path on the reference's own benchmark shapes
    (benchmark/bench_kv_cache.py, bench_rope.py, bench_softmax.py:20-25) and a few more. These calls run
    for tens of microseconds, less than the Python call path and not much more than the eight or so
    microseconds a lone kernel between two events costs anyway, so each op is timed as a CUDA graph of
    several calls on DIFFERENT inputs (together several times the 126 MB of L2, so no call finds its
    input there) and the time is divided by the number of calls. Bytes as the reference counts them."""
    from kernels.kv_cache import kv_paged_append, kv_paged_lookup
    from kernels.rope import apply_rope_, build_rope_tables
    from kernels.softmax import online_softmax
    peak, _ = measured_peak()
    bf, f16, f32 = torch.bfloat16, torch.float16, torch.float32
    out = {}

    def timed(calls):
        """calls: closures, one per input set; returns ms per call."""
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            for c in calls:
                c()
            torch.cuda.synchronize()
            cg = torch.cuda.CUDAGraph()
            with torch.cuda.graph(cg, stream=side):
                for c in calls:
                    c()
        torch.cuda.synchronize()
        total_ms, _ = timed_steps(cg.replay, args.steps, args.warmup, None, None)
        return total_ms / args.steps / len(calls)

    def put(name, ms, nbytes, n_inputs):
        out[name] = {"us": ms * 1e3, "gbs": nbytes / (ms * 1e-3) / 1e9, "frac_of_hbm_peak": nbytes / (ms * 1e-3) / 1e9 / peak,
                     "calls_per_timed_graph": n_inputs}

    def copies(nbytes_per_call):  # enough inputs that a graph replay touches at least four times L2
        return max(2, min(16, -(-4 * 126_000_000 // max(nbytes_per_call, 1))))

    def want(label):
        return not getattr(args, "small_filter", None) or args.small_filter in label

    g = torch.Generator(device=device).manual_seed(11)
    N, H, D, bs = 131072, 8, 128, 16
    if want("kv_paged_append 131072 tokens x 8 heads bf16"):
        k = torch.randn(N, H, D, device=device, generator=g).to(bf)
        v = torch.randn(N, H, D, device=device, generator=g).to(bf)
        kc = torch.zeros(N // bs + 8, H, bs, D, dtype=bf, device=device)
        vc = torch.zeros_like(kc)
        slots = torch.randperm(kc.shape[0] * bs, device=device, generator=g)[:N]
        nb = 2 * 2 * N * H * D * 2 + 8 * N
        put("kv_paged_append 131072 tokens x 8 heads bf16", timed([lambda: kv_paged_append(k, v, kc, vc, slots)] * 2), nb, 2)
        del k, v, kc, vc
    B, ctx, H = 8, 8192, 32
    if want("kv_paged_lookup 8 x 8192 x 32 heads bf16"):
        kc = torch.randn(B * ctx // bs, H, bs, D, device=device, generator=g).to(bf)
        vc = torch.randn(B * ctx // bs, H, bs, D, device=device, generator=g).to(bf)
        bt = torch.randperm(kc.shape[0], device=device, generator=g).view(B, -1)
        lens = torch.full((B,), ctx, dtype=torch.int32, device=device)
        nb = 2 * 2 * B * H * ctx * D * 2
        put("kv_paged_lookup 8 x 8192 x 32 heads bf16", timed([lambda: kv_paged_lookup(kc, vc, bt, lens, ctx)] * 2), nb, 2)
        del kc, vc
    if want("apply_rope_ 8 x 2048 x 32 x 128 bf16"):
        cos, sin = build_rope_tables(2048, D, base=1e6, device=device, dtype=bf)
        nb = 2 * 8 * 2048 * 32 * D * 2
        xs = [torch.randn(8, 2048, 32, D, device=device, generator=g).to(bf) for _ in range(copies(nb))]
        put("apply_rope_ 8 x 2048 x 32 x 128 bf16", timed([(lambda t=t: apply_rope_(t, cos, sin)) for t in xs]), nb, len(xs))
        del xs
    # online_softmax: the reference's four (bench_softmax.py:20-25), then bf16 / fp32 shapes of the path
    # (the reference writes its two causal cases as [B, 32*S, S], which its own square check refuses,
    # triton_softmax.py:146-151; here the same rows as [B*32, S, S])
    shapes = [("attn_score_2k", (4 * 32, 2048, 2048), f16, True, False), ("attn_score_8k", (4, 8192, 8192), f16, True, False),
              ("lm_head_50k", (8, 1024, 50257), f16, False, False), ("logsoftmax_1k", (8, 1024, 1024), f16, False, True),
              ("", (4096, 4096), bf, False, False), ("", (512, 50257), bf, False, False), ("", (32768, 1024), bf, False, False),
              ("", (8192, 8192), bf, False, False), ("", (8192, 8192), f32, False, False), ("", (4096, 4096), f32, False, False)]
    for tag, shape, dt, causal, log in shapes:
        numel = 1
        for d_ in shape:
            numel *= d_
        nb = 2 * numel * torch.empty((), dtype=dt).element_size()
        n_in = copies(nb) if nb < 1_000_000_000 else 1
        label = f"online_softmax {tag + ' ' if tag else ''}{' x '.join(map(str, shape))} {str(dt)[6:]}" + \
                (" causal" if causal else "") + (" log" if log else "")
        if not want(label):
            continue
        xs = [torch.randn(*shape, device=device, generator=g, dtype=torch.float32).to(dt) for _ in range(n_in)]
        calls = [(lambda t=t: online_softmax(t, is_causal=causal, log=log)) for t in xs]
        if n_in == 1:
            calls = calls * 2
        put(label, timed(calls), nb, len(calls))
        del xs, calls
        torch.cuda.empty_cache()
    return out


def check_against_oracle(res, n_req=2):
    """Cheap sanity outside every timed region: first requests of the batch vs the CPU oracle."""
    import oracle
    b = res["batch"]
    held, res["step"].gather = res["step"].gather, None  # this check runs on one rank alone: local heads, plain combine
    out = res["step"].run()
    torch.cuda.synchronize()
    res["step"].gather = held
    n = min(n_req, b.B)
    errs = []
    for r in range(n):
        ctx = int(b.context_lens[r])
        npg = (ctx + b.block_size - 1) // b.block_size
        pages = b.block_table[r, :npg]
        kc, vc = b.k_cache[pages].cpu(), b.v_cache[pages].cpu()
        bt = torch.arange(npg).view(1, -1)
        pos = b.positions[r:r + 1].cpu().long()
        cos, sin = b.cos.cpu(), b.sin.cpu()
        q_rot = oracle.apply_rope(b.q_new[r:r + 1].cpu().unsqueeze(0), cos[pos], sin[pos])[0]
        ref = oracle.paged_attention_composed(q_rot, kc, vc, bt, torch.tensor([ctx], dtype=torch.int32))
        errs.append((out[r].cpu().float() - ref[0].float()).abs().max().item())
    return max(errs) if errs else 0.0


def emit_block(name: str, block: dict) -> None:
    """A secondary block as its own stdout line, ahead of the result line."""
    print(json.dumps({"block": name, **block}), flush=True)


def run_ours(args):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus > 1 and world == 1:
        # convenience: relaunch under torchrun
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", "29531", __file__] + sys.argv[1:]
        raise SystemExit(subprocess.call(cmd))
    use_package()
    from kernels import _native
    _native.lib()  # no fallback: fail here if the CUDA library is missing
    assert torch.cuda.is_available(), "bench.py needs a GPU for --impl ours"
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist_mod.init_process_group("nccl", device_id=device)
        dist = dist_mod

    shard = args.shard or "request"
    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.start()
    res = measure(args.workload, args, device, rank, world, dist, sampler=sampler, shard=shard, gather_kind=args.gather)
    clocks = sampler.stop() if sampler else None
    total_ms, e2e_ms, kernel_ms, all_tokens, all_bytes = whole_job(res, dist, device, shard, world)

    peak, peak_kind = measured_peak()
    line = None
    if rank == 0:
        achieved = res["kv_bytes"] / (res["kernel_ms"] * 1e-3) / 1e9  # this rank's kernel, GB/s
        line = {
            "metric": METRIC,
            "value": all_tokens * args.steps / (total_ms * 1e-3),
            "unit": UNIT,
            "n_gpus": world,
            "steps": args.steps,
            "warmup": args.warmup,
            "ms_per_step": total_ms / args.steps,
            "higher_is_better": True,
            "scaling": "weak" if shard == "replica" else "strong",
            "vs_baseline": None,
            "dtype": "bf16",
            "data": "synthetic",
            "config": line_config(args.workload, shard, {
                **({"head_gather": args.gather, "head_gather_check": res["gather_check"]}
                   if shard == "head" and world > 1 else {}),
                **({"requests_override": args.requests} if args.requests else {}),
                **({"cuda_graph": True} if args.graph else {})}),
            "e2e": {"value": all_tokens * args.steps / (e2e_ms * 1e-3), "unit": UNIT,
                    "h2d_bytes_per_step": res["h2d"], "d2h_bytes_per_step": res["d2h"],
                    "ms_per_step": e2e_ms / args.steps},
            "gpu_launches": res["launches"],
            "roofline": {"bound": "hbm", "kernel": "decode_mma_kernel" if res["kernel_kind"] == 1 else "paged_partial_generic_kernel",
                         "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_kind": peak_kind, "frac_of_nominal_8000": achieved / 8000.0,
                         "algorithmic_bytes_per_launch": res["kv_bytes"], "kernel_ms": res["kernel_ms"],
                         "kernel_ms_min": res["kernel_ms_min"], "traffic": None},
            "step_fixed_cost_ms": (total_ms / args.steps) - kernel_ms,
            "ms_per_step_plan_reused": (res["plan_reused_ms"] / args.steps) if res.get("plan_reused_ms") else None,
            "clocks": clocks,
            "device_status_word": res["status"],
        }
        # DRAM bytes per algorithmic byte from the ncu captures summarised under profiles/
        # (decode_mma_kernel_cfg4.md: 16-request case, traffic grows in proportion to the keys;
        # decode_mma_kernel_cfg2.md: the whole configuration).
        ratio = {"cfg4": 1.0049, "cfg2": 1.0386}[args.workload]
        if res["kernel_kind"] == 1:
            line["roofline"]["traffic"] = ratio * res["kv_bytes"]
            line["roofline"]["traffic_note"] = f"{ratio} x algorithmic bytes, ncu dram__bytes_read+write, see profiles/"
        line["max_abs_err_vs_oracle"] = check_against_oracle(res)
    release(res)

    if world > 1 and args.shard is None:
        # The same one batch in the other partitionings, all on this run's clock: kv-head sharding with
        # the gather fused into the combine kernel and with an NCCL all-gather, and independent replicas.
        others = {}
        for name, sh, gk in (("head_fused", "head", "fused"), ("head_nccl", "head", "nccl"), ("replica", "replica", None)):
            if dist is not None:
                dist.barrier()
            r2 = measure(args.workload, args, device, rank, world, dist, want_e2e=False, shard=sh, gather_kind=gk or "fused")
            t_ms, _, k_ms, toks, _ = whole_job(r2, dist, device, sh, world)
            others[name] = {"value": toks * args.steps / (t_ms * 1e-3), "unit": UNIT, "ms_per_step": t_ms / args.steps,
                            "kernel_ms": k_ms, "step_fixed_cost_ms": t_ms / args.steps - k_ms,
                            "scaling": "weak" if sh == "replica" else "strong", "device_status_word": r2["status"],
                            **({"head_gather_check": r2["gather_check"]} if name == "head_fused" else {})}
            release(r2)
        if line is not None:
            line["other_shards"] = others

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(args.workload, args.cpu_sample)
    if world == 1 and not args.no_extra:
        secondary = {}
        other = "cfg2" if args.workload == "cfg4" else "cfg4"
        r2 = measure(other, args, device, rank, world, dist)
        ach2 = r2["kv_bytes"] / (r2["kernel_ms"] * 1e-3) / 1e9
        blk = {"config": workload_desc(other)["workload"], "value": r2["tokens"] * args.steps / (r2["total_ms"] * 1e-3),
               "unit": UNIT, "ms_per_step": r2["total_ms"] / args.steps, "e2e_ms_per_step": r2["e2e_ms"] / args.steps,
               "roofline_achieved_gbs": ach2, "roofline_frac": ach2 / peak, "kernel_ms": r2["kernel_ms"],
               "ms_per_step_plan_reused": (r2["plan_reused_ms"] / args.steps) if r2["plan_reused_ms"] else None,
               "plan_reused_note": "layers 2..N of a decode step: the plan of layer 1 is kept (reuse_plan), two launches",
               "l2": r2["flush"], "device_status_word": r2["status"]}
        emit_block(other, blk)
        secondary[f"{other}_frac"] = blk["roofline_frac"]
        secondary[f"{other}_ms_per_step"] = blk["ms_per_step"]
        release(r2)
        blk = measure_prefill(args, device)
        emit_block("cfg3", blk)
        secondary.update(cfg3_frac=blk["roofline"]["frac"], cfg3_kernel_ms=blk["kernel_ms"])
        torch.cuda.empty_cache()
        blk = measure_mixed(args, device)
        emit_block("cfg5", blk)
        secondary.update(cfg5_frac=blk["hbm_frac"], cfg5_kernel_ms=blk["kernel_ms"])
        torch.cuda.empty_cache()
        blk = measure_int8_kv(args, device)
        emit_block("cfg4_int8_kv", blk)
        secondary.update(cfg4_int8_frac=blk["hbm_frac"], cfg4_int8_ms_per_step=blk["ms_per_step"])
        torch.cuda.empty_cache()
        blk = measure_linear_norm(args, device)
        emit_block("fused_linear_norm", blk)
        torch.cuda.empty_cache()
        blk = measure_small_ops(args, device)
        emit_block("small_ops", blk)
        secondary["small_ops_frac"] = {k: round(v["frac_of_hbm_peak"], 3) for k, v in blk.items()}
        line["secondary"] = secondary
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def run_only(args):
    use_package()
    from kernels import _native
    _native.lib()
    assert torch.cuda.is_available(), "bench.py needs a GPU"
    device = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    block = {"cfg3": measure_prefill, "cfg5": measure_mixed, "linear_norm": measure_linear_norm,
             "small_ops": measure_small_ops, "int8_kv": measure_int8_kv, "clocks": measure_steps_vs_clocks}[args.only](args, device)
    print(json.dumps({"only": args.only, "steps": args.steps, "warmup": args.warmup, **block}), flush=True)


def main():
    args = parse_args()
    if args.only:
        run_only(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
