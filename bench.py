#!/usr/bin/env python
"""Benchmark of the MoBA prefill hot path (routing + forward + backward) on B200.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (N = 1 and per rank for N > 1): GQA prefill forward+backward at the Qwen2-0.5B attention
shape: 4 packed sequences of 32768 tokens, 14 query / 2 KV heads, head_dim 64, MoBA chunk 2048,
topk 3, bf16 Q/K/V ~ N(0,1)/sqrt(64), dO ~ N(0,1); synthetic, seeded.  One step = one pass of
routing + forward + backward over that batch.  The metric is attended TFLOP/s: 14 * D * pairs * Hq
FLOPs per step (pairs = attended (query, key) pairs per head) divided by the step time.

One JSON line is printed by rank 0.  `value` times the step with inputs resident in HBM; `e2e` times
the same call with pinned host buffers, including the host->device copies of q, k, v, dO and the
device->host copies of out, dq, dk, dv.  `roofline` is the backward main kernel (the dominant
kernel) timed with CUDA events recorded around its launch inside the timed region.  `cpu_baseline`
times the reference's FP64 CPU oracle on a bounded sample of the same workload.

At every N the line also carries `long_prefill`: the long-context configuration (131072 tokens, 32 / 8
heads, D=128, chunk 4096, topk 12) split by KV-head group over the N ranks (strong scaling: N = 1 runs
all 8 groups), with the NCCL all-gather of the forward output inside the timed region; `decode`:
64 paged-decode requests spread over the ranks by context length; and, at N > 1, `headline_split`: the
headline configuration itself as one job over the ranks, split by KV head and then by sequence (its 2 KV
heads x 4 sequences are 8 independent units), outputs all-gathered the same way.

--impl reference times the CPU implementation of the path on all host threads: the reference's own
reference/grouped_reference.py (forward + autograd backward, FP64) when oracle/make_ref.py has put it
under oracle/_ref, else the numpy port of it.
"""
import argparse
import json
import os
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT / "moba-merge-cuda_b200"))
sys.path.insert(0, str(ROOT))

WORKLOADS = {
    # BASELINE configs[1]: the configuration the metric is quoted on
    "cfg2": dict(name="gqa_prefill_4x32768_h14kv2_d64_c2048_k3", lens=(32768,) * 4, hq=14, hkv=2, dim=64, chunk=2048, topk=3),
    # one of the four sequences: the small case used for multi-pass profiler captures
    "small": dict(name="gqa_prefill_1x32768_h14kv2_d64_c2048_k3", lens=(32768,), hq=14, hkv=2, dim=64, chunk=2048, topk=3),
    # BASELINE configs[2], the shard one GPU gets at 8 GPUs (one KV head and its 4 query heads), and half of it for
    # multi-pass profiler captures; unit-variance inputs as that config states
    "cfg3_shard": dict(name="gqa_prefill_1x131072_h4kv1_d128_c4096_k12", lens=(131072,), hq=4, hkv=1, dim=128, chunk=4096, topk=12,
                       unit_variance=True),
    "cfg3_small": dict(name="gqa_prefill_1x65536_h4kv1_d128_c4096_k12", lens=(65536,), hq=4, hkv=1, dim=128, chunk=4096, topk=12,
                       unit_variance=True),
}
WORKLOAD = WORKLOADS["cfg2"]
TRAFFIC_TABLE = ROOT / "profiles" / "dram_traffic.txt"
METRIC = "moba_prefill_fwd_bwd_attended_tflops"
UNIT = "TFLOP/s"


def attended_pairs(lens, chunk, topk):
    total = 0
    for length in lens:
        n = (length + chunk - 1) // chunk
        for c in range(n):
            s = chunk if c < n - 1 else length - (n - 1) * chunk
            total += s * (s + 1) // 2 + s * min(topk - 1, c) * chunk
    return total


def step_flops(w):
    return 14.0 * w["dim"] * attended_pairs(w["lens"], w["chunk"], w["topk"]) * w["hq"]


def kernel_source_digest(*names):
    """sha256 (16 hex digits) over the named files of the kernel sources: ties a profiled figure to the code it was
    taken from."""
    import hashlib
    h = hashlib.sha256()
    for name in names:
        h.update((ROOT / "moba-merge-cuda_b200" / "csrc" / name).read_bytes())
    return h.hexdigest()[:16]


def measured_traffic(kernel, sources, units):
    """DRAM bytes per launch (ncu dram__bytes_read.sum + dram__bytes_write.sum) of `kernel` from the table of
    profiled figures, scaled by `units` (the table is per unit, e.g. per 32768-token sequence), or None when the
    kernel's sources have changed since the figure was taken."""
    if not TRAFFIC_TABLE.exists():
        return None, "no profiled figure"
    digest = kernel_source_digest(*sources)
    for line in TRAFFIC_TABLE.read_text().splitlines():
        f = line.split()
        if len(f) >= 4 and not line.startswith("#") and f[0] == kernel:
            if f[1] == digest:
                return float(f[2]) * units, "ncu dram__bytes_read.sum + dram__bytes_write.sum of one launch on %s, times %d" % (" ".join(f[3:]), units)
            return None, "kernel sources changed since the profiled figure was taken"
    return None, "no profiled figure"


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return dict(tflops=float(d["bf16_tflops_sustained"]), hbm=float(d["hbm_gbs"]), source="measured")
    return dict(tflops=1400.0, hbm=6650.0, source="fallback")


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML while the timed region runs (read-only)."""

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.max_mhz = index, [], set(), None
        self._halt = threading.Event()

    def run(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            h = nv.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)
            names = {getattr(nv, k): k for k in dir(nv) if k.startswith("nvmlClocksEventReason") or
                     k.startswith("nvmlClocksThrottleReason")}
            while not self._halt.is_set():
                self.samples.append(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM))
                try:
                    bits = nv.nvmlDeviceGetCurrentClocksEventReasons(h)
                except Exception:
                    bits = nv.nvmlDeviceGetCurrentClocksThrottleReasons(h)
                for value, name in names.items():
                    if isinstance(value, int) and value and bits & value and "None" not in name and "All" not in name:
                        self.reasons.add(name.replace("nvmlClocksEventReason", "").replace("nvmlClocksThrottleReason", ""))
                time.sleep(0.01)
        except Exception as exc:  # NVML missing: report that instead of clocks
            self.reasons.add(f"nvml_unavailable:{type(exc).__name__}")

    def stop(self):
        self._halt.set()
        self.join(timeout=2)
        mhz = float(np.median(self.samples)) if self.samples else None
        return dict(sm_mhz=mhz, sm_max_mhz=self.max_mhz, reasons=sorted(self.reasons), samples=len(self.samples))


# ----------------------------------------------------------------------------- CPU arm
CPU_SAMPLE_TOKENS = 6144


def cpu_sample(threads):
    """The CPU implementation of the path on a bounded sample of the workload: the first 6144 tokens (three chunks, so
    rows with 0, 1 and 2 routed blocks) of sequence 0 with KV head 0 and its 7 query heads.  Attention is causal, so
    this prefix is computed exactly as inside the full batch.  Routing (numpy port of the reference's torch routing,
    which has no CPU entry point of its own) + the reference's reference/grouped_reference.py forward + autograd
    backward in FP64 when oracle/_ref holds it, else the numpy port of that oracle.
    Returns (TFLOP/s on attended FLOPs, description, seconds, kind)."""
    import torch
    from oracle import moba_oracle as mo
    from oracle.make_ref import load_ref
    w = WORKLOAD
    L, G, D, C = min(CPU_SAMPLE_TOKENS, w["lens"][0]), w["hq"] // w["hkv"], w["dim"], w["chunk"]
    rng = np.random.default_rng(0)
    bf = mo.bf16_round
    scale = 1.0 if w.get("unit_variance") else D ** -0.5
    q = bf(rng.standard_normal((L, G, D)) * scale)
    k = bf(rng.standard_normal((L, 1, D)) * scale)
    v = bf(rng.standard_normal((L, 1, D)) * scale)
    do = bf(rng.standard_normal((L, G, D)))
    cu = np.array([0, L])
    ref = load_ref()
    torch.set_num_threads(threads)
    t0 = time.perf_counter()
    r = mo.route_prefill(q, k, cu, C, w["topk"])
    if ref is not None:
        grouped_reference = ref[0]
        route = dict(cu_chunk=torch.from_numpy(r["cu_chunk"]), chunk_to_batch=torch.from_numpy(r["chunk_to_batch"]),
                     filtered_chunk_indices=torch.from_numpy(r["filtered"]), selected=torch.from_numpy(r["selected"]),
                     cu_seqlens=torch.from_numpy(cu))
        qt, kt, vt = (torch.from_numpy(x).requires_grad_(True) for x in (q, k, v))
        out = grouped_reference(qt, kt, vt, torch.from_numpy(cu), route)
        torch.autograd.grad(out, (qt, kt, vt), grad_outputs=torch.from_numpy(do))
        kind, what = "reference", "the reference's reference/grouped_reference.py forward + autograd backward (FP64 torch)"
    else:
        mo.attention_fixed_route(q, k, v, cu, r["sel"], C, d_out=do)
        kind, what = "port", "numpy FP64 port of the reference's grouped_reference oracle, forward + backward"
    dt = time.perf_counter() - t0
    flops = 14.0 * D * attended_pairs((L,), C, w["topk"]) * G
    desc = ("first %d tokens of sequence 0, KV head 0 with its %d query heads: routing (numpy port) + %s" % (L, G, what))
    return flops / dt / 1e12, desc, dt, kind


def cpu_decode_sample(threads):
    """CPU baseline of the decode leg: the reference's reference/decode_reference.py (per-(row, head) FP64 loop; the
    numpy port of it when oracle/_ref is absent) on the first 4 requests of the decode workload, routed by the numpy
    port of the reference's decode routing.  Returns dict(tokens_per_s, requests, seconds, kind)."""
    import torch
    from oracle import moba_oracle as mo
    from oracle.make_ref import load_ref
    w = DECODE
    rng = np.random.default_rng(0)
    lens = [int(x) for x in rng.integers(w["lo"], w["hi"] + 1, size=w["requests"])][:4]
    bf = mo.bf16_round
    keys = [bf(rng.standard_normal((n, w["hkv"], w["dim"]))) for n in lens]
    values = [bf(rng.standard_normal((n, w["hkv"], w["dim"]))) for n in lens]
    q = bf(rng.standard_normal((len(lens), w["hq"], w["dim"])))
    ids, pos = list(range(len(lens))), [n - 1 for n in lens]
    ref = load_ref()
    torch.set_num_threads(threads)
    t0 = time.perf_counter()
    means = [mo.chunk_means(kk, w["chunk"], rounding=bf) for kk in keys]
    sel = mo.decode_route(q, means, ids, pos, w["chunk"], w["topk"])["selected"]
    if ref is not None:
        ref[1](torch.from_numpy(q), [torch.from_numpy(x) for x in keys], [torch.from_numpy(x) for x in values], ids, pos,
               chunk_size=w["chunk"], selected_blocks=torch.from_numpy(sel))
        kind = "reference"
    else:
        mo.decode_attend(q, keys, values, ids, pos, w["chunk"], sel)
        kind = "port"
    dt = time.perf_counter() - t0
    return dict(tokens_per_s=len(lens) / dt, requests=len(lens), seconds=dt, kind=kind, cores=threads,
                sample="first 4 requests: chunk means + routing (numpy port) + decode_reference (FP64)")


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    vals = []
    for i in range(args.warmup + args.steps):
        val, sample, dt, kind = cpu_sample(threads)
        if i >= args.warmup:
            vals.append((val, dt))
        if sum(d for _, d in vals) > 100 or (i + 1) * dt > 160:  # keep the whole run within a few minutes
            if not vals:
                vals.append((val, dt))
            break
    value = float(np.mean([v for v, _ in vals]))
    ms = float(np.mean([d for _, d in vals])) * 1e3
    line = dict(impl="reference", metric=METRIC, value=value, unit=UNIT, n_gpus=args.gpus, steps=len(vals),
                warmup=args.warmup, ms_per_step=ms, higher_is_better=True, scaling="weak", vs_baseline=None, dtype="f64",
                data="synthetic", config=dict(workload=WORKLOAD["name"], sample=sample),
                cpu_baseline=dict(value=value, unit=UNIT, cores=threads, kind=kind, sample=sample),
                e2e=dict(value=value, unit=UNIT, h2d_bytes_per_step=0, d2h_bytes_per_step=0), gpu_launches=0)
    print(json.dumps(line))


# ----------------------------------------------------------------------------- decode leg
DECODE = dict(name="paged_decode_64req_ctx4k-64k_page48_c2048_k4_h12kv2_d128", requests=64, lo=4096, hi=65536, page=48,
              chunk=2048, topk=4, hq=12, hkv=2, dim=128, steps=512)


def run_decode(dev, rank, world, steps, lib):
    """BASELINE configs[3]: 64 requests spread over the ranks (independent shards, each rank its own cache and
    captured step), context lengths uniform in [4096, 65536] from seed 0, page 48, chunk 2048, topk 4, 12/2 heads,
    D=128, K/V ~ N(0,1) in randomly permuted physical pages; one new token per request per step under
    prepare_decode + CUDA graph.  Requests go to ranks by the bytes a step is expected to read for them
    (sharding.balance_requests over sharding.expected_decode_tokens), not round-robin: the step time of the job is
    the slowest rank's.  Returns tokens/s, algorithmic HBM bytes per step (union of attended tokens per (request,
    kv head), K and V, from the actual selected tables) and timings, among them the step with the all-gather of
    the step's outputs to every rank (sharding.RowGather) included."""
    import torch
    import torch.distributed as dist
    from moba_opt import PagedKVCache, sharding
    w = DECODE
    rng = np.random.default_rng(0)
    all_lens = [int(x) for x in rng.integers(w["lo"], w["hi"] + 1, size=w["requests"])]
    costs = [sharding.expected_decode_tokens(n, w["chunk"], w["topk"], w["hq"] // w["hkv"]) for n in all_lens]
    assignment = sharding.balance_requests(costs, world)
    lens = [all_lens[i] for i in assignment[rank]]
    b = len(lens)
    extra = steps + 5 + 4 + 8 + 3 + min(steps, 128) + 16     # every step this leg takes: warm-up, timed, sampled, eager, gathered
    max_len = w["hi"] + extra
    pages = sum(-(-(n + extra) // w["page"]) for n in lens)
    cache = PagedKVCache(b, max_len, w["hkv"], w["dim"], page_size=w["page"], num_pages=pages, chunk_size=w["chunk"])
    free = list(cache._layout.free_pages)
    np.random.default_rng(1 + rank).shuffle(free)          # physical pages in random order
    cache._layout.free_pages = tuple(free)
    gen = torch.Generator(device=dev).manual_seed(7 + rank)
    slab = 2048
    done = [0] * b
    while any(d < n for d, n in zip(done, lens)):
        ids, counts = [], []
        for i in range(b):
            if done[i] < lens[i]:
                ids.append(i)
                counts.append(min(slab, lens[i] - done[i]))
        total = sum(counts)
        k = torch.randn(total, w["hkv"], w["dim"], device=dev, generator=gen).bfloat16()
        v = torch.randn(total, w["hkv"], w["dim"], device=dev, generator=gen).bfloat16()
        cache.append(k, v, sequence_ids=ids, cu_seqlens=[0] + [int(x) for x in np.cumsum(counts)])
        for i, c in zip(ids, counts):
            done[i] += c
    plan = cache.prepare_decode(list(range(b)), w["hq"], topk=w["topk"], check_finite=False, stable_routes=True)
    plan.capture("step")
    qs = torch.randn(8, b, w["hq"], w["dim"], device=dev, generator=gen).bfloat16()
    ks = torch.randn(8, b, w["hkv"], w["dim"], device=dev, generator=gen).bfloat16()
    vs = torch.randn(8, b, w["hkv"], w["dim"], device=dev, generator=gen).bfloat16()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(5):
        plan.step(qs[0], ks[0], vs[0], use_graph=True)
    torch.cuda.synchronize()
    sampled_bytes = []
    G = w["hq"] // w["hkv"]
    e0.record()
    h0 = time.perf_counter()
    for i in range(steps):
        r = plan.step(qs[i % 8], ks[i % 8], vs[i % 8], use_graph=True)
    host_ms = (time.perf_counter() - h0) * 1e3 / steps      # what the host spends enqueueing a step (no wait inside)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    # algorithmic bytes from the route tables of a few extra steps (outside the timed region)
    for i in range(4):
        r = plan.step(qs[i], ks[i], vs[i], use_graph=True)
        sel = r.selected_blocks.cpu().numpy()
        total = 0
        for row, pos in enumerate(r.positions):
            for g in range(w["hkv"]):
                chunks = set(int(c) for c in sel[row, g * G:(g + 1) * G].ravel() if c >= 0)
                cur = pos // w["chunk"]
                tokens = sum((pos + 1 - c * w["chunk"]) if c == cur else w["chunk"] for c in chunks)
                total += tokens * 2 * w["dim"] * 2
            total += (pos // w["chunk"]) * w["hkv"] * w["dim"] * 2      # chunk means read by routing
        sampled_bytes.append(total)
    # attention kernel alone, eager launches with events around the kernel
    a0.record(); a1.record()
    lib.moba_profile_events(4, a0.cuda_event, a1.cuda_event)
    att = []
    for i in range(8):
        plan.step(qs[i], ks[i], vs[i], use_graph=False)
        torch.cuda.synchronize()
        att.append(a0.elapsed_time(a1))
    lib.moba_profile_events(4, None, None)
    # the same steps with every rank receiving all outputs, in request order, after each step
    gather_ms = None
    if world > 1:
        n = min(steps, 128)
        gather = sharding.RowGather(assignment, plan.output)
        for _ in range(3):
            gather(plan.step(qs[0], ks[0], vs[0], use_graph=True).output)
        dist.barrier()
        torch.cuda.synchronize()
        e0.record()
        for i in range(n):
            gather(plan.step(qs[i % 8], ks[i % 8], vs[i % 8], use_graph=True).output)
        e1.record()
        torch.cuda.synchronize()
        gather_ms = e0.elapsed_time(e1) / n
    plan.close()
    return dict(ms_per_step=ms, host_ms_per_step=host_ms, requests=b, bytes_per_step=float(np.mean(sampled_bytes)),
                attend_ms=float(np.median(att)),
                context_tokens=int(sum(lens)), gather_ms_per_step=gather_ms)


def run_decode_against_reference(dev):
    """Same-machine GPU baseline of the decode leg: the reference's own PagedKVCache + prepare_decode + CUDA graph (its
    Triton kernels, from the unmodified copy oracle/make_ref.py puts under oracle/_ref) beside this package's, on one
    workload both accept - the reference's kernels stop at chunk 1024, so this is the decode configuration with chunk 1024,
    16 requests and contexts in [2048, 16384].  Returns None where oracle/_ref or triton is missing."""
    import torch
    from oracle.make_ref import load_ref_decode
    from moba_opt import PagedKVCache
    mods = load_ref_decode()
    if mods is None:
        return None
    w = dict(DECODE, requests=16, lo=2048, hi=16384, chunk=1024, steps=128)
    lens = [int(x) for x in np.random.default_rng(3).integers(w["lo"], w["hi"] + 1, size=w["requests"])]
    b, extra = len(lens), w["steps"] + 32
    out = {}
    for label, cls in (("ours", PagedKVCache), ("reference", mods[0].PagedKVCache)):
        cache = cls(b, w["hi"] + extra, w["hkv"], w["dim"], page_size=w["page"], chunk_size=w["chunk"])
        gen = torch.Generator(device=dev).manual_seed(11)
        done = [0] * b
        while any(d < n for d, n in zip(done, lens)):
            ids = [i for i in range(b) if done[i] < lens[i]]
            counts = [min(2048, lens[i] - done[i]) for i in ids]
            k = torch.randn(sum(counts), w["hkv"], w["dim"], device=dev, generator=gen).bfloat16()
            v = torch.randn(sum(counts), w["hkv"], w["dim"], device=dev, generator=gen).bfloat16()
            cache.append(k, v, sequence_ids=ids, cu_seqlens=[0] + [int(x) for x in np.cumsum(counts)])
            for i, c in zip(ids, counts):
                done[i] += c
        plan = cache.prepare_decode(list(range(b)), w["hq"], topk=w["topk"], check_finite=False, stable_routes=True)
        plan.capture("step")
        q = torch.randn(b, w["hq"], w["dim"], device=dev, generator=gen).bfloat16()
        kn = torch.randn(b, w["hkv"], w["dim"], device=dev, generator=gen).bfloat16()
        for _ in range(5):
            plan.step(q, kn, kn, use_graph=True)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(w["steps"]):
            plan.step(q, kn, kn, use_graph=True)
        e1.record()
        torch.cuda.synchronize()
        out[label] = e0.elapsed_time(e1) / w["steps"]
        plan.close()
        del cache, plan
    return dict(workload="paged_decode_16req_ctx2k-16k_page48_c1024_k4_h12kv2_d128", steps=w["steps"],
                ms_per_step=out["ours"], reference_ms_per_step=out["reference"],
                reference="the reference's PagedKVCache + prepare_decode + CUDA graph (Triton kernels), same inputs, same GPU",
                speedup=out["reference"] / out["ours"])


# ----------------------------------------------------------------------------- split-prefill legs
LONG_PREFILL = dict(name="gqa_prefill_1x131072_h32kv8_d128_c4096_k12_by_kv_group", lens=(131072,), hq=32, hkv=8, dim=128,
                    chunk=4096, topk=12, unit_variance=True)
# BASELINE configs[1] as one job over the ranks: 2 KV heads x 4 sequences = 8 independent units
HEADLINE_SPLIT = dict(WORKLOADS["cfg2"], name="gqa_prefill_4x32768_h14kv2_d64_c2048_k3_by_kv_head_and_sequence")


def run_long_prefill(dev, rank, world, steps, warmup, with_host_leg=True, w=None):
    """A prefill configuration as ONE job over the ranks (strong scaling), split into its independent units.
    w = LONG_PREFILL (default), BASELINE configs[2]: one sequence of 131072 tokens, 32 query / 8 KV heads, D=128, chunk
    4096, topk 12, bf16 Q/K/V ~ N(0,1), split by KV-head group: rank r owns 8/world KV heads and their query heads
    (world = 1 runs all eight).  w = HEADLINE_SPLIT, BASELINE configs[1]: 4 sequences of 32768 tokens, 14 / 2 heads,
    D=64, which has only two KV heads, so the ranks beyond two take whole sequences (sharding.unit_slices: 2 ranks = one KV
    head each, 4 = one KV head of two sequences, 8 = one KV head of one sequence).
    One step = routing + forward + backward on the rank's units, and the all-gather of the forward output
    [T/seq parts, Hq/head parts, D] of every rank into [T, Hq, D] on every rank (NCCL over NVLink), issued on a second
    stream as soon as the forward is done so that it runs beside the backward; the step ends when both are done.
    Gradients stay with the units they belong to (dK, dV of a KV head of a sequence live wholly on its rank), so nothing
    else is exchanged.  Timed on the device, maximum over ranks."""
    import torch
    import torch.distributed as dist
    import moba_opt
    import moba_opt.grouped_attention as ga
    from moba_opt import sharding
    w = w or LONG_PREFILL
    lens = w["lens"]
    try:
        head_parts, seq_parts = sharding.unit_grid(w["hkv"], len(lens), world)
    except ValueError:
        return None
    D, G = w["dim"], w["hq"] // w["hkv"]
    qs, ks, seqs = sharding.unit_slices(w["hq"], w["hkv"], len(lens), world, rank)
    groups = range(ks.start, ks.stop)
    my_lens = [lens[i] for i in seqs]
    T, T_all = sum(my_lens), sum(lens)
    if len(set(lens)) != 1:
        return None                               # the gather below wants equal shapes on every rank
    scale = 1.0 if w.get("unit_variance") else D ** -0.5
    per_seq = {"q": [], "k": [], "v": [], "do": []}
    for sq in seqs:                               # data of a (sequence, KV group) does not depend on how many ranks there are
        parts = {"q": [], "k": [], "v": [], "do": []}
        for g in groups:
            gen = torch.Generator(device=dev).manual_seed(500 + g + 64 * sq)
            for name, h, sc in (("q", G, scale), ("k", 1, scale), ("v", 1, scale), ("do", G, 1.0)):
                parts[name].append((torch.randn(lens[sq], h, D, device=dev, generator=gen) * sc).bfloat16())
        for n in parts:
            per_seq[n].append(torch.cat(parts[n], dim=1))
    res = {n: torch.cat(p, dim=0).contiguous() for n, p in per_seq.items()}
    del per_seq, parts
    cu = torch.tensor(np.concatenate(([0], np.cumsum(my_lens))), dtype=torch.int32, device=dev)
    cfg = {"chunk_size": w["chunk"], "topk": w["topk"], "route_precision": "fp32", "stable_routes": True}
    hq_local = G * len(groups)
    gathered = torch.empty(world, T, hq_local, D, dtype=torch.bfloat16, device=dev) if world > 1 else None
    full = torch.empty(T_all, w["hq"], D, dtype=torch.bfloat16, device=dev) if world > 1 else None
    side = torch.cuda.Stream(dev)
    main = torch.cuda.current_stream(dev)

    def gather(out):
        """[T/seq parts, Hq/head parts, D] of every rank (rank = sequence part * head parts + head part) -> [T, Hq, D]
        in token and head order on this rank."""
        dist.all_gather_into_tensor(gathered, out)
        full.view(seq_parts, T, head_parts, hq_local, D).copy_(
            gathered.view(seq_parts, head_parts, T, hq_local, D).permute(0, 2, 1, 3, 4))

    def step(t, overlap=True):
        q, k, v = (t[n].detach().requires_grad_(True) for n in ("q", "k", "v"))
        out = moba_opt.run_impl("opt_gqa_cuda", q, k, v, cu, max(my_lens), cfg)
        if world > 1:
            det = out.detach()
            if overlap:
                side.wait_stream(main)
                with torch.cuda.stream(side):
                    det.record_stream(side)
                    gather(det)
            else:
                gather(det)
        grads = torch.autograd.grad(out, (q, k, v), grad_outputs=t["do"])
        if world > 1 and overlap:
            main.wait_stream(side)
        return (out.detach() if world == 1 else full,) + grads

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, n):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        barrier()
        t = torch.tensor([e0.elapsed_time(e1) / n], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    for _ in range(max(1, warmup)):
        step(res)
    ms = timed(lambda: step(res), steps)
    ga.check_status()
    ms_serial = gather_ms = None
    if world > 1:
        ms_serial = timed(lambda: step(res, overlap=False), steps)      # gather between forward and backward
        probe = res["q"]                                                # same shape and dtype as the forward output
        gather(probe)
        gather_ms = timed(lambda: gather(probe), 5)                    # the collective (and the reorder) alone
    flops = 14.0 * D * attended_pairs(lens, w["chunk"], w["topk"]) * w["hq"]
    out = dict(workload=w["name"], scaling="strong", kv_groups_per_rank=len(groups), sequences_per_rank=len(my_lens),
               steps=steps, ms_per_step=ms,
               tflops=flops / (ms * 1e-3) / 1e12, flops_per_step=flops,
               gather=dict(collective="nccl all_gather_into_tensor of the forward output, on a second stream beside the backward",
                           bytes_received_per_rank=(world - 1) * T * hq_local * D * 2 if world > 1 else 0,
                           ms_alone=gather_ms, ms_per_step_with_gather_in_line=ms_serial))
    if with_host_leg:
        # the same step fed from pinned host memory: this rank's heads only go up (q, k, v, dO) and come back (out of
        # its heads, dq, dk, dv); the gathered output stays on the device
        host = {n: t.cpu().pin_memory() for n, t in res.items()}
        back = {n: torch.empty_like(host[src]) .pin_memory() for n, src in (("out", "q"), ("dq", "q"), ("dk", "k"), ("dv", "k"))}
        dev_in = {n: torch.empty_like(t) for n, t in res.items()}

        def host_step():
            for n, t in host.items():
                dev_in[n].copy_(t, non_blocking=True)
            outs = step(dev_in)
            local = outs[0] if world == 1 else outs[0].view(seq_parts, T, w["hq"], D)[rank // head_parts][:, qs]
            for dst, src in zip(("out", "dq", "dk", "dv"), (local,) + outs[1:]):
                back[dst].copy_(src, non_blocking=True)

        host_step()
        ms_host = timed(host_step, max(2, steps // 2))
        out["e2e"] = dict(ms_per_step=ms_host, tflops=flops / (ms_host * 1e-3) / 1e12,
                          h2d_bytes_per_step_per_rank=sum(t.numel() * 2 for t in host.values()),
                          d2h_bytes_per_step_per_rank=sum(t.numel() * 2 for t in back.values()))
    return out

# ----------------------------------------------------------------------------- full-model leg
FULL_MODEL = dict(name="qwen2_0.5b_random_prompt16384_greedy256_moba12of24_c512_k4", prompt=16384, steps=256, chunk=512, topk=4,
                  page=16, dense_layers=tuple(range(0, 24, 2)))


FULL_MODEL_LONG = dict(FULL_MODEL, name="qwen2_0.5b_random_prompt131072_greedy64_moba12of24_c512_k4", prompt=131072, steps=64)


def run_full_model(dev, w=None):
    """BASELINE configs[4] (and, with w = FULL_MODEL_LONG, the same model on a 131072-token prompt, where a dense layer's
    K/V is 67 MB per step and attention bytes are what a step waits for): random-init Qwen2-0.5B architecture (24 layers, hidden 896, 14/2 heads, D=64, FFN 4864,
    vocab 151936, N(0, 0.02) bf16), 12 of the 24 layers MoBA (the odd ones; chunk 512, topk 4), batch 1, a prompt of
    16384 uniform-random token ids, then 256 greedy steps under one whole-model CUDA graph, beside the all-dense
    session on the same weights and prompt.  Returns prefill and per-step times (CUDA events)."""
    import torch
    sys.path.insert(0, str(ROOT / "moba-merge-cuda_b200" / "examples"))
    from full_qwen2 import FullQwen2Session, random_qwen2
    w = w or FULL_MODEL
    model = random_qwen2(device=dev, max_positions=max(32768, w["prompt"] + w["steps"] + 64))
    ids = torch.randint(0, model.config.vocab_size, (1, w["prompt"]), generator=torch.Generator().manual_seed(0)).to(dev)
    with FullQwen2Session(model, 2048, chunk=w["chunk"], topk=w["topk"], page=w["page"], mode="moba") as s:   # warm-up
        s.prefill(ids[:, :1536])
        s.prepare()
        s.greedy_step()
    res = {}
    for label, kw in (("moba", dict(mode="moba", dense_layers=w["dense_layers"])), ("dense", dict(mode="dense"))):
        with FullQwen2Session(model, w["prompt"] + w["steps"] + 64, chunk=w["chunk"], topk=w["topk"], page=w["page"],
                              backend="model_graph", stable_routes=True, **kw) as s:
            e = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
            e[0].record()
            s.prefill(ids)
            e[1].record()
            s.prepare()
            for _ in range(8):
                s.greedy_step()
            e[2].record()
            tokens = s.generate(w["steps"] - 8)
            e[3].record()
            torch.cuda.synchronize()
            res[label] = dict(prefill_ms=e[0].elapsed_time(e[1]), ms_per_step=e[2].elapsed_time(e[3]) / (w["steps"] - 8),
                              last_token=int(tokens[-1]))
    del model
    torch.cuda.empty_cache()
    return dict(workload=w["name"], moba_layers=12, prompt_tokens=w["prompt"], greedy_steps=w["steps"],
                decode_tokens_per_s=1e3 / res["moba"]["ms_per_step"], decode_ms_per_step=res["moba"]["ms_per_step"],
                prefill_ms=res["moba"]["prefill_ms"], dense_decode_ms_per_step=res["dense"]["ms_per_step"],
                dense_prefill_ms=res["dense"]["prefill_ms"],
                decode_speedup_vs_dense=res["dense"]["ms_per_step"] / res["moba"]["ms_per_step"],
                mode="whole-model CUDA graph, greedy token kept on the device")


def run_full_model_only(args):
    """Profiler runs: the MoBA session of BASELINE configs[4] launch by launch (no graph), prefill and four steps
    outside, `--only-full-model N` greedy steps inside a cudaProfilerStart/Stop range (`ncu --profile-from-start off`)."""
    import torch
    sys.path.insert(0, str(ROOT / "moba-merge-cuda_b200" / "examples"))
    from full_qwen2 import FullQwen2Session, random_qwen2
    w = FULL_MODEL
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    model = random_qwen2(device=dev)
    ids = torch.randint(0, model.config.vocab_size, (1, w["prompt"]), generator=torch.Generator().manual_seed(0)).to(dev)
    with FullQwen2Session(model, w["prompt"] + 64 + args.only_full_model, chunk=w["chunk"], topk=w["topk"], page=w["page"],
                          backend="eager", stable_routes=True, mode="moba", dense_layers=w["dense_layers"]) as s:
        s.prefill(ids)
        s.prepare()
        for _ in range(4):
            s.greedy_step()
        torch.cuda.synchronize()
        e = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
        torch.cuda.profiler.start()
        e[0].record()
        for _ in range(args.only_full_model):
            s.greedy_step()
        e[1].record()
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
    print(json.dumps(dict(full_model_only=True, workload=w["name"], steps=args.only_full_model, backend="eager",
                          ms_per_step=e[0].elapsed_time(e[1]) / args.only_full_model)))


# ----------------------------------------------------------------------------- GPU arm
def run_decode_only(args):
    import torch
    import moba_opt.grouped_attention as ga
    from moba_opt import _ext
    torch.cuda.set_device(0)
    dec = run_decode(torch.device("cuda", 0), 0, 1, args.decode_steps, _ext.lib())
    ga.check_status()
    sec = dec["ms_per_step"] * 1e-3
    print(json.dumps(dict(decode_only=True, workload=DECODE["name"], ms_per_step=dec["ms_per_step"], tokens_per_s=dec["requests"] / sec,
                          hbm_gbs=dec["bytes_per_step"] / sec / 1e9, attend_kernel_ms=dec["attend_ms"],
                          algorithmic_bytes_per_step=dec["bytes_per_step"])))


def bind_to_gpu_numa(local):
    """Best effort: run this rank (and so first-touch its pinned host buffers) on the CPUs of the NUMA node
    the GPU hangs off, so that with several ranks the host copies do not all cross one socket's memory."""
    try:
        import torch
        pr = torch.cuda.get_device_properties(local)
        dev = "%04x:%02x:%02x.0" % (pr.pci_domain_id, pr.pci_bus_id, pr.pci_device_id)
        node = int(open("/sys/bus/pci/devices/%s/numa_node" % dev).read())
        if node < 0:
            return None
        cpus = set()
        for part in open("/sys/devices/system/node/node%d/cpulist" % node).read().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = cpus & os.sched_getaffinity(0)
        if allowed:
            os.sched_setaffinity(0, allowed)
            return node
    except Exception:
        pass
    return None


def probe_host_nodes(dev):
    """When sysfs does not say which NUMA node the GPU hangs off: pin a 64 MB buffer from the CPUs of each node this
    process may run on, time host->device copies from it, and stay on the fastest node while the real host buffers
    are allocated (pinned pages land on the node of the thread that allocates them).  Returns (node, GB/s per node)
    or (None, {}) when there is nothing to choose from."""
    import glob
    import torch
    try:
        before = os.sched_getaffinity(0)
        nodes = {}
        for path in glob.glob("/sys/devices/system/node/node[0-9]*"):
            cpus = set()
            for part in open(path + "/cpulist").read().strip().split(","):
                if part:
                    lo, _, hi = part.partition("-")
                    cpus.update(range(int(lo), int(hi or lo) + 1))
            if cpus & before:
                nodes[int(path.rsplit("node", 1)[1])] = cpus & before
        if len(nodes) < 2:
            return None, {}
        n = 64 << 20
        dst = torch.empty(n, dtype=torch.uint8, device=dev)
        rates = {}
        for node, cpus in sorted(nodes.items()):
            os.sched_setaffinity(0, cpus)
            src = torch.empty(n, dtype=torch.uint8).pin_memory()
            src.fill_(1)
            dst.copy_(src, non_blocking=True)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(4):
                dst.copy_(src, non_blocking=True)
            e1.record()
            torch.cuda.synchronize()
            rates[node] = 4 * n / (e0.elapsed_time(e1) * 1e-3) / 1e9
            del src
        best = max(rates, key=rates.get)
        os.sched_setaffinity(0, nodes[best])
        return best, {k: round(v, 1) for k, v in rates.items()}
    except Exception:
        return None, {}


def run_ours(args):
    import torch
    import torch.distributed as dist
    import moba_opt
    import moba_opt.grouped_attention as ga
    from moba_opt import _ext

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    lib = _ext.lib()  # fails loudly when the CUDA library is missing
    affinity = os.sched_getaffinity(0)
    numa_node, numa_rates = bind_to_gpu_numa(local), {}
    if numa_node is None:
        numa_node, numa_rates = probe_host_nodes(dev)

    w = WORKLOAD
    T, Hq, Hkv, D = sum(w["lens"]), w["hq"], w["hkv"], w["dim"]
    gen = torch.Generator().manual_seed(1000 + rank)
    host = {}
    qkv_scale = 1.0 if w.get("unit_variance") else D ** -0.5
    for name, h, scale in (("q", Hq, qkv_scale), ("k", Hkv, qkv_scale), ("v", Hkv, qkv_scale), ("do", Hq, 1.0)):
        host[name] = (torch.randn(T, h, D, generator=gen) * scale).bfloat16().pin_memory()
    cu = torch.tensor(np.concatenate(([0], np.cumsum(w["lens"]))), dtype=torch.int32, device=dev)
    max_len = max(w["lens"])
    cfg = {"chunk_size": w["chunk"], "topk": w["topk"], "route_precision": "fp32", "stable_routes": True,
           "deterministic_merge": True}
    res = {n: t.to(dev) for n, t in host.items()}
    host_out = {n: torch.empty_like(host[src]).pin_memory() for n, src in (("out", "q"), ("dq", "q"), ("dk", "k"), ("dv", "k"))}
    for t in host_out.values():
        t.zero_()                       # touch the pages from this node before the affinity is widened again
    os.sched_setaffinity(0, affinity)   # the CPU legs use every core

    def step(q, k, v, do):
        q, k, v = (t.detach().requires_grad_(True) for t in (q, k, v))
        out = moba_opt.run_impl("opt_gqa_cuda", q, k, v, cu, max_len, cfg)
        dq, dk, dv = torch.autograd.grad(out, (q, k, v), grad_outputs=do)
        return out.detach(), dq, dk, dv

    # End-to-end leg: every step's q, k, v, dO come from pinned host memory and its out, dq, dk, dv go back
    # to pinned host memory, all inside the timed region.  As in a real input pipeline the copies run on
    # their own streams, double-buffered: step i+1's inputs arrive and step i-1's results leave while
    # step i computes.
    copy_in, copy_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    dev_in = [{n: torch.empty_like(t, device=dev) for n, t in host.items()} for _ in range(2)]

    def run_e2e(steps):
        main = torch.cuda.current_stream(dev)
        arrived = [torch.cuda.Event(), torch.cuda.Event()]
        consumed = [torch.cuda.Event(), torch.cuda.Event()]

        def fetch(i):
            buf = i % 2
            with torch.cuda.stream(copy_in):
                if i >= 2:
                    copy_in.wait_event(consumed[buf])
                for n, t in host.items():
                    dev_in[buf][n].copy_(t, non_blocking=True)
                arrived[buf].record(copy_in)

        copy_in.wait_stream(main)
        copy_out.wait_stream(main)
        fetch(0)
        for i in range(steps):
            buf = i % 2
            if i + 1 < steps:
                fetch(i + 1)
            main.wait_event(arrived[buf])
            outs = step(dev_in[buf]["q"], dev_in[buf]["k"], dev_in[buf]["v"], dev_in[buf]["do"])
            consumed[buf].record(main)
            copy_out.wait_event(consumed[buf])
            with torch.cuda.stream(copy_out):
                for dst, src in zip(("out", "dq", "dk", "dv"), outs):
                    src.record_stream(copy_out)
                    host_out[dst].copy_(src, non_blocking=True)
        main.wait_stream(copy_out)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, warmup, hooks=None):
        for _ in range(warmup):
            fn()
        barrier()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for i in range(steps):
            if hooks:
                hooks(i)
            fn()
        stop.record()
        barrier()
        ms = start.elapsed_time(stop)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    # events around the backward main kernel of every timed step
    pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    for a, b in pairs:
        a.record(); b.record()  # materialise the handles

    def hook(i):
        lib.moba_profile_events(3, pairs[i][0].cuda_event, pairs[i][1].cuda_event)

    sampler = ClockSampler(local)
    sampler.start()
    ms_total = timed(lambda: step(res["q"], res["k"], res["v"], res["do"]), args.steps, max(args.warmup, 3), hook)
    clocks = sampler.stop()
    lib.moba_profile_events(3, None, None)
    ga.check_status()
    bwd_ms = float(np.mean([a.elapsed_time(b) for a, b in pairs]))
    e2e_steps = max(4, args.steps)
    ms_e2e = None
    if not args.kernels_only:
        run_e2e(2)
        ms_e2e = timed(lambda: run_e2e(e2e_steps), 1, 0)
    ga.check_status()

    dec = None
    if not args.kernels_only and not args.no_decode:
        dec = run_decode(dev, rank, world, args.decode_steps, lib)
        ga.check_status()
        dec["per_rank"] = [dict(requests=dec["requests"], context_tokens=dec["context_tokens"], ms_per_step=dec["ms_per_step"],
                                host_ms_per_step=dec["host_ms_per_step"])]
        if world > 1:
            mine = torch.tensor([dec["ms_per_step"], dec["attend_ms"], dec["gather_ms_per_step"], dec["bytes_per_step"],
                                 float(dec["requests"]), float(dec["context_tokens"]), dec["host_ms_per_step"]], device=dev, dtype=torch.float64)
            every = torch.empty(world, mine.numel(), device=dev, dtype=torch.float64)
            dist.all_gather_into_tensor(every, mine)
            every = every.cpu().numpy()
            dec.update(ms_per_step=float(every[:, 0].max()), attend_ms=float(every[:, 1].max()),
                       gather_ms_per_step=float(every[:, 2].max()), bytes_per_step=float(every[:, 3].sum()),
                       requests=int(every[:, 4].sum()),
                       per_rank=[dict(requests=int(r[4]), context_tokens=int(r[5]), ms_per_step=float(r[0]),
                                      host_ms_per_step=float(r[6])) for r in every])
            # the same 64 requests on EVERY rank (independent replicas of the whole decode configuration): what the ranks
            # deliver when each has a full batch, beside the split above where each has an eighth of one
            full = run_decode(dev, 0, 1, args.decode_steps, lib)
            ga.check_status()
            slowest = torch.tensor([full["ms_per_step"]], device=dev, dtype=torch.float64)
            dist.all_reduce(slowest, op=dist.ReduceOp.MAX)
            dec["replicated"] = dict(requests_per_rank=full["requests"], ms_per_step=float(slowest.item()),
                                     tokens_per_s=world * full["requests"] / (float(slowest.item()) * 1e-3), scaling="weak")

    long_leg = None
    if not args.kernels_only and not args.no_long_prefill:
        long_leg = run_long_prefill(dev, rank, world, args.long_steps, 2)
        ga.check_status()
    split_leg = None
    if world > 1 and not args.kernels_only and not args.no_long_prefill and WORKLOAD is WORKLOADS["cfg2"]:
        split_leg = run_long_prefill(dev, rank, world, max(args.long_steps, 8), 3, w=HEADLINE_SPLIT)   # the headline config as one job
        ga.check_status()

    flops = step_flops(w)
    value = world * flops / (ms_total / args.steps * 1e-3) / 1e12
    e2e_value = None if ms_e2e is None else world * flops / (ms_e2e / e2e_steps * 1e-3) / 1e12
    h2d = sum(t.numel() * 2 for t in host.values())
    d2h = sum(t.numel() * 2 for t in host_out.values())
    if rank == 0:
        pk = peaks()
        bwd_flops = flops * 10.0 / 14.0
        achieved = bwd_flops / (bwd_ms * 1e-3) / 1e12
        cpu_val, cpu_desc, cpu_dt, cpu_kind = (cpu_sample(os.cpu_count() or 1) if world == 1 and not args.kernels_only
                                               else (None, None, None, None))
        bwd_sources = (("prefill_attn_bwd_ws.cu", "prefill_bwd.cuh", "prefill_common.cuh", "sm100.cuh") if D <= 64 else
                       ("prefill_attn_bwd_ws128.cu", "prefill_bwd.cuh", "prefill_common.cuh", "sm100.cuh"))
        bwd_kernel = "attn_bwd_ws_kernel" if D <= 64 else "attn_bwd_ws128_kernel"
        traffic, traffic_source = (measured_traffic(bwd_kernel, bwd_sources, len(w["lens"])) if w["lens"][0] == 32768 and D == 64
                                   else (None, "no profiled figure for this workload"))
        line = dict(metric=METRIC, value=value, unit=UNIT, n_gpus=world, steps=args.steps, warmup=max(args.warmup, 3),
                    ms_per_step=ms_total / args.steps, higher_is_better=True, scaling="weak", vs_baseline=None,
                    dtype="bf16", data="synthetic",
                    config=dict(workload=w["name"], sequences=len(w["lens"]), seq_len=w["lens"][0], hq=Hq, hkv=Hkv,
                                head_dim=D, chunk=w["chunk"], topk=w["topk"],
                                per_rank="one full batch per GPU, no collective (the split by KV-head group with its "
                                         "output gather is the long_prefill leg, the split by request the decode leg)",
                                l2="inputs (q, k, v, dO, out: %.2f GB per step) exceed the 126 MB L2, no flush needed" % (T * (3 * Hq + 2 * Hkv) * D * 2 / 1e9)),
                    clocks=clocks,
                    e2e=dict(value=e2e_value, unit=UNIT, h2d_bytes_per_step=h2d, d2h_bytes_per_step=d2h,
                             ms_per_step=None if ms_e2e is None else ms_e2e / e2e_steps, steps=e2e_steps,
                             mode="host copies on their own streams, double-buffered across steps", numa_node=numa_node,
                             numa_h2d_gbs=numa_rates),
                    gpu_launches=13 * args.steps,  # route 5, pack 2, forward 2, backward 4 (memsets not counted)
                    roofline=dict(bound="tensor", kernel=bwd_kernel, achieved=achieved, peak=pk["tflops"],
                                  unit="TFLOP/s", frac=achieved / pk["tflops"], peak_source=pk["source"] + " (sustained bf16)",
                                  traffic=traffic, traffic_source=traffic_source,
                                  ms_per_launch=bwd_ms, flops_per_launch=bwd_flops))
        if dec is not None:
            sec = dec["ms_per_step"] * 1e-3
            line["decode"] = dict(workload=DECODE["name"], requests=dec["requests"], steps=args.decode_steps,
                                  tokens_per_s=dec["requests"] / sec, ms_per_step=dec["ms_per_step"],
                                  algorithmic_bytes_per_step=dec["bytes_per_step"], hbm_gbs=dec["bytes_per_step"] / sec / 1e9,
                                  frac_of_hbm_peak=dec["bytes_per_step"] / sec / 1e9 / pk["hbm"] / world, hbm_peak=pk["hbm"],
                                  attend_kernel_ms=dec["attend_ms"],
                                  attend_kernel_gbs=dec["bytes_per_step"] / (dec["attend_ms"] * 1e-3) / 1e9,
                                  mode="prepare_decode + CUDA graph, one token per request per step",
                                  placement="requests spread over the ranks by expected bytes per step, largest first",
                                  per_rank=dec["per_rank"],
                                  ms_per_step_with_output_gather=dec["gather_ms_per_step"])
            if "replicated" in dec:
                line["decode"]["replicated"] = dec["replicated"]
            line["decode"]["scaling"] = "strong"
            if world == 1 and not args.kernels_only:
                line["decode"]["cpu_baseline"] = cpu_decode_sample(os.cpu_count() or 1)
                try:
                    line["decode"]["reference_gpu"] = run_decode_against_reference(dev)
                except Exception as exc:      # the reference's Triton kernels are outside this package's control
                    line["decode"]["reference_gpu"] = {"error": "%s: %s" % (type(exc).__name__, exc)}
        if long_leg is not None:
            long_leg["frac_of_tensor_peak"] = long_leg["tflops"] / world / pk["tflops"]
            line["long_prefill"] = long_leg
        if split_leg is not None:
            split_leg["frac_of_tensor_peak"] = split_leg["tflops"] / world / pk["tflops"]
            line["headline_split"] = split_leg
        if world == 1 and not args.kernels_only and not args.no_full_model:
            try:
                line["full_model"] = run_full_model(dev)
                line["full_model_long"] = run_full_model(dev, FULL_MODEL_LONG)
            except Exception as exc:  # the optional leg must not take the line with it
                line.setdefault("full_model", {"error": "%s: %s" % (type(exc).__name__, exc)})
                if "error" not in line["full_model"]:
                    line["full_model_long"] = {"error": "%s: %s" % (type(exc).__name__, exc)}
        if cpu_val is not None:
            line["cpu_baseline"] = dict(value=cpu_val, unit=UNIT, cores=os.cpu_count() or 1, kind=cpu_kind, sample=cpu_desc,
                                        seconds=cpu_dt)
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg2", choices=sorted(WORKLOADS))
    ap.add_argument("--no-decode", action="store_true", help="skip the paged-decode leg")
    ap.add_argument("--no-full-model", action="store_true", help="skip the full-model decode leg")
    ap.add_argument("--no-long-prefill", action="store_true", help="skip the long-prefill leg (split by KV-head group)")
    ap.add_argument("--long-steps", type=int, default=4, help="timed steps of the long-prefill leg")
    ap.add_argument("--only-decode", action="store_true", help="run only the paged-decode leg (profiler runs)")
    ap.add_argument("--only-full-model", type=int, default=0, metavar="N",
                    help="run only N launch-by-launch decode steps of the full-model session (profiler runs)")
    ap.add_argument("--decode-steps", type=int, default=DECODE["steps"])
    ap.add_argument("--kernels-only", action="store_true", help="skip the host-buffer and CPU legs (profiler runs)")
    args = ap.parse_args()
    global WORKLOAD
    WORKLOAD = WORKLOADS[args.workload]
    if args.impl == "reference":
        run_reference(args)
    elif args.only_decode:
        run_decode_only(args)
    elif args.only_full_model:
        run_full_model_only(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
