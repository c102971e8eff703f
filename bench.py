#!/usr/bin/env python
"""Benchmark of the USP attention hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload flux|wan] [--impl ours|reference]

One *step* is the attention work of one DiT denoising step: one ``USP`` call per transformer
layer (Wan2.1-14B 720p: 40 layers of 40 heads x 128 over 75,600 tokens; Flux.1-dev 1024x1024:
57 layers of 24 heads x 128 over 4608 tokens) on synthetic q/k/v (N(0,1), seeded).  Consecutive
layers use different input sets whose total size (several GB) never fits in L2.  The default
workload is the 75.6 K-token video case, the one the scaling target is stated on; the Flux
numbers ride along in the same JSON line (and ``--workload flux`` swaps the roles).  ``value`` is
algorithmic TFLOP/s (4*Sq*Sk*H*D per call) over all GPUs with inputs resident in HBM; ``e2e``
is the same metric through ``xdit_b200.USP`` with the step's inputs in pinned host memory and
the results read back, copies inside the timed region.

Before anything is timed, every rank runs one ``USP`` call of each workload and compares sampled
rows of its result with the oracle's dense attention over the regenerated global tensors; the line
carries ``parity`` and the process exits non-zero when a row is outside max-abs 2e-2 / cosine
0.9999.

N > 1 is launched by ``torch.distributed.run`` (one rank per GPU, NCCL); the sequence is sharded
over N ranks (strong scaling) with Ulysses degree N, which is the fastest split behind NVSwitch;
``--sp ULYSSESxRING`` selects another split, e.g. ``--sp 2x4`` for Ulysses 2 x ring 4, the split the
Wan2.1 workload is usually quoted with.  Ring splits are also measured (and checked) as legs under
``extra``, with the K/V rotation by copy-engine transfers into the next rank's buffer and over NCCL
send/recv; the Ulysses exchange runs by stores into the peers' memory (``--exchange peer``, the default,
kept only if a probing call succeeds on every rank) with the NCCL form as a leg.

``--impl reference`` times the reference's own ``USP()`` (its unmodified Python, taken from
``oracle/_ref``) on the host cores of rank 0, on a bounded sample of the same workload; without
those sources it times the oracle's restatement instead and says so (``kind``).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: layers, heads, head_dim, tokens
    "flux": dict(desc="Flux.1-dev 1024x1024 MMDiT self-attention: 57 layers x (24 heads x 128, 512 text + 4096 image tokens)",
                 layers=57, sets=57, H=24, D=128, S=4608),
    "wan": dict(desc="Wan2.1-14B 81f 720x1280 self-attention: 40 layers x (40 heads x 128, 75,600 tokens)",
                layers=40, sets=2, H=40, D=128, S=75600),
    # legs reported under `extra`
    "hunyuan": dict(desc="HunyuanVideo 129f 720p self-attention: 24 heads x 128, 256 text + 118,800 image tokens, "
                         "text sharded with the image",
                    layers=60, sets=1, H=24, D=128, S=119056),
}
TOL_MAX_ABS, TOL_COS = 2e-2, 0.9999


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return (float(p["bf16_tflops"]), float(p.get("bf16_tflops_sustained", p["bf16_tflops"])),
                float(p["hbm_gbs"]), "measured")
    return 1590.0, 1400.0, 6650.0, "fallback"


def roofline(w, res, per_gpu_tf, kernel_ms, world, tf_burst, tf_sustained, peak_kind):
    """Roofline entry of the attention kernel.

    Denominator: the cuBLAS bf16 figure measured as a seconds-long loop under the power cap when the
    timed region itself is such a loop (back-to-back launches for longer than a second), the burst
    figure otherwise; the fraction against the other one rides along.  `traffic` is DRAM bytes per
    launch scaled from an ncu capture of one Flux layer of the same kernel: 85.2 MB read for 84.9 MB of
    q/k/v (every input byte fetched once, K/V re-reads served by L2) and at most the output bytes
    written, both proportional to the tensors' sizes.
    """
    long_loop = res["ms_per_step"] * max(1, res.get("steps", 1)) >= 1000.0
    peak = tf_sustained if long_loop else tf_burst
    in_bytes = 3 * w["H"] * w["S"] * w["D"] * 2 / world
    out_bytes = w["H"] * w["S"] * w["D"] * 2 / world
    return {
        "kernel": "attn_fwd_sm100_kernel", "bound": "tensor", "achieved": per_gpu_tf, "peak": peak,
        "unit": "TFLOP/s", "frac": per_gpu_tf / peak,
        "peak_kind": f"of {peak_kind} (cuBLAS bf16, " + ("sustained loop under the power cap: the timed region is "
                     "seconds of back-to-back launches)" if long_loop else "burst)"),
        "frac_of_burst": per_gpu_tf / tf_burst, "peak_burst": tf_burst,
        "frac_of_sustained": per_gpu_tf / tf_sustained, "peak_sustained": tf_sustained,
        "avg_call_ms": kernel_ms,
        "traffic": 1.004 * in_bytes + out_bytes,
        "traffic_kind": "bytes per launch, scaled by tensor bytes from the ncu capture of one Flux layer",
        "algorithmic_bytes": in_bytes + out_bytes,
    }


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while a region runs."""

    def __init__(self, index: int):
        self.index = index
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4),
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for k, bit in names.items():
                    if mask & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            time.sleep(0.005)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(1.0)

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": 0}
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2], "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}


def bind_to_gpu_numa_node(index: int) -> bool:
    """Run this rank on the cores next to its GPU (the affinity NVML reports), so that the pinned host
    buffers of the end-to-end leg are first touched on that memory node.  A setting of this process
    only; returns whether it could be applied."""
    try:
        import pynvml

        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(index)
        words = ((os.cpu_count() or 64) + 63) // 64
        mask = pynvml.nvmlDeviceGetCpuAffinity(h, words)
        cpus = {64 * i + b for i, word in enumerate(mask) for b in range(64) if (word >> b) & 1}
        cpus &= os.sched_getaffinity(0)
        if cpus:
            os.sched_setaffinity(0, cpus)
            return True
    except Exception:
        pass
    return False


def flops_per_call(w):
    return 4.0 * w["S"] * w["S"] * w["H"] * w["D"]


# --------------------------------------------------------------------------------------------
# reference arm and CPU baseline: the reference's own USP() on the host cores
# --------------------------------------------------------------------------------------------
def _reference_usp_callable():
    """(callable(q, k, v) -> out, kind).  The reference's own ``USP`` at sequence-parallel degree 1
    (``usp.py:316-323``: its ``SDPA`` back-end body, no collectives) when its sources are under
    ``oracle/_ref``; otherwise the oracle's restatement of that call."""
    from oracle import ref_import

    if ref_import.root() is not None:
        try:
            usp, backend, _cache, _rts = ref_import.import_usp()
            ref_import.configure_usp(usp, backend, 1, 1, 0, None, None)
            return usp.USP, "reference"
        except Exception as e:  # noqa: BLE001
            sys.stderr.write(f"bench: the reference's sources under oracle/_ref did not import ({e!r}); timing the port\n")
    from oracle import usp_oracle as O

    return O.attention_dense_torch_cpu, "port"


def _config1_gloo_worker(rank, world, port, threads, q):
    """Two gloo ranks running the reference's ``USP`` on the Flux-shaped fp32 joint case: Ulysses 2,
    24 heads x 128, 4096 image tokens sharded + 512 text tokens replicated (joint, rear), N(0,1) from
    seed 0.  One warm-up and five timed calls, each followed by a barrier; rank 0 reports the median."""
    import torch
    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(threads)
    from oracle import ref_import

    usp, backend, _cache, _rts = ref_import.import_usp()
    pg = dist.new_group(list(range(world)), backend="gloo")
    ref_import.configure_usp(usp, backend, world, 1, rank, pg, None)
    g = torch.Generator().manual_seed(0)
    B, H, D, S, Sj = 1, 24, 128, 4096, 512
    qg, kg, vg = (torch.randn(B, H, S, D, generator=g) for _ in range(3))
    jq, jk, jv = (torch.randn(B, H, Sj, D, generator=g) for _ in range(3))
    sh = lambda t: t.chunk(world, dim=2)[rank].contiguous()
    ql, kl, vl = sh(qg), sh(kg), sh(vg)
    ts = []
    for it in range(6):
        dist.barrier()
        t0 = time.perf_counter()
        out = usp.USP(ql, kl, vl, joint_query=jq, joint_key=jk, joint_value=jv, joint_strategy="rear")
        dist.barrier()
        if it:
            ts.append(time.perf_counter() - t0)
    if rank == 0:
        ts.sort()
        # parity of what was timed: rank 0's rows against dense attention over all keys
        import torch.nn.functional as F

        dense = F.scaled_dot_product_attention(torch.cat([ql, jq], 2), torch.cat([kg, jk], 2), torch.cat([vg, jv], 2))
        q.put({"median_s": ts[len(ts) // 2], "calls": len(ts), "max_abs_vs_dense": float((out - dense).abs().max())})
    dist.destroy_process_group()


def reference_config1_gloo(cores):
    """The reference's ``USP`` under 2 gloo ranks on the host cores (threads = cores / 2 each)."""
    from oracle import ref_import

    if ref_import.root() is None:
        return {"unavailable": "the reference's sources are not under oracle/_ref"}
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    threads = max(1, cores // 2)
    port = 29400 + os.getpid() % 500
    procs = [ctx.Process(target=_config1_gloo_worker, args=(r, 2, port, threads, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
    for p in procs:
        if p.is_alive():
            p.terminate()
    if q.empty() or any(p.exitcode != 0 for p in procs):
        return {"unavailable": "the 2-rank gloo run did not finish"}
    r = q.get()
    fl = 4.0 * (4096 + 512) * (4096 + 512) * 24 * 128  # text rows counted once
    return {"tflops": fl / r["median_s"] / 1e12, "median_ms": r["median_s"] * 1e3, "calls": r["calls"],
            "ranks": 2, "threads_per_rank": threads, "cores": cores, "dtype": "f32",
            "max_abs_vs_dense": r["max_abs_vs_dense"],
            "what": "reference USP(), Ulysses 2 over gloo, 24 x 128, 4096 image + 512 joint text tokens (rear), "
                    "1 warm-up + 5 timed calls, median"}


def host_sample(w, budget_s, steps, warmup):
    """Time the reference's CPU path on a bounded sample (a number of heads of one layer) of workload
    ``w``; returns (TFLOP/s, ms per step, description, kind, cores)."""
    import torch

    fn, kind = _reference_usp_callable()
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    S, D = w["S"], w["D"]
    g = torch.Generator().manual_seed(0)

    def make(heads):
        return tuple(torch.randn(1, heads, S, D, generator=g) for _ in range(3))

    def one(qkv):
        t0 = time.perf_counter()
        fn(*qkv)
        return time.perf_counter() - t0

    t_head = one(make(1))
    per_step = budget_s / max(1, steps + warmup)
    heads = int(max(1, min(w["H"], per_step / max(t_head, 1e-3))))
    qkv = make(heads)  # one input set, larger than any CPU cache (heads x S x 128 fp32 x 3)
    for _ in range(warmup):
        one(qkv)
    total = 0.0
    for _ in range(steps):
        total += one(qkv)
    fl = 4.0 * S * S * heads * D
    name = "the reference's USP() at sequence-parallel degree 1 (its SDPA back-end)" if kind == "reference" \
        else "the oracle's restatement of the reference's SDPA back-end"
    sample = (f"{heads} of {w['H']} heads of one layer, {S} tokens, fp32, {name} on {cores} threads, per step")
    return fl * steps / total / 1e12, total / steps * 1e3, sample, kind, cores


def run_reference(args, w, name):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    val, ms, sample, kind, cores = host_sample(w, 90.0, args.steps, args.warmup)
    line = {
        "impl": "reference", "metric": "usp_attn_tflops", "value": val, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": name, "desc": w["desc"]},
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "extra": {"flux_joint_fp32_ulysses2_gloo": reference_config1_gloo(cores)},
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------------
# our arm
# --------------------------------------------------------------------------------------------
def global_head(torch, device, set_idx, tensor_idx, head, S, D, rows=None):
    """N(0,1) rows of one head of a *global* tensor, drawn on the device from a seed that depends only
    on (input set, tensor, head): every rank can regenerate any head, which is what lets each rank
    check its own output rows against dense attention over all keys.  bf16 [S, D] (or the row range)."""
    g = torch.Generator(device=device)
    g.manual_seed(1000003 * (set_idx + 1) + 10007 * tensor_idx + head)
    t = torch.randn(S, D, generator=g, dtype=torch.float32, device=device).to(torch.bfloat16)
    return t if rows is None else t[rows[0]:rows[1]]


def make_layer_inputs(torch, w, P, rank, sets, device, pinned=False):
    """``sets`` distinct input sets of local shards [1, H, S/P, D] bf16 (a step cycles through them
    layer by layer); rank r holds rows [r*S/P, (r+1)*S/P) of the global tensors."""
    S, H, D = w["S"], w["H"], w["D"]
    s = S // P
    out = []
    for si in range(sets):
        qkv = []
        for i in range(3):
            t = torch.empty(1, H, s, D, dtype=torch.bfloat16, device=device)
            for h in range(H):
                t[0, h].copy_(global_head(torch, device, si, i, h, S, D, (rank * s, (rank + 1) * s)))
            if pinned:
                t = t.cpu().pin_memory()
            qkv.append(t)
        out.append(tuple(qkv))
    return out


def parity_check(torch, dist, out, w, P, rank, device, multi, set_idx=0):
    """Sampled rows (first / middle / last 64 of this rank's shard, first and last head) of ``out``
    [1,H,s,D] against the oracle's dense attention in float64 over the regenerated global K and V."""
    import numpy as np

    from oracle import usp_oracle as O

    S, H, D = w["S"], w["H"], w["D"]
    s = S // P
    n = min(64, s)
    rows = sorted(set(list(range(n)) + list(range(s // 2 - n // 2, s // 2 - n // 2 + n)) + list(range(s - n, s))))
    heads = sorted({0, H - 1})
    idx = torch.tensor(rows, device=device)
    f64 = lambda t: t.float().cpu().double().numpy()
    max_abs, cos_min = 0.0, 1.0
    for h in heads:
        q = global_head(torch, device, set_idx, 0, h, S, D, (rank * s, (rank + 1) * s))[idx]
        k = global_head(torch, device, set_idx, 1, h, S, D)
        v = global_head(torch, device, set_idx, 2, h, S, D)
        want, _ = O.attention_dense(f64(q)[None, None], f64(k)[None, None], f64(v)[None, None])
        got = f64(out[0, h][idx])
        want = want[0, 0]
        max_abs = max(max_abs, float(np.abs(got - want).max()))
        cos_min = min(cos_min, float((got * want).sum() / (np.linalg.norm(got) * np.linalg.norm(want) + 1e-30)))
    finite = bool(torch.isfinite(out.float()).all().item())
    nrows = len(rows) * len(heads)
    if multi:
        t = torch.tensor([max_abs, -cos_min, 0.0 if finite else 1.0], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        max_abs, cos_min, finite = float(t[0]), -float(t[1]), float(t[2]) == 0.0
        nrows *= dist.get_world_size()
    ok = finite and max_abs <= TOL_MAX_ABS and cos_min >= TOL_COS
    return {"max_abs": max_abs, "cos": cos_min, "rows": nrows, "heads": heads, "finite": finite, "ok": ok,
            "against": "oracle dense attention (float64) over the regenerated global q/k/v",
            "tolerance": {"max_abs": TOL_MAX_ABS, "cos": TOL_COS}}


def timed_region(torch, dist, fn, steps, warmup, device, multi):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize(device)
    if multi:
        dist.barrier()
    torch.cuda.synchronize(device)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(steps):
        fn()
    ev1.record()
    torch.cuda.synchronize(device)
    if multi:
        dist.barrier()
    ms = ev0.elapsed_time(ev1)
    if multi:
        t = torch.tensor([ms], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms


def choose_exchange(torch, dist, xdit_b200, ops, inputs, device, want):
    """Which form of the Ulysses exchange a leg uses.  ``want`` = "peer": direct stores into the peers'
    buffers (xdit_b200.peer_exchange), kept only if one probing call succeeds on EVERY rank (the ranks agree
    through an all-reduce, so they never take different paths); otherwise NCCL (pipelined by head groups for
    large shards).  Returns (name, note)."""
    from xdit_b200 import peer_exchange

    if want != "peer":
        peer_exchange.enable(False)
        return "nccl", None
    ok, note = 1.0, None
    try:
        peer_exchange.enable(True)
        xdit_b200.USP(*inputs[0])
        torch.cuda.synchronize(device)
        ops.check_status()
    except Exception as e:  # noqa: BLE001
        ok, note = 0.0, repr(e)[:200]
        try:
            torch.cuda.synchronize(device)
            ops.clear_status()
        except Exception:  # noqa: BLE001
            pass
    t = torch.tensor([ok], dtype=torch.float32, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    if float(t.item()) < 1.0:
        peer_exchange.enable(False)
        return "nccl", note or "the probing call failed on another rank"
    return "peer_stores", None


def run_workload(torch, dist, xdit_b200, ops, name, w, args, device, rank, world, layers, with_e2e, U, R,
                 exchange="nccl"):
    xdit_b200.init_sequence_parallel(U, R)
    P = U * R
    S = w["S"]
    assert P == world and S % P == 0
    nsets = max(1, min(layers, w["sets"]))
    inputs = make_layer_inputs(torch, w, P, rank, nsets, device)
    multi = world > 1
    exchange_note = None
    if multi:
        exchange, exchange_note = choose_exchange(torch, dist, xdit_b200, ops, inputs, device, exchange)
        if exchange == "peer_stores" and R > 1:
            # ring legs: the K/V rotation by copy-engine transfers into the next rank's buffer; a Ulysses
            # part in front of the ring (U > 1) stays on NCCL
            exchange = "peer_copies"
    else:
        exchange = "none"

    # correctness first: one call, sampled rows against the oracle
    out = xdit_b200.USP(*inputs[0])
    torch.cuda.synchronize(device)
    ops.check_status()
    parity = parity_check(torch, dist, out, w, P, rank, device, multi)
    del out

    def step_eager():
        for layer in range(layers):
            q, k, v = inputs[layer % nsets]
            xdit_b200.USP(q, k, v)

    step = step_eager
    graphed = False
    per_step_launches = None
    if args.graph == "on" or (args.graph == "auto" and multi):
        # launch-bound for small shards: replay the whole step as one CUDA graph
        from xdit_b200.graph import GraphedStep

        n_before = ops.launch_count
        gs = GraphedStep(step_eager, warmup=2)
        per_step_launches = (ops.launch_count - n_before) // 3  # 2 warm-up runs + the captured one
        step = gs.replay
        graphed = True

    n0 = ops.launch_count
    sampler = ClockSampler(device.index)
    with sampler:
        ms = timed_region(torch, dist, step, args.steps, args.warmup, device, multi)
    launches = (ops.launch_count - n0) * args.steps // (args.steps + args.warmup)
    if graphed:
        launches = per_step_launches * args.steps  # replayed from the graph, counted at capture time
    ops.check_status()
    fl_step = flops_per_call(w) * layers
    res = {
        "ms_per_step": ms / args.steps,
        "tflops": fl_step * args.steps / (ms * 1e-3) / 1e12,
        "launches": launches,
        "clocks": sampler.summary(),
        "U": U, "R": R, "layers": layers, "cuda_graph": graphed, "sets": nsets, "steps": args.steps,
        "parity": parity, "exchange": exchange,
    }
    if exchange_note:
        res["exchange_note"] = exchange_note
    if with_e2e:
        host = make_layer_inputs(torch, w, P, rank, nsets, device, pinned=True)
        s = S // P
        host_out = [torch.empty(1, w["H"], s, w["D"], dtype=torch.bfloat16).pin_memory() for _ in range(nsets)]

        # The way a serving loop stages a layer's tensors: three device slots, the next layers' q/k/v
        # copied in on one side stream while this layer's USP call runs, the result copied out on
        # another.  Every byte still crosses PCIe inside the timed region, every step.
        NSLOT = 3
        cur = torch.cuda.current_stream(device)
        s_in, s_out = torch.cuda.Stream(device), torch.cuda.Stream(device)
        slots = [[torch.empty(1, w["H"], s, w["D"], dtype=torch.bfloat16, device=device) for _ in range(3)]
                 for _ in range(NSLOT)]
        ev_in = [torch.cuda.Event() for _ in range(NSLOT)]
        ev_done = [torch.cuda.Event() for _ in range(NSLOT)]

        def stage(layer):
            slot = layer % NSLOT
            s_in.wait_event(ev_done[slot])  # the call that last read this slot has finished
            with torch.cuda.stream(s_in):
                for dst, src in zip(slots[slot], host[layer % nsets]):
                    dst.copy_(src, non_blocking=True)
                ev_in[slot].record(s_in)

        def step_e2e():
            for e in ev_done:
                e.record(cur)
            for layer in range(min(NSLOT - 1, layers)):
                stage(layer)
            for layer in range(layers):
                slot = layer % NSLOT
                if layer + NSLOT - 1 < layers:
                    stage(layer + NSLOT - 1)
                cur.wait_event(ev_in[slot])
                out = xdit_b200.USP(*slots[slot])
                ev_done[slot].record(cur)
                s_out.wait_event(ev_done[slot])
                with torch.cuda.stream(s_out):
                    host_out[layer % nsets].copy_(out, non_blocking=True)
                out.record_stream(s_out)
            cur.wait_stream(s_out)  # the step ends when its last result is in host memory

        e2e_steps = max(1, min(args.steps, 5))
        ms_e = timed_region(torch, dist, step_e2e, e2e_steps, 1, device, multi)
        ops.check_status()
        bytes_in = 3 * layers * w["H"] * s * w["D"] * 2
        bytes_out = layers * w["H"] * s * w["D"] * 2
        res["e2e"] = {"value": fl_step * e2e_steps / (ms_e * 1e-3) / 1e12, "unit": "TFLOP/s",
                      "h2d_bytes_per_step": bytes_in, "d2h_bytes_per_step": bytes_out,
                      "ms_per_step": ms_e / e2e_steps, "steps": e2e_steps, "warmup": 1,
                      "host_gbs_per_rank": (bytes_in + bytes_out) / (ms_e / e2e_steps * 1e-3) / 1e9}
        del host, host_out, slots
    del inputs
    if exchange in ("peer_stores", "peer_copies"):
        from xdit_b200 import peer_exchange

        peer_exchange.enable(False)
        peer_exchange.close_all()  # every rank gets here: the groups of this leg are not used again
    torch.cuda.empty_cache()
    return res


def leg(torch, dist, xdit_b200, ops, name, w, args, device, rank, world, layers, U, R, tf_peak, steps=3,
        exchange="nccl"):
    """A secondary measurement (another workload or another split): same timing rules, same parity
    check, a few layers or steps, no end-to-end part.  Never takes the main line down."""
    try:
        a2 = argparse.Namespace(steps=max(1, min(args.steps, steps)), warmup=3, graph=args.graph)
        r = run_workload(torch, dist, xdit_b200, ops, name, w, a2, device, rank, world, layers, False, U, R,
                         exchange=exchange)
        P = U * R
        out = {
            "desc": w["desc"], "layers_timed": layers, "ulysses": U, "ring": R, "cuda_graph": r["cuda_graph"],
            "exchange": r["exchange"],
            "tflops_all_gpus": r["tflops"], "tflops_per_gpu": r["tflops"] / world,
            "ms_per_layer_call": r["ms_per_step"] / layers,
            "frac_of_measured_bf16_burst_peak": r["tflops"] / world / tf_peak,
            "parity": r["parity"],
        }
        if P > 1:
            out["nvlink"] = nvlink_bytes(w, U, R)
        return out, r["parity"]["ok"]
    except Exception as e:  # noqa: BLE001
        import traceback

        # a leg that could not run is reported as such; only a result that was computed and is wrong makes
        # the process exit non-zero
        try:
            from xdit_b200 import peer_exchange

            peer_exchange.enable(False)
            ops.clear_status()
        except Exception:  # noqa: BLE001
            pass
        return {"error": repr(e)[:300], "trace": traceback.format_exc()[-600:]}, True


def nvlink_bytes(w, U, R):
    """Algorithmic bytes one rank sends per attention call: the Ulysses exchanges move (U-1)/U of q, k,
    v and of the output; the ring sends the local K/V shard R-1 times.  ``floor_ms`` is that volume at
    the nominal 900 GB/s per direction."""
    P = U * R
    n = w["H"] * (w["S"] // P) * w["D"] * 2  # bytes of one local tensor
    uly = 4 * n * (U - 1) / U if U > 1 else 0.0
    ring = (R - 1) * 2 * (w["H"] // U) * (w["S"] // R) * w["D"] * 2 if R > 1 else 0.0
    return {"ulysses_bytes_per_call": uly, "ring_bytes_per_call": ring,
            "floor_ms_at_900GBs": (uly + ring) / 900e9 * 1e3}


def hbm_kernels(torch, ops, device, hbm_peak, peak_kind):
    """Achieved HBM GB/s (algorithmic bytes = read + write of the moved rows) of the HBM-bound
    kernels at the shapes of the configs, CUDA events around four back-to-back launches, 512 MB written
    between repeats to flush L2."""
    flush = torch.empty(512 << 20, dtype=torch.uint8, device=device)

    def timeit(fn, reps=10, inner=4):
        # `inner` launches back to back between the events: the host-side cost of one call (tens of
        # microseconds of Python and ctypes) would otherwise sit inside the measured interval while the
        # GPU idles.  The tensors of one call are larger than L2 or are flushed by the call before it.
        ts = []
        for _ in range(3):
            fn()
        for _ in range(reps):
            flush.fill_(1)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            fn()  # queue depth: the timed launches below are issued while this one runs
            e0.record()
            for _ in range(inner):
                fn()
            e1.record()
            torch.cuda.synchronize(device)
            ts.append(e0.elapsed_time(e1) / inner)
        ts.sort()
        return ts[len(ts) // 2] * 1e-3

    res = {}
    bf = torch.bfloat16
    # Ulysses pack of Wan q,k,v at R4xU2: three [1,40,9450,128] tensors viewed from [1,9450,40,128]
    H, s, D, U = 40, 9450, 128, 2
    srcs = [torch.randn(1, s, H, D, device=device, dtype=bf).transpose(1, 2) for _ in range(3)]
    blk = (H // U) * s * D
    send = torch.empty(3 * U * blk, dtype=bf, device=device)
    items = [dict(src=t, dst=send[i * blk:], peer_stride=3 * blk) for i, t in enumerate(srcs)]
    t = timeit(lambda: ops.ulysses_pack(items, U))
    nbytes = 2 * 3 * H * s * D * 2
    res["ulysses_pack_wan_qkv"] = {"bytes": nbytes, "ms": t * 1e3, "achieved": nbytes / t / 1e9}
    del srcs, send
    # fused prologue on the same shard: RMSNorm(q, k) over 5120 + rotary embedding + head split + pack of
    # the three [1, 9450, 5120] projections of a Wan layer (plus the fp32 cos/sin rows of a token)
    proj = [torch.randn(1, s, H * D, device=device, dtype=bf) for _ in range(3)]
    wn = torch.ones(H * D, device=device, dtype=bf)
    ang = torch.randn(s, D // 2, device=device)
    cs, sn = ang.cos().repeat_interleave(2, 1).contiguous(), ang.sin().repeat_interleave(2, 1).contiguous()
    send = torch.empty(3 * U * blk, dtype=bf, device=device)
    t = timeit(lambda: ops.qk_norm_rope_pack(proj[0], proj[1], proj[2], H, send, send[blk:], send[2 * blk:],
                                             (3 * blk, 3 * blk, 3 * blk), U, norm_q_weight=wn, norm_k_weight=wn,
                                             cos=cs, sin=sn))
    nbytes = 2 * 3 * H * s * D * 2 + 2 * 2 * s * D * 4
    res["qk_norm_rope_pack_wan"] = {"bytes": nbytes, "ms": t * 1e3, "achieved": nbytes / t / 1e9}
    del proj, send
    # PipeFusion stale-KV patch, PixArt-Sigma 2048^2: 2048 fresh rows of 16 x 72 into 16384-row caches
    kc = torch.zeros(1, 16, 16384, 72, dtype=bf, device=device)
    vc = torch.zeros_like(kc)
    kn = torch.randn(1, 2048, 16, 72, device=device, dtype=bf).transpose(1, 2)
    vn = torch.randn(1, 2048, 16, 72, device=device, dtype=bf).transpose(1, 2)
    t = timeit(lambda: ops.kv_patch_update(kc, vc, kn, vn, 4096))
    nbytes = 2 * 2 * 16 * 2048 * 72 * 2
    res["kv_patch_pixart"] = {"bytes": nbytes, "ms": t * 1e3, "achieved": nbytes / t / 1e9}
    # stand-alone merge at one Wan ring step: rows = 20 heads x 18900, D = 128
    rows = 20 * 18900
    oa = torch.randn(rows, 128, device=device)
    la = torch.randn(rows, device=device)
    ob = torch.randn(rows, 128, device=device, dtype=bf)
    lb = torch.randn(rows, device=device)
    t = timeit(lambda: ops.merge_out_lse(oa, la, ob, lb, first=False))
    nbytes = rows * 128 * (4 + 4 + 2) + rows * 12
    res["merge_wan_ring_step"] = {"bytes": nbytes, "ms": t * 1e3, "achieved": nbytes / t / 1e9}
    for r in res.values():
        r["unit"] = "GB/s"
        r["peak"] = hbm_peak
        r["frac"] = r["achieved"] / hbm_peak
        r["peak_kind"] = f"of {peak_kind} (copy)"
    return res


def pixart_leg(torch, xdit_b200, ops, device, tf_peak):
    """PixArt-Sigma 2048x2048 with PipeFusion in its steady state, as one GPU of the pipeline sees it:
    16 heads x 72, a patch of 2048 fresh tokens attends to the layer's 16,384-token K/V buffer of which
    7/8 is stale; every call first writes the patch's fresh K/V rows into the buffer
    (``USP(..., attn_layer=...)`` -> stale-KV manager -> ``xdit_kv_patch_update``), then attends.
    7 layers of a pipeline stage x 8 patches per timed pass."""
    import numpy as np

    from oracle import usp_oracle as O

    H, D, S, NP, LAYERS = 16, 72, 16384, 8, 7
    n = S // NP
    xdit_b200.init_sequence_parallel(1, 1)
    rs = xdit_b200.initialize_runtime_state()
    rs.set_patches([n] * NP)
    mgr = xdit_b200.get_cache_manager()
    bf = torch.bfloat16
    g = torch.Generator(device=device)
    g.manual_seed(72)
    mk = lambda rows: torch.randn(1, rows, H, D, generator=g, device=device, dtype=torch.float32).to(bf).transpose(1, 2)
    layers = [f"pixart_layer_{i}" for i in range(LAYERS)]
    full = {}
    rs.set_patched_mode(False)
    for name in layers:  # warm-up step: full sequence, fills the buffers
        mgr.register_cache_entry(name, "attn", "naive_cache")
        q, k, v = mk(S), mk(S), mk(S)
        full[name] = (k, v)
        xdit_b200.USP(q, k, v, attn_layer=name)
    fresh = {name: [(mk(n), mk(n), mk(n)) for _ in range(NP)] for name in layers}
    rs.set_patched_mode(True)

    def one_pass():
        for p in range(NP):
            rs.pipeline_patch_idx = p
            for name in layers:
                q, k, v = fresh[name][p]
                xdit_b200.USP(q, k, v, attn_layer=name)

    # parity of one steady-state call: patch 3 of layer 0 against dense attention over the buffer it
    # must see (warm-up rows, rows of patch 3 replaced by the fresh ones)
    name, p = layers[0], 3
    rs.pipeline_patch_idx = p
    q, k, v = fresh[name][p]
    out = xdit_b200.USP(q, k, v, attn_layer=name)
    torch.cuda.synchronize(device)
    kk, vv = full[name][0].clone(), full[name][1].clone()
    kk[:, :, p * n:(p + 1) * n], vv[:, :, p * n:(p + 1) * n] = k, v
    f64 = lambda t: t.float().cpu().double().numpy()
    rows = slice(0, 96)
    want, _ = O.attention_dense(f64(q[:, :2, rows]), f64(kk[:, :2]), f64(vv[:, :2]))
    got = f64(out[:, :2, rows])
    max_abs = float(np.abs(got - want).max())
    cos = float((got * want).sum() / (np.linalg.norm(got) * np.linalg.norm(want)))
    ok = max_abs <= TOL_MAX_ABS and cos >= TOL_COS
    for _ in range(3):
        one_pass()
    torch.cuda.synchronize(device)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = 5
    e0.record()
    for _ in range(reps):
        one_pass()
    e1.record()
    torch.cuda.synchronize(device)
    ops.check_status()
    ms = e0.elapsed_time(e1) / reps
    calls = NP * LAYERS
    fl = 4.0 * n * S * H * D * calls
    rs.set_patched_mode(False)
    rs.set_patches([])
    return {"desc": "PixArt-Sigma 2048x2048 PipeFusion steady state on one GPU: 16 heads x 72, 2048 fresh of 16,384 "
                    "tokens per call, stale-KV patch update + attention, 7 layers x 8 patches per pass",
            "calls_per_pass": calls, "ms_per_call": ms / calls, "tflops_per_gpu": fl / (ms * 1e-3) / 1e12,
            "frac_of_measured_bf16_burst_peak": fl / (ms * 1e-3) / 1e12 / tf_peak,
            "l2": "7 layers x (2 x 37.7 MB of K/V buffers + fresh rows) = 0.6 GB cycled, larger than L2",
            "parity": {"max_abs": max_abs, "cos": cos, "rows": 192, "ok": ok,
                       "against": "oracle dense attention over the patched K/V buffer"}}, ok


def head_dim_legs(torch, ops, device, tf_peak):
    """The tcgen05 kernel at the other head dims the reference's models use: 64 (SD3 / CogVideoX: 24 heads,
    8192 tokens here) and 72 (PixArt: 16 heads over the full 16,384 tokens of a 2048 x 2048 image), dense,
    one GPU, several input sets cycled so that K and V come from HBM; sampled rows against the oracle."""
    import numpy as np

    from oracle import usp_oracle as O

    res, all_ok = {}, True
    for label, H, S, D, sets in (("d64_h24_s8192", 24, 8192, 64, 8), ("d72_h16_s16384", 16, 16384, 72, 4)):
        g = torch.Generator(device=device)
        g.manual_seed(D)
        ins = [tuple(torch.randn(1, H, S, D, generator=g, device=device).to(torch.bfloat16) for _ in range(3))
               for _ in range(sets)]
        out = torch.empty_like(ins[0][0])
        for q, k, v in ins[:3]:
            ops.attn_fwd(q, k, v, out=out)
        q, k, v = ins[0]
        ops.attn_fwd(q, k, v, out=out)
        torch.cuda.synchronize(device)
        f64 = lambda t: t.float().cpu().double().numpy()
        rows = [0, S // 2, S - 64]
        got = np.concatenate([f64(out[:, :2, r:r + 64]) for r in rows], axis=2)
        want = np.concatenate([O.attention_dense(f64(q[:, :2, r:r + 64]), f64(k[:, :2]), f64(v[:, :2]))[0]
                               for r in rows], axis=2)
        max_abs = float(np.abs(got - want).max())
        cos = float((got * want).sum() / (np.linalg.norm(got) * np.linalg.norm(want)))
        ok = max_abs <= TOL_MAX_ABS and cos >= TOL_COS
        all_ok &= ok
        reps = 5
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            for q, k, v in ins:
                ops.attn_fwd(q, k, v, out=out)
        e1.record()
        torch.cuda.synchronize(device)
        ops.check_status()
        ms = e0.elapsed_time(e1) / (reps * sets)
        tf = 4.0 * S * S * H * D / (ms * 1e-3) / 1e12
        res[label] = {"heads": H, "tokens": S, "head_dim": D, "ms_per_call": ms, "tflops_per_gpu": tf,
                      "frac_of_measured_bf16_burst_peak": tf / tf_peak,
                      "l2": f"{sets} input sets of {3 * H * S * D * 2 / 1e6:.0f} MB cycled",
                      "parity": {"max_abs": max_abs, "cos": cos, "rows": 384, "ok": ok}}
        del ins, out
        torch.cuda.empty_cache()
    return res, all_ok


def pixart_pipeline_leg(torch, dist, xdit_b200, ops, device, rank, world, steps=3):
    """PixArt-Sigma 2048x2048 with PipeFusion across GPUs, as a random-init stand-in: 28 blocks (hidden 1152,
    16 heads x 72, text cross-attention to 300 tokens, MLP x4) cut into 4 pipeline stages of 7 blocks, 16,384
    tokens in 8 patches that travel stage to stage (``xdit_b200.pipefusion``), stale K/V for the other
    patches; with 8 GPUs two such pipelines run side by side as the two classifier-free-guidance branches
    and the last stages combine their predictions per patch.  Timed: denoising steps of the asynchronous
    phase (after one full-sequence warm-up step), CUDA events, max over ranks.  Checked: an echo pass
    through the same pipe (every stage adds 1) must reach the last stage as input + stages, patch by patch."""
    import torch.nn.functional as F

    from xdit_b200.model_boundary import gather_cfg
    from xdit_b200.pipefusion import PatchPipe, run_async_steps

    PP = 4
    if world % PP:
        return {"skipped": f"needs a multiple of {PP} GPUs"}, True
    branches = world // PP
    branch, stage_idx = rank // PP, rank % PP
    pp_group = cfg_group = None
    for b_ in range(branches):
        gpg = dist.new_group(list(range(b_ * PP, (b_ + 1) * PP)))
        if b_ == branch:
            pp_group = gpg
    for st in range(PP):
        gcf = dist.new_group([b_ * PP + st for b_ in range(branches)])
        if st == stage_idx:
            cfg_group = gcf
    H, D, S, NP, LPS, TXT = 16, 72, 16384, 8, 7, 300
    hid, n = H * D, S // NP
    bf = torch.bfloat16
    xdit_b200.init_sequence_parallel(1, 1)
    rs = xdit_b200.initialize_runtime_state()
    rs.set_patches([n] * NP)
    mgr = xdit_b200.get_cache_manager()
    g = torch.Generator(device=device)
    g.manual_seed(100 + stage_idx)  # the two branches hold the same weights
    lin = lambda i, o: torch.randn(o, i, device=device, dtype=torch.float32, generator=g).mul_(0.02).to(bf)
    blocks = [dict(qkv=lin(hid, 3 * hid), o=lin(hid, hid), cq=lin(hid, hid), ckv=lin(hid, 2 * hid), co=lin(hid, hid),
                   up=lin(hid, 4 * hid), down=lin(4 * hid, hid), name=f"pixart_pp_{stage_idx}_{i}") for i in range(LPS)]
    for b_ in blocks:
        mgr.register_cache_entry(b_["name"], "attn", "naive_cache")
    ctx = torch.randn(1, TXT, hid, device=device, generator=g).to(bf)

    def stage(x, step, p):
        rows = x.shape[1]
        for b_ in blocks:
            q, k, v = F.linear(F.layer_norm(x, (hid,)), b_["qkv"]).view(1, rows, 3, H, D).unbind(2)
            a = xdit_b200.USP(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), attn_layer=b_["name"])
            x = x + F.linear(a.transpose(1, 2).reshape(1, rows, hid), b_["o"])
            cq = F.linear(x, b_["cq"]).view(1, rows, H, D).transpose(1, 2)
            ck, cv = F.linear(ctx, b_["ckv"]).view(1, TXT, 2, H, D).unbind(2)
            c = xdit_b200.attention(cq, ck.transpose(1, 2), cv.transpose(1, 2))
            x = x + F.linear(c.transpose(1, 2).reshape(1, rows, hid), b_["co"])
            x = x + F.linear(F.gelu(F.linear(F.layer_norm(x, (hid,)), b_["up"]), approximate="tanh"), b_["down"])
        return x

    def finish(y, step, p):
        if branches == 1:
            return y
        both = gather_cfg(y, cfg_group, branches)  # [2, n, hid]: the two guidance branches of this patch
        return (both[0:1] + 4.5 * (both[1:2] - both[0:1])).to(y.dtype)

    pipe = PatchPipe(pp_group, [n] * NP, 1, hid, bf, device)
    first, last_rank = branch * PP, branch * PP + PP - 1
    x0 = torch.randn(1, S, hid, device=device, generator=g).to(bf)
    with torch.no_grad():
        # warm-up step: the full sequence through the stages, K/V buffers filled
        rs.set_patched_mode(False)
        y = x0
        if stage_idx > 0:
            y = torch.empty_like(x0)
            dist.recv(y, src=rank - 1)
        y = stage(y, -1, 0)
        dist.send(y.contiguous(), dst=rank + 1 if stage_idx < PP - 1 else first)
        first_input = None
        if stage_idx == 0:
            warm = torch.empty_like(x0)
            dist.recv(warm, src=last_rank)
            first_input = list(warm.split(n, dim=1))
        run_async_steps(pipe, stage, 1, rs, first_input=first_input, finish_patch=finish)  # untimed first async step
        torch.cuda.synchronize(device)
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        run_async_steps(pipe, stage, steps, rs, first_input=first_input, finish_patch=finish)
        e1.record()
        torch.cuda.synchronize(device)
        ops.check_status()
        ms = e0.elapsed_time(e1) / steps
        # echo pass through the same pipe: every stage adds 1 to whatever it is handed
        echo_in = [torch.full((1, n, hid), float(p), device=device, dtype=bf) for p in range(NP)]
        out = run_async_steps(pipe, lambda x, i, p: x + 1, 1, rs, first_input=echo_in if stage_idx == 0 else None)
        ok = 1.0
        if stage_idx == PP - 1:
            ok = float(all(bool((out[p] == p + PP).all()) for p in range(NP)))
    t = torch.tensor([ms, -ok], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ok = float(t[1]) == -1.0
    fl = 4.0 * n * S * H * D * NP * LPS * PP  # self-attention flop of one denoising step of one branch
    return {"desc": "PixArt-Sigma 2048x2048 stand-in, PipeFusion: 4 stages x 7 blocks, 8 patches of 2048 tokens, "
                    "stale K/V, patch hand-off over NCCL point-to-point" + (", 2 guidance branches" if branches > 1 else ""),
            "pipeline_stages": PP, "cfg_branches": branches, "steps_timed": steps, "ms_per_denoising_step": float(t[0]),
            "self_attention_tflops_per_branch": fl / (float(t[0]) * 1e-3) / 1e12,
            "parity": {"ok": ok, "what": "echo pass: input + 4 at the last stage, every patch in its place"}}, ok


def gpu_backends(torch, device, ours_ms, tf_peak):
    """The library kernels the reference would dispatch to on this GPU, timed as black boxes next to
    this package's kernel: one Flux layer and one Wan layer, local tensors on one GPU, CUDA events.
    Called through the reference's own registered back-end functions
    (``xfuser/core/distributed/attention_backend.py:504-516, 550-566, 887-918, 644-673``) when its sources are
    under ``oracle/_ref``, else through the same aten / flash_attn calls those functions make."""
    shapes = {"flux": (24, 4608, 128, 5), "wan": (40, 75600, 128, 2)}
    calls = {}
    source = "aten / flash_attn calls as the reference's back-end functions make them"
    try:
        from oracle import ref_import

        if ref_import.root() is not None:
            _usp, backend, _c, _r = ref_import.import_usp()
            T = backend.AttentionBackendType
            reg = backend.ATTENTION_FUNCTION_REGISTRY
            for key, member in (("cudnn", T.CUDNN), ("sdpa_flash", T.SDPA_FLASH), ("flash", T.FLASH),
                                ("flash_4", T.FLASH_4)):
                if member in reg:
                    calls[key] = (lambda q, k, v, f=reg[member]: f(q, k, v, 0.0, False))
            source = "the reference's own registered back-end functions (oracle/_ref)"
    except Exception:  # noqa: BLE001
        calls = {}
    aten = torch.ops.aten
    calls.setdefault("cudnn", lambda q, k, v: aten._scaled_dot_product_cudnn_attention(
        q, k, v, attn_bias=None, compute_log_sumexp=True, dropout_p=0.0, is_causal=False))
    calls.setdefault("sdpa_flash", lambda q, k, v: aten._scaled_dot_product_flash_attention(
        q, k, v, dropout_p=0.0, is_causal=False))

    def _fa2(q, k, v):
        from flash_attn import flash_attn_func

        return flash_attn_func(q.permute(0, 2, 1, 3), k.permute(0, 2, 1, 3), v.permute(0, 2, 1, 3), dropout_p=0.0,
                               causal=False, return_attn_probs=True)

    def _fa4(q, k, v):
        from flash_attn.cute.interface import flash_attn_func as fa4

        return fa4(q.permute(0, 2, 1, 3).contiguous(), k.permute(0, 2, 1, 3).contiguous(),
                   v.permute(0, 2, 1, 3).contiguous(), causal=False)

    calls.setdefault("flash", _fa2)
    calls.setdefault("flash_4", _fa4)
    res = {"source": source}
    for wname, (H, S, D, reps) in shapes.items():
        g = torch.Generator(device=device)
        g.manual_seed(5)
        q, k, v = (torch.randn(1, H, S, D, generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
                   for _ in range(3))
        fl = 4.0 * S * S * H * D
        row = {"ours_ms": ours_ms.get(wname), "ours_tflops": fl / (ours_ms[wname] * 1e-3) / 1e12
               if ours_ms.get(wname) else None}
        for key, fn in calls.items():
            try:
                for _ in range(2):
                    fn(q, k, v)
                torch.cuda.synchronize(device)
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(reps):
                    fn(q, k, v)
                e1.record()
                torch.cuda.synchronize(device)
                ms = e0.elapsed_time(e1) / reps
                row[key] = {"ms": ms, "tflops": fl / (ms * 1e-3) / 1e12,
                            "ours_over_it": (ms / ours_ms[wname]) if ours_ms.get(wname) else None}
            except Exception as e:  # noqa: BLE001
                row[key] = {"unavailable": "unavailable on this box: " + repr(e)[:160]}
                try:
                    torch.cuda.synchronize(device)
                except Exception:  # noqa: BLE001
                    pass
        res[wname] = row
        del q, k, v
        torch.cuda.empty_cache()
    return res


# --------------------------------------------------------------------------------------------
# DiT step latency on random-init stand-ins of the named architectures (plain torch bf16 for
# everything but attention; no checkpoint or diffusers is available here)
# --------------------------------------------------------------------------------------------
def dit_step_latency(torch, dist, xdit_b200, kind, device, rank, world, reps=5, fused_prologue=True):
    """One transformer forward (= one denoising step) of a Flux.1-dev-shaped MMDiT or a
    Wan2.1-14B-shaped video DiT: QKV/out projections, MLPs and norms in torch bf16 with N(0, 0.02)
    weights, the sequence sharded over the ranks (Ulysses degree = ranks), and the model-exit sequence
    gather that hands every rank the full output.  Self-attention from the projections on: with
    ``fused_prologue`` through ``xdit_b200.prologue.attention_from_projections`` (q/k RMS-norm, rotary
    embedding, head split and pack in one kernel; the head merge feeds the output projection without a
    re-layout copy), otherwise q/k RMS-norm and rotary embedding in torch and ``xdit_b200.USP``, the way
    the reference's processors are written.  Text cross-attention through ``xdit_b200.attention``.
    Returns milliseconds (median)."""
    import torch.nn.functional as F

    from xdit_b200.model_boundary import gather_sequence
    from xdit_b200.prologue import attention_from_projections

    bf = torch.bfloat16
    w = WORKLOADS[kind]
    U, R = world, 1
    xdit_b200.init_sequence_parallel(U, R)
    P = U * R
    H, D, S = w["H"], w["D"], w["S"]
    hid = H * D
    s = S // P
    g = torch.Generator(device=device)
    g.manual_seed(0)

    def lin(i, o):
        return torch.randn(o, i, device=device, dtype=torch.float32, generator=g).mul_(0.02).to(bf)

    per_head = kind == "flux"  # Flux normalises q and k per head, Wan over all heads of a token
    wq = (1 + 0.1 * torch.randn(D if per_head else hid, device=device, generator=g)).to(bf)
    wk = (1 + 0.1 * torch.randn(D if per_head else hid, device=device, generator=g)).to(bf)
    ang = torch.randn(s, D // 2, device=device, generator=g)
    cos = ang.cos().repeat_interleave(2, 1).contiguous()  # fp32 [s, D], each frequency twice
    sin = ang.sin().repeat_interleave(2, 1).contiguous()
    rotary = (cos[None, :, None, :], sin[None, :, None, :])

    def rope(x):  # x [B, s, H, D], interleaved pairs as in the reference's Wan processor
        x1, x2 = x.unflatten(-1, (-1, 2)).unbind(-1)
        out = torch.empty_like(x)
        out[..., 0::2] = x1 * rotary[0][..., 0::2] - x2 * rotary[1][..., 1::2]
        out[..., 1::2] = x1 * rotary[1][..., 1::2] + x2 * rotary[0][..., 0::2]
        return out

    def attn(q, k, v, w_out):  # [B, s, H, D] views of the projections -> output projection applied
        if fused_prologue:
            return attention_from_projections(q.reshape(1, s, hid), k.reshape(1, s, hid), v.reshape(1, s, hid), H,
                                              norm_q_weight=wq, norm_k_weight=wk, eps=1e-6, norm_per_head=per_head,
                                              rotary_emb=rotary, out_proj_weight=w_out)
        if per_head:
            q, k = F.rms_norm(q, (D,), wq, 1e-6), F.rms_norm(k, (D,), wk, 1e-6)
        else:
            q = F.rms_norm(q.reshape(1, s, hid), (hid,), wq, 1e-6).view(1, s, H, D)
            k = F.rms_norm(k.reshape(1, s, hid), (hid,), wk, 1e-6).view(1, s, H, D)
        o = xdit_b200.USP(rope(q).transpose(1, 2), rope(k).transpose(1, 2), v.transpose(1, 2))
        return F.linear(o.transpose(1, 2).reshape(1, s, hid), w_out)

    x = torch.randn(1, s, hid, device=device, generator=g).to(bf)
    if kind == "flux":
        mlp = 4 * hid
        dbl = [dict(qkv=lin(hid, 3 * hid), proj=lin(hid, hid), up=lin(hid, mlp), down=lin(mlp, hid)) for _ in range(19)]
        sgl = [dict(l1=lin(hid, 3 * hid + mlp), l2a=lin(hid, hid), l2m=lin(mlp, hid)) for _ in range(38)]

        def forward(x):
            # text and image tokens form one sharded sequence; a double block differs from a single
            # one by its separate attention/MLP projections (per-stream weights are applied to the
            # whole shard here: same flops and bytes per token)
            for b in dbl:
                h_ = F.layer_norm(x, (hid,))
                q, k, v = F.linear(h_, b["qkv"]).view(1, s, 3, H, D).unbind(2)
                x = x + attn(q, k, v, b["proj"])
                x = x + F.linear(F.gelu(F.linear(F.layer_norm(x, (hid,)), b["up"]), approximate="tanh"), b["down"])
            for b in sgl:
                h_ = F.linear(F.layer_norm(x, (hid,)), b["l1"])
                q, k, v = h_[..., : 3 * hid].view(1, s, 3, H, D).unbind(2)
                # the single block's output projection over cat(attention, MLP) is the sum of its two halves
                x = x + attn(q, k, v, b["l2a"]) + F.linear(F.gelu(h_[..., 3 * hid:], approximate="tanh"), b["l2m"])
            return gather_sequence(x, dim=1)
    else:
        ffn, txt_len, txt_dim = 13824, 512, 4096
        ctx = torch.randn(1, txt_len, txt_dim, device=device, generator=g).to(bf)
        blocks = [dict(q=lin(hid, hid), k=lin(hid, hid), v=lin(hid, hid), o=lin(hid, hid), cq=lin(hid, hid),
                       ck=lin(txt_dim, hid), cv=lin(txt_dim, hid), co=lin(hid, hid), up=lin(hid, ffn),
                       down=lin(ffn, hid)) for _ in range(40)]

        def forward(x):
            for b in blocks:
                h_ = F.layer_norm(x, (hid,))
                q, k, v = (F.linear(h_, b[n]).view(1, s, H, D) for n in ("q", "k", "v"))
                x = x + attn(q, k, v, b["o"])
                h_ = F.layer_norm(x, (hid,))
                cq = F.linear(h_, b["cq"]).view(1, s, H, D).transpose(1, 2)
                ck = F.linear(ctx, b["ck"]).view(1, txt_len, H, D).transpose(1, 2)
                cv = F.linear(ctx, b["cv"]).view(1, txt_len, H, D).transpose(1, 2)
                x = x + F.linear(xdit_b200.attention(cq, ck, cv).transpose(1, 2).reshape(1, s, hid), b["co"])
                x = x + F.linear(F.gelu(F.linear(F.layer_norm(x, (hid,)), b["up"]), approximate="tanh"), b["down"])
            return gather_sequence(x, dim=1)

    with torch.no_grad():
        for _ in range(2 if kind == "flux" else 1):
            forward(x)
        times = []
        for _ in range(reps):
            torch.cuda.synchronize(device)
            if world > 1:
                dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); forward(x); e1.record()
            torch.cuda.synchronize(device)
            times.append(e0.elapsed_time(e1))
    times.sort()
    ms = times[len(times) // 2]
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return {"ms_per_step": ms, "ulysses": U, "ring": R, "reps": reps,
            "what": "one forward of a random-init stand-in (torch bf16 linears/norms/MLPs + xdit_b200 attention + "
                    "the model-exit sequence gather; "
                    + ("q/k norm + rotary embedding + head split fused with the pack, head merge fed to the output "
                       "projection without a copy" if fused_prologue
                       else "q/k norm and rotary embedding in torch, as the reference's processors do") + ")"}


def cpu_baseline(w):
    try:
        val, ms, sample, kind, cores = host_sample(w, 15.0, 3, 1)
    except Exception as e:  # noqa: BLE001  (a host-side import problem must not cost the GPU line)
        return {"value": None, "unit": "TFLOP/s", "cores": os.cpu_count(), "kind": "unavailable", "sample": repr(e)[:200]}
    return {"value": val, "unit": "TFLOP/s", "cores": cores, "kind": kind, "sample": sample}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="wan", choices=["flux", "wan"])
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-extra", action="store_true", help="skip the secondary workloads, legs and the CPU baseline")
    ap.add_argument("--extras", default="all",
                    help="comma list of the legs to run under `extra`: other,alt_exchange,ring,hunyuan,pp,pixart,head_dims,hbm,"
                         "backends,dit,cpu (default: all)")
    ap.add_argument("--layers", type=int, default=0, help="time only this many layers per step (profiling aid)")
    ap.add_argument("--dit", default="both", choices=["none", "flux", "wan", "both"],
                    help="also time one DiT forward of a random-init stand-in of this architecture (extra.dit_step)")
    ap.add_argument("--sp", default=None, help="override the sequence-parallel degrees of the main workload: ULYSSESxRING, e.g. 2x4")
    ap.add_argument("--no-e2e", action="store_true", help="skip the end-to-end (host buffers) leg")
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"],
                    help="Ulysses exchange at N > 1: stores into the peers' memory (kept only if a probing call "
                         "succeeds on every rank) or NCCL all-to-alls")
    ap.add_argument("--graph", default="auto", choices=["auto", "on", "off"],
                    help="replay the step as a CUDA graph (auto: only when N > 1, where the step is launch-bound)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    name = args.workload
    w = WORKLOADS[name]

    if args.impl == "reference":
        run_reference(args, w, name)
        return

    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the kernels have no CPU fallback")
    cpus_before = os.sched_getaffinity(0)
    numa_bound = bind_to_gpu_numa_node(local)
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)

    import xdit_b200
    from xdit_b200 import build, ops

    if rank == 0:
        build.build()
    if world > 1:
        dist.barrier()
    assert ops.query_caps()["supported"] == 1, "not an sm_100 device"

    tf_peak, tf_sustained, hbm_peak, peak_kind = peaks()
    if args.layers > 0:
        w = dict(w, layers=min(args.layers, w["layers"]))
    U, R = world, 1
    if args.sp:
        U, R = (int(x) for x in args.sp.lower().split("x"))
        assert U * R == world, "--sp UxR must multiply to the number of GPUs"
    main_res = run_workload(torch, dist, xdit_b200, ops, name, w, args, device, rank, world, w["layers"],
                            not args.no_e2e, U, R, exchange=args.exchange)
    all_ok = main_res["parity"]["ok"]
    extra = {}
    want = (lambda k: True) if args.extras == "all" else (lambda k, sel=set(args.extras.split(",")): k in sel)
    other = "wan" if name == "flux" else "flux"
    layers = 4 if other == "wan" else WORKLOADS[other]["layers"]
    if not args.no_extra and want("other"):
        wo = WORKLOADS[other]
        extra[other], ok = leg(torch, dist, xdit_b200, ops, other, wo, args, device, rank, world, layers, world, 1,
                               tf_peak, exchange=args.exchange)
        all_ok &= ok
    if not args.no_extra:
        # the same Ulysses split with the other form of the exchange (NCCL all-to-alls when the main legs
        # use stores into the peers' memory, and the other way round), a few layers each
        if world > 1 and want("alt_exchange"):
            alt = "nccl" if main_res["exchange"] == "peer_stores" else "peer"
            for wl, nl in ((other, min(layers, 19)), (name, min(4, w["layers"]))):
                extra[f"{wl}_{'nccl' if alt == 'nccl' else 'peer_stores'}"], ok = leg(
                    torch, dist, xdit_b200, ops, wl, WORKLOADS[wl], args, device, rank, world, nl, world, 1, tf_peak,
                    exchange=alt)
                all_ok &= ok
            try:
                from xdit_b200 import peer_exchange

                peer_exchange.enable(False)
            except Exception:  # noqa: BLE001
                pass
            torch.cuda.empty_cache()
        # ring legs: the K/V rotation over NCCL with the merge in the kernel epilogue, checked the same way
        if world > 1 and want("ring"):
            splits = [(1, world)] + ([(2, 4)] if world == 8 else []) + ([(2, 2)] if world == 4 else [])
            for (u, r) in splits:
                extra[f"wan_ring_u{u}r{r}"], ok = leg(torch, dist, xdit_b200, ops, "wan", WORKLOADS["wan"], args,
                                                      device, rank, world, 4, u, r, tf_peak, steps=2,
                                                      exchange=args.exchange)
                all_ok &= ok
                if extra[f"wan_ring_u{u}r{r}"].get("exchange") == "peer_copies":
                    # the same split with the rotation over NCCL send/recv
                    extra[f"wan_ring_u{u}r{r}_nccl"], ok = leg(torch, dist, xdit_b200, ops, "wan", WORKLOADS["wan"],
                                                               args, device, rank, world, 4, u, r, tf_peak, steps=2,
                                                               exchange="nccl")
                    all_ok &= ok
        # the ring-dominant long-context case (119,056 tokens); ring degree = ranks, one GPU runs it dense
        wh = WORKLOADS["hunyuan"]
        if wh["S"] % world == 0 and want("hunyuan"):
            extra["hunyuan_ring"], ok = leg(torch, dist, xdit_b200, ops, "hunyuan", wh, args, device, rank, world,
                                            2, 1, world, tf_peak, steps=2, exchange=args.exchange)
            all_ok &= ok
        if world % 4 == 0 and want("pp"):
            try:
                extra["pixart_pipefusion_pp4"], ok = pixart_pipeline_leg(torch, dist, xdit_b200, ops, device, rank, world)
                all_ok &= ok
            except Exception as e:  # noqa: BLE001
                import traceback

                extra["pixart_pipefusion_pp4"] = {"error": repr(e)[:300], "trace": traceback.format_exc()[-600:]}
            torch.cuda.empty_cache()
        if world == 1 and want("pixart"):
            try:
                extra["pixart_pipefusion_steady"], ok = pixart_leg(torch, xdit_b200, ops, device, tf_peak)
                all_ok &= ok
            except Exception as e:  # noqa: BLE001
                extra["pixart_pipefusion_steady"] = {"error": repr(e)[:300]}
        if world == 1 and want("head_dims"):
            try:
                extra["head_dims"], ok = head_dim_legs(torch, ops, device, tf_peak)
                all_ok &= ok
            except Exception as e:  # noqa: BLE001
                extra["head_dims"] = {"error": repr(e)[:300]}
        if world == 1 and want("hbm"):
            try:
                extra["hbm_kernels"] = hbm_kernels(torch, ops, device, hbm_peak, peak_kind)
            except Exception as e:  # noqa: BLE001
                extra["hbm_kernels"] = {"error": repr(e)[:200]}
        if world == 1 and want("backends"):
            try:
                ours_ms = {name: main_res["ms_per_step"] / w["layers"]}
                if "ms_per_layer_call" in extra.get(other, {}):
                    ours_ms[other] = extra[other]["ms_per_layer_call"]
                extra["gpu_backends"] = gpu_backends(torch, device, ours_ms, tf_peak)
            except Exception as e:  # noqa: BLE001
                extra["gpu_backends"] = {"error": repr(e)[:200]}
        if args.dit != "none" and want("dit"):
            extra["dit_step"] = {}
            for kind in (("flux", "wan") if args.dit == "both" else (args.dit,)):
                try:
                    reps = 5 if kind == "flux" else 2
                    r_f = dit_step_latency(torch, dist, xdit_b200, kind, device, rank, world, reps=reps)
                    if kind == "flux":
                        r_t = dit_step_latency(torch, dist, xdit_b200, kind, device, rank, world, reps=reps,
                                               fused_prologue=False)
                        r_f["ms_per_step_torch_prologue"] = r_t["ms_per_step"]
                    extra["dit_step"][kind] = r_f
                except Exception as e:  # noqa: BLE001
                    import traceback

                    extra["dit_step"][kind] = {"error": repr(e)[:200], "trace": traceback.format_exc()[-500:]}
                torch.cuda.empty_cache()

    if rank == 0:
        calls = w["layers"]
        kernel_ms = main_res["ms_per_step"] / calls
        per_gpu_tf = main_res["tflops"] / world
        line = {
            "metric": "usp_attn_tflops", "value": main_res["tflops"], "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": main_res["ms_per_step"],
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": {
                "workload": name, "desc": w["desc"], "step": f"{calls} USP attention calls (one per layer)",
                "ulysses": main_res["U"], "ring": main_res["R"], "cuda_graph": main_res["cuda_graph"],
                "exchange": main_res["exchange"], "exchange_note": main_res.get("exchange_note"),
                "tokens": w["S"], "heads": w["H"],
                "head_dim": w["D"], "global_batch": 1,
                "l2": f"inputs larger than L2: {main_res['sets']} distinct q/k/v sets cycled layer by layer "
                      f"({main_res['sets'] * 3 * w['H'] * w['S'] * w['D'] * 2 / 1e9:.1f} GB over all ranks)",
                "host_numa_bound": numa_bound,
            },
            "tflops_per_gpu": per_gpu_tf,
            "parity": dict(main_res["parity"], all_legs_ok=bool(all_ok)),
            "roofline": roofline(w, main_res, per_gpu_tf, kernel_ms, world, tf_peak, tf_sustained, peak_kind),
            "e2e": main_res.get("e2e"),
            "clocks": main_res["clocks"],
            "gpu_launches": main_res["launches"],
            "extra": extra,
        }
        if world > 1:
            line["nvlink"] = nvlink_bytes(w, main_res["U"], main_res["R"])
        if world == 1 and not args.no_extra and want("cpu"):
            os.sched_setaffinity(0, cpus_before)  # the host baseline gets every core again
            line["cpu_baseline"] = cpu_baseline(w)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if not all_ok:
        raise SystemExit("parity check failed: a sampled row is outside max-abs 2e-2 / cosine 0.9999 (see `parity`)")


if __name__ == "__main__":
    main()
