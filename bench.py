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

N > 1 is launched by ``torch.distributed.run`` (one rank per GPU, NCCL); the sequence is sharded
over N ranks (strong scaling) with Ulysses degree N, which is the fastest split behind NVSwitch
(measured at 8 GPUs on the 75.6K workload: U8 7755, U4xR2 7438, U2xR4 6872, R8 6046 TFLOP/s);
``--sp ULYSSESxRING`` selects another split, e.g. ``--sp 2x4`` for Ulysses 2 x ring 4, the split the Wan2.1 workload is usually quoted with.

``--impl reference`` times the CPU restatement of the reference's algorithm (the oracle) on the
host cores of rank 0, on a bounded sample (a subset of heads) of the same workload.
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
    # name: layers, heads, head_dim, tokens, {n_gpus: (ulysses, ring)}
    "flux": dict(desc="Flux.1-dev 1024x1024 MMDiT self-attention: 57 layers x (24 heads x 128, 512 text + 4096 image tokens)",
                 layers=57, sets=57, H=24, D=128, S=4608, degrees={1: (1, 1), 2: (2, 1), 4: (4, 1), 8: (8, 1)}),
    "wan": dict(desc="Wan2.1-14B 81f 720x1280 self-attention: 40 layers x (40 heads x 128, 75,600 tokens)",
                layers=40, sets=2, H=40, D=128, S=75600, degrees={1: (1, 1), 2: (2, 1), 4: (4, 1), 8: (8, 1)}),
}


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


def flops_per_call(w):
    return 4.0 * w["S"] * w["S"] * w["H"] * w["D"]


# --------------------------------------------------------------------------------------------
# reference arm: the CPU restatement of the reference algorithm on the host cores
# --------------------------------------------------------------------------------------------
def run_reference(args, w, name):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch

    from oracle import usp_oracle as O

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    S, D = w["S"], w["D"]
    g = torch.Generator().manual_seed(0)

    def make(heads):
        return tuple(torch.randn(1, heads, S, D, generator=g) for _ in range(3))

    def one(qkv):
        t0 = time.perf_counter()
        O.attention_dense_torch_cpu(*qkv)
        return time.perf_counter() - t0

    # size the per-step sample (a number of heads of one layer) so that the whole run stays near 90 s
    t_head = one(make(1))
    budget = 90.0 / max(1, args.steps + args.warmup)
    heads = int(max(1, min(w["H"], budget / max(t_head, 1e-3))))
    qkv = make(heads)  # one input set, larger than any CPU cache (heads x 75,600 x 128 fp32 x 3)
    for _ in range(args.warmup):
        one(qkv)
    total = 0.0
    for _ in range(args.steps):
        total += one(qkv)
    fl = 4.0 * S * S * heads * D
    val = fl * args.steps / total / 1e12
    sample = (f"{heads} of {w['H']} heads of one layer, {S} tokens, fp32 torch CPU SDPA "
              f"(the reference's SDPA back-end body) on {cores} threads, per step")
    line = {
        "impl": "reference", "metric": "usp_attn_tflops", "value": val, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": total / args.steps * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": name, "desc": w["desc"]},
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------------
# our arm
# --------------------------------------------------------------------------------------------
def make_layer_inputs(torch, w, P, rank, layers, device, pinned=False):
    """``layers`` distinct input sets of local shards [1, H, S/P, D] bf16 (a step cycles through
    them layer by layer)."""
    S, H, D = w["S"], w["H"], w["D"]
    s = S // P
    out = []
    gg = torch.Generator(device=device)
    for layer in range(layers):
        qkv = []
        for i in range(3):
            # N(0,1) drawn on the device from a seed per (layer, tensor, rank); host sets are copies
            gg.manual_seed(1000003 * (layer + 1) + 1009 * i + rank)
            t = torch.randn(1, H, s, D, generator=gg, dtype=torch.float32, device=device).to(torch.bfloat16)
            if pinned:
                t = t.cpu().pin_memory()
            qkv.append(t)
        out.append(tuple(qkv))
    return out


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


def run_workload(torch, dist, xdit_b200, ops, name, w, args, device, rank, world, layers, with_e2e):
    U, R = w["degrees"][world]
    if getattr(args, "sp", None):
        U, R = (int(x) for x in args.sp.lower().split("x"))
        assert U * R == world, "--sp UxR must multiply to the number of GPUs"
    xdit_b200.init_sequence_parallel(U, R)
    P = U * R
    S = w["S"]
    assert S % P == 0
    nsets = max(1, min(layers, w["sets"]))
    inputs = make_layer_inputs(torch, w, P, rank, nsets, device)
    multi = world > 1

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
    }
    if with_e2e:
        host = make_layer_inputs(torch, w, P, rank, nsets, device, pinned=True)
        s = S // P
        host_out = [torch.empty(1, w["H"], s, w["D"], dtype=torch.bfloat16).pin_memory() for _ in range(nsets)]

        # The way a serving loop stages a layer's tensors: two device slots, the next layer's q/k/v
        # copied in on one side stream while this layer's USP call runs, the result copied out on
        # another.  Every byte still crosses PCIe inside the timed region, every step.
        cur = torch.cuda.current_stream(device)
        s_in, s_out = torch.cuda.Stream(device), torch.cuda.Stream(device)
        slots = [[torch.empty(1, w["H"], s, w["D"], dtype=torch.bfloat16, device=device) for _ in range(3)]
                 for _ in range(2)]
        ev_in = [torch.cuda.Event() for _ in range(2)]
        ev_done = [torch.cuda.Event() for _ in range(2)]

        def stage(layer):
            slot = layer & 1
            s_in.wait_event(ev_done[slot])  # the call that last read this slot has finished
            with torch.cuda.stream(s_in):
                for dst, src in zip(slots[slot], host[layer % nsets]):
                    dst.copy_(src, non_blocking=True)
                ev_in[slot].record(s_in)

        def step_e2e():
            for e in ev_done:
                e.record(cur)
            stage(0)
            for layer in range(layers):
                slot = layer & 1
                if layer + 1 < layers:
                    stage(layer + 1)
                cur.wait_event(ev_in[slot])
                out = xdit_b200.USP(*slots[slot])
                ev_done[slot].record(cur)
                s_out.wait_event(ev_done[slot])
                with torch.cuda.stream(s_out):
                    host_out[layer % nsets].copy_(out, non_blocking=True)
                out.record_stream(s_out)
            cur.wait_stream(s_out)  # the step ends when its last result is in host memory

        e2e_steps = max(1, min(args.steps, 2 if w["S"] > 20000 else 5))
        ms_e = timed_region(torch, dist, step_e2e, e2e_steps, 1, device, multi)
        bytes_in = 3 * layers * w["H"] * s * w["D"] * 2
        bytes_out = layers * w["H"] * s * w["D"] * 2
        res["e2e"] = {"value": fl_step * e2e_steps / (ms_e * 1e-3) / 1e12, "unit": "TFLOP/s",
                      "h2d_bytes_per_step": bytes_in, "d2h_bytes_per_step": bytes_out,
                      "ms_per_step": ms_e / e2e_steps, "steps": e2e_steps}
        del host, host_out
    del inputs
    torch.cuda.empty_cache()
    return res


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


# --------------------------------------------------------------------------------------------
# DiT step latency on random-init stand-ins of the named architectures (plain torch bf16 for
# everything but attention; no checkpoint or diffusers is available here)
# --------------------------------------------------------------------------------------------
def dit_step_latency(torch, dist, xdit_b200, kind, device, rank, world, reps=5, fused_prologue=True):
    """One transformer forward (= one denoising step) of a Flux.1-dev-shaped MMDiT or a
    Wan2.1-14B-shaped video DiT: QKV/out projections, MLPs and norms in torch bf16 with N(0, 0.02)
    weights, the sequence sharded over the ranks.  Self-attention from the projections on: with
    ``fused_prologue`` through ``xdit_b200.prologue.attention_from_projections`` (q/k RMS-norm, rotary
    embedding, head split and pack in one kernel), otherwise q/k RMS-norm and rotary embedding in
    torch and ``xdit_b200.USP``, the way the reference's processors are written.  Text cross-attention
    through ``xdit_b200.attention``.  Returns milliseconds (median)."""
    import torch.nn.functional as F

    from xdit_b200.prologue import attention_from_projections

    bf = torch.bfloat16
    w = WORKLOADS[kind]
    U, R = w["degrees"][world]
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

    def attn(q, k, v):  # [B, s, H, D] views of the projections -> [B, s, H*D]
        if fused_prologue:
            return attention_from_projections(q.reshape(1, s, hid), k.reshape(1, s, hid), v.reshape(1, s, hid), H,
                                              norm_q_weight=wq, norm_k_weight=wk, eps=1e-6, norm_per_head=per_head,
                                              rotary_emb=rotary)
        if per_head:
            q, k = F.rms_norm(q, (D,), wq, 1e-6), F.rms_norm(k, (D,), wk, 1e-6)
        else:
            q = F.rms_norm(q.reshape(1, s, hid), (hid,), wq, 1e-6).view(1, s, H, D)
            k = F.rms_norm(k.reshape(1, s, hid), (hid,), wk, 1e-6).view(1, s, H, D)
        o = xdit_b200.USP(rope(q).transpose(1, 2), rope(k).transpose(1, 2), v.transpose(1, 2))
        return o.transpose(1, 2).reshape(1, s, hid)

    x = torch.randn(1, s, hid, device=device, generator=g).to(bf)
    if kind == "flux":
        mlp = 4 * hid
        dbl = [dict(qkv=lin(hid, 3 * hid), proj=lin(hid, hid), up=lin(hid, mlp), down=lin(mlp, hid)) for _ in range(19)]
        sgl = [dict(l1=lin(hid, 3 * hid + mlp), l2=lin(hid + mlp, hid)) for _ in range(38)]

        def forward(x):
            # text and image tokens form one sharded sequence; a double block differs from a single
            # one by its separate attention/MLP projections (per-stream weights are applied to the
            # whole shard here: same flops and bytes per token)
            for b in dbl:
                h_ = F.layer_norm(x, (hid,))
                q, k, v = F.linear(h_, b["qkv"]).view(1, s, 3, H, D).unbind(2)
                x = x + F.linear(attn(q, k, v), b["proj"])
                x = x + F.linear(F.gelu(F.linear(F.layer_norm(x, (hid,)), b["up"]), approximate="tanh"), b["down"])
            for b in sgl:
                h_ = F.linear(F.layer_norm(x, (hid,)), b["l1"])
                q, k, v = h_[..., : 3 * hid].view(1, s, 3, H, D).unbind(2)
                x = x + F.linear(torch.cat([attn(q, k, v), F.gelu(h_[..., 3 * hid:], approximate="tanh")], -1), b["l2"])
            return x
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
                x = x + F.linear(attn(q, k, v), b["o"])
                h_ = F.layer_norm(x, (hid,))
                cq = F.linear(h_, b["cq"]).view(1, s, H, D).transpose(1, 2)
                ck = F.linear(ctx, b["ck"]).view(1, txt_len, H, D).transpose(1, 2)
                cv = F.linear(ctx, b["cv"]).view(1, txt_len, H, D).transpose(1, 2)
                x = x + F.linear(xdit_b200.attention(cq, ck, cv).transpose(1, 2).reshape(1, s, hid), b["co"])
                x = x + F.linear(F.gelu(F.linear(F.layer_norm(x, (hid,)), b["up"]), approximate="tanh"), b["down"])
            return x

    with torch.no_grad():
        for _ in range(2):
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
            "what": "one forward of a random-init stand-in (torch bf16 linears/norms/MLPs + xdit_b200 attention; "
                    + ("q/k norm + rotary embedding + head split fused with the pack" if fused_prologue
                       else "q/k norm and rotary embedding in torch, as the reference's processors do") + ")"}


def cpu_baseline(w):
    import torch

    from oracle import usp_oracle as O

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    S, D, heads = w["S"], w["D"], w["H"]
    if S > 20000:
        S, heads = 9450, 8  # a shard-sized sample: the full score matrix is too much for a bounded host run
    g = torch.Generator().manual_seed(0)
    total, fl, reps = 0.0, 0.0, 0
    q, k, v = (torch.randn(1, heads, S, D, generator=g) for _ in range(3))
    O.attention_dense_torch_cpu(q, k, v)  # warm-up
    t_end = time.perf_counter() + 12.0
    while time.perf_counter() < t_end and reps < 20:
        t0 = time.perf_counter()
        O.attention_dense_torch_cpu(q, k, v)
        total += time.perf_counter() - t0
        fl += 4.0 * S * S * heads * D
        reps += 1
    return {"value": fl / total / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": "port",
            "sample": f"{reps} x one layer call ({heads} heads, {S} tokens, fp32), torch CPU SDPA as the "
                      f"reference's SDPA back-end calls it, {cores} threads"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="wan", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-extra", action="store_true", help="skip the secondary workload and the CPU baseline")
    ap.add_argument("--layers", type=int, default=0, help="time only this many layers per step (profiling aid)")
    ap.add_argument("--dit", default="flux", choices=["none", "flux", "wan", "both"],
                    help="also time one DiT forward of a random-init stand-in of this architecture (extra.dit_step)")
    ap.add_argument("--sp", default=None, help="override the sequence-parallel degrees of the main workload: ULYSSESxRING, e.g. 2x4")
    ap.add_argument("--no-e2e", action="store_true", help="skip the end-to-end (host buffers) leg")
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
    main_res = run_workload(torch, dist, xdit_b200, ops, name, w, args, device, rank, world, w["layers"],
                            not args.no_e2e)
    extra = {}
    if not args.no_extra:
        other = "wan" if name == "flux" else "flux"
        wo = WORKLOADS[other]
        a2 = argparse.Namespace(steps=max(1, min(args.steps, 3)), warmup=3, graph=args.graph, sp=None)
        layers = 4 if other == "wan" else wo["layers"]
        try:
            r2 = run_workload(torch, dist, xdit_b200, ops, other, wo, a2, device, rank, world, layers, False)
            extra[other] = {
                "desc": wo["desc"], "layers_timed": layers, "ulysses": r2["U"], "ring": r2["R"],
                "cuda_graph": r2["cuda_graph"],
                "tflops_all_gpus": r2["tflops"], "tflops_per_gpu": r2["tflops"] / world,
                "ms_per_layer_call": r2["ms_per_step"] / layers,
                "frac_of_measured_bf16_burst_peak": r2["tflops"] / world / tf_peak,
            }
        except Exception as e:  # the secondary workload must not take the main line down
            extra[other] = {"error": repr(e)[:200]}
        if world == 1:
            try:
                extra["hbm_kernels"] = hbm_kernels(torch, ops, device, hbm_peak, peak_kind)
            except Exception as e:
                extra["hbm_kernels"] = {"error": repr(e)[:200]}
        if args.dit != "none":
            extra["dit_step"] = {}
            for kind in (("flux", "wan") if args.dit == "both" else (args.dit,)):
                try:
                    reps = 5 if kind == "flux" else 3
                    r_f = dit_step_latency(torch, dist, xdit_b200, kind, device, rank, world, reps=reps)
                    r_t = dit_step_latency(torch, dist, xdit_b200, kind, device, rank, world, reps=reps,
                                           fused_prologue=False)
                    r_f["ms_per_step_torch_prologue"] = r_t["ms_per_step"]
                    extra["dit_step"][kind] = r_f
                except Exception as e:
                    extra["dit_step"][kind] = {"error": repr(e)[:200]}
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
                "tokens": w["S"], "heads": w["H"],
                "head_dim": w["D"], "global_batch": 1,
                "l2": f"inputs larger than L2: {main_res['sets']} distinct q/k/v sets cycled layer by layer "
                      f"({main_res['sets'] * 3 * w['H'] * w['S'] * w['D'] * 2 / 1e9:.1f} GB over all ranks)",
            },
            "tflops_per_gpu": per_gpu_tf,
            "roofline": roofline(w, main_res, per_gpu_tf, kernel_ms, world, tf_peak, tf_sustained, peak_kind),
            "e2e": main_res.get("e2e"),
            "clocks": main_res["clocks"],
            "gpu_launches": main_res["launches"],
            "extra": extra,
        }
        if world == 1 and not args.no_extra:
            line["cpu_baseline"] = cpu_baseline(w)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
