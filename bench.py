#!/usr/bin/env python
"""Benchmark of the int4 dequant-matmul path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

One STEP is one pass of the hot path over a rotation of distinct weight sets (together larger than the
126 MB L2, so every launch streams its weights from HBM); the launches of a step are replayed from a CUDA
graph so host launch cost does not enter the device-timed number. Rank 0 prints one JSON line.

Workloads
  prefill_gemm_m512  X[512,2048] f16 times int4 W[8192,2048] (group 64, affine), f16 out. TFLOP/s. (default)
  decode_gemv        x[1,2048] times the same weight format, GB/s of algorithmic bytes.
  decode_layer_set   the 8B-class projections at M=1 (q,k,v,o,gate,up,down,lm_head), GB/s; decode_layer_set_m4: at M=4.
  shape:NxKxM[xf32][xq3]  one projection of any size (GB/s for M <= 8, TFLOP/s above; q3 = 3-bit codes): profiles, sweeps.

  layer_set_nshard   the same eight projections with their output rows sharded over the ranks and one all-gather
                     per projection (strong scaling, GB/s of the whole layer set); --m-rows 1|4
  moe_ep             35B-A3B-class MoE block (256 experts + shared, hidden 2048, ffn 512, top-8), experts sharded
                     over the ranks, all-to-all dispatch / combine (TFLOP/s); --tokens T per rank (--ep-scaling weak,
                     default) or in total (--ep-scaling strong)

With N > 1 the first three workloads run as independent replicas, one per rank, on their own weight sets (a single
GEMM / GEMV does not shard); value is the aggregate over ranks divided by the slowest rank's device time.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "int4 matmul HBM GB/s (decode M=1) and TFLOP/s (prefill M=512) vs roofline"
L2_BYTES = 126 * 1024 * 1024


BITS = 4   # code width of the timed workload: 3 for shape:...xq3, else 4


def algorithmic_bytes(N, K, M, bits=None, group=64, affine=True, out_bytes=2):
    bits = BITS if bits is None else bits
    """weights + scales (+ biases) + activations + outputs, each touched once."""
    return N * K * bits // 8 + (2 if affine else 1) * (N * K // group) * 2 + M * K * 2 + M * N * out_bytes


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return dict(hbm=d["hbm_gbs"], tf_burst=d["bf16_tflops"], tf_sustained=d.get("bf16_tflops_sustained"),
                    src="measured")
    return dict(hbm=6650.0, tf_burst=1590.0, tf_sustained=1400.0, src="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.rows, self.proc, self.index = [], None, index

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *a):
        if self.proc:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        ok = [r for r in self.rows if len(r) >= 8 and r[0].isdigit()]
        if not ok:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        reasons = set()
        for r in ok:
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median([int(r[0]) for r in ok])), "sm_max_mhz": float(ok[0][1]),
                "power_w_max": max(float(r[2]) for r in ok), "samples": len(ok), "reasons": sorted(reasons)}


# ---------------------------------------------------------------------------------------------------
def workload_shapes(name):
    """(label, N, K, M, out_f32) launches of one rotation element."""
    import zero_tvm_b200 as z
    if name == "prefill_gemm_m512":
        return [("W[8192,2048] M=512", 8192, 2048, 512, False)]
    if name == "decode_gemv":
        return [("W[8192,2048] M=1", 8192, 2048, 1, False)]
    if name in ("decode_layer_set", "decode_layer_set_m4"):
        M = 4 if name.endswith("_m4") else 1
        return [(n, N, K, M, f32) for n, N, K, f32 in z.synth.DENSE_LAYER_SET]
    if name.startswith("shape:"):      # shape:NxKxM (f16 out) or shape:NxKxMxf32 — any one projection, e.g. for profiling
        parts = name[6:].split("x")
        N, K, M = (int(v) for v in parts[:3])
        f32 = "f32" in parts[3:]
        global BITS
        BITS = 3 if "q3" in parts[3:] else 4
        return [(f"W{'3' if BITS == 3 else ''}[{N},{K}] M={M}", N, K, M, f32)]
    raise SystemExit(f"unknown workload {name}")


def make_sets(shapes, seed, torch, device):
    """Distinct weight sets until one rotation exceeds 4x L2 (codes random; scales/biases as the configs say)."""
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    per_set = sum(algorithmic_bytes(N, K, 1) for _, N, K, _, _ in shapes)
    R = max(2, int(np.ceil(4 * L2_BYTES / per_set)))
    sets = []
    for _ in range(R):
        one = []
        for _, N, K, M, f32 in shapes:
            W = torch.randint(-2**31, 2**31 - 1, (N, K * BITS // 32), dtype=torch.int32, device=device, generator=g)
            s = (torch.randn((N, K // 64), device=device, generator=g) * 0.01).abs().to(torch.float16)
            b = (torch.randn((N, K // 64), device=device, generator=g) * 0.05).to(torch.float16)
            y = torch.empty((M, N), dtype=torch.float32 if f32 else torch.float16, device=device)
            one.append((W, s, b, y))
        sets.append(one)
    return sets, R


def cpu_baseline(shapes, limit_s=12.0):
    """The oracle's reference-order CPU matmul (C, OpenMP, all host threads) on a bounded sample."""
    import zero_tvm_b200 as z
    from oracle import ztvm_oracle_c as zc
    zc.build()
    label, N, K, M, f32 = shapes[0]
    Ms = min(M, 16)
    p = z.synth.projection(N, K, M=Ms, seed=0)
    zc.gemv_ref(p["x"], p["W"], p["scales"], p["biases"], 64, out_f32=f32)  # warm
    t0, n = time.perf_counter(), 0
    while True:
        zc.gemv_ref(p["x"], p["W"], p["scales"], p["biases"], 64, out_f32=f32)
        n += 1
        dt = time.perf_counter() - t0
        if dt > limit_s or n >= 50:
            break
    per = dt / n
    return dict(seconds_per_sample=per, rows=Ms, N=N, K=K, cores=zc.num_threads(),
                sample=f"{n} x ({label.split()[0]} with M={Ms} of {M} rows), reference word order, C/OpenMP")


def run_reference_arm(args, rank):
    """The reference's CPU-side arithmetic for this path (its WGSL cannot run without WebGPU): the oracle's C
    restatement, all host threads, on a bounded sample of the same workload."""
    if rank != 0:
        return
    shapes = workload_shapes(args.workload)
    is_gemm = shapes[0][3] > 8
    vals = []
    for _ in range(max(1, args.steps)):
        cb = cpu_baseline(shapes, limit_s=max(2.0, 20.0 / max(1, args.steps)))
        label, N, K, M, f32 = shapes[0]
        if is_gemm:
            vals.append(2.0 * cb["rows"] * N * K / cb["seconds_per_sample"] / 1e12)
        else:
            vals.append(algorithmic_bytes(N, K, cb["rows"]) / cb["seconds_per_sample"] / 1e9)
    v = float(np.median(vals))
    unit = "TFLOP/s" if is_gemm else "GB/s"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": v, "unit": unit, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": cb["seconds_per_sample"] * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f16 x int4 -> f32 accumulate", "data": "synthetic",
        "config": {"workload": args.workload, "shape": shapes[0][0]},
        "cpu_baseline": {"value": v, "unit": unit, "cores": cb["cores"], "kind": "port", "sample": cb["sample"]},
        "e2e": {"value": v, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def run_sharded(args, rank, world, local):
    """Row-sharded layer set / expert-parallel MoE: the two forms of the path that shard (zero-tvm_b200/sharded.py)."""
    import torch
    import torch.distributed as dist
    import zero_tvm_b200 as z
    from zero_tvm_b200 import sharded
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    be = z.backend.CudaMatmulBackend(local)
    k = sharded.CudaKernels(be)
    g = torch.Generator(device=device)
    g.manual_seed(99)          # same weights on every rank, each keeps its shard

    def rand_w(lead, N, K):
        W = torch.randint(-2**31, 2**31 - 1, (*lead, N, K // 8), dtype=torch.int32, device=device, generator=g)
        sc = (torch.randn((*lead, N, K // 64), device=device, generator=g) * 0.01).abs().to(torch.float16)
        b = (torch.randn((*lead, N, K // 64), device=device, generator=g) * 0.05).to(torch.float16)
        return W, sc, b

    verified = None
    if args.workload == "layer_set_nshard":
        M = args.m_rows
        projs, xs, total_bytes = [], [], 0
        for name, N, K, f32 in z.synth.DENSE_LAYER_SET:
            W, sc, b = rand_w((), N, K)
            lo, hi = sharded.shard_rows(N, world, rank)
            projs.append(sharded.NShardedProjection(k, W[lo:hi].contiguous(), sc[lo:hi].contiguous(), b[lo:hi].contiguous(),
                                                    N, K, out_f32=f32, fused=args.nshard_gather == "fused", max_m=max(1, M)))
            xs.append(torch.randn((M, K), device=device, generator=g).to(torch.float16))
            total_bytes += algorithmic_bytes(N, K, M, out_bytes=4 if f32 else 2)
            if name == "k_proj" and rank == 0:
                from oracle import ztvm_oracle_c as zc
                y = projs[-1].forward(xs[-1], M)
                y64 = zc.matmul_f64(xs[-1].cpu().numpy(), W.cpu().numpy().view(np.uint32), sc.cpu().numpy(), b.cpu().numpy(), 64)
                fl = 1e-3 * float(np.sqrt(np.mean(y64 * y64)))
                err = float(np.max(np.abs(y.float().cpu().numpy() - y64) / np.maximum(np.abs(y64), fl)))
                verified = {"projection": name, "max_rel_err": err, "ok": bool(err <= 2e-3)}
            elif name == "k_proj":
                projs[-1].forward(xs[-1], M)

        def step():
            for pj, x in zip(projs, xs):
                pj.forward(x, M)
        units, unit, launches = total_bytes / 1e9, "GB/s", len(projs)
        cfg = {"workload": args.workload, "M": M, "shapes": [n for n, *_ in z.synth.DENSE_LAYER_SET],
               "parallelism": f"output rows / {world} + " + ("peer stores from the GEMV + barrier" if args.nshard_gather == "fused" and world > 1 else "all-gather"), "l2": "inputs larger than L2: 459 MB of weights per step"}
        bound, peak = "hbm", measured_peaks()["hbm"] * world
    else:
        E, top_k, d, ffn, T = 256, 8, 2048, 512, args.tokens
        epr = E // world
        sel = torch.tensor(list(range(rank * epr, (rank + 1) * epr)) + [E], device=device)
        stacks = []
        for N, K in ((ffn, d), (ffn, d), (d, ffn)):
            W, sc, b = rand_w((E + 1,), N, K)
            stacks.append((W[sel].contiguous(), sc[sel].contiguous(), b[sel].contiguous()))
            del W, sc, b
        moe = sharded.ExpertParallelMoE(k, *stacks, E=E, top_k=top_k, d=d, ffn=ffn)
        tl = T if args.ep_scaling == "weak" else max(1, T // world)   # weak: --tokens is per rank
        x = torch.randn((tl, d), device=device).to(torch.float16)
        logits = torch.randn((tl, E + 1), device=device)

        def step():
            moe.forward(x, logits)
        pairs = tl * world * (top_k + 1)
        units, unit, launches = pairs * 3 * 2.0 * ffn * d / 1e12, "TFLOP/s", 9
        cfg = {"workload": args.workload, "tokens": tl * world, "tokens_per_rank": tl, "ep_scaling": args.ep_scaling, "experts": E, "top_k": top_k, "hidden": d, "ffn": ffn,
               "parallelism": f"experts / {world} + all-to-all", "l2": "inputs larger than L2: 455 MB of expert weights"}
        bound, peak = "hbm", measured_peaks()["hbm"] * world
    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    # The row-sharded layer set is pure kernel launches (GEMV with peer stores + barrier kernel, or one GPU): replay it
    # from a CUDA graph so the host's launch cost does not enter the device-timed number. The NCCL and the MoE forms
    # need the host between launches (split sizes) and run eagerly.
    replay = None
    if args.workload == "layer_set_nshard" and (world == 1 or args.nshard_gather == "fused"):
        side = torch.cuda.Stream(device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            step(); step()                      # both output buffers seen once on the capture stream
            side.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                step(); step()                  # an even number: the double buffers end where they started
            side.synchronize()
        replay = graph
        cfg["launch"] = "CUDA graph of two steps"
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clocks:
        ev0.record()
        if replay is not None:
            for _ in range((args.steps + 1) // 2):
                replay.replay()
        else:
            for _ in range(args.steps):
                step()
        ev1.record()
        torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    ms = ev0.elapsed_time(ev1)
    if world > 1:
        t = torch.tensor([ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ms_per_step = ms / (2 * ((args.steps + 1) // 2) if replay is not None else args.steps)
    value = units / (ms_per_step * 1e-3)
    out = {"metric": METRIC, "value": value, "unit": unit, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
           "ms_per_step": ms_per_step, "higher_is_better": True,
           "scaling": "weak" if (args.workload == "moe_ep" and args.ep_scaling == "weak") else "strong", "vs_baseline": None,
           "dtype": "f16 x int4 -> f32 accumulate", "data": "synthetic", "config": cfg,
           "gpu_launches": int(args.steps * launches), "clocks": clocks.summary(), "verified": verified}
    if unit == "GB/s":
        out["roofline"] = {"bound": bound, "achieved": value, "peak": peak, "unit": "GB/s", "frac": value / peak,
                           "traffic": None, "peak_kind": "measured copy bandwidth x ranks"}
    if rank == 0:
        print(json.dumps(out))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def quick_device_rate(ctx, torch, device, z, workload, steps, warmup, seed=4321):
    """Device-timed rate of another workload, same method as the main one (rotating sets >= 4x L2, CUDA-graph replay,
    CUDA events on the launching stream): the decode half of the metric, reported beside the prefill GEMM."""
    shapes = workload_shapes(workload)
    sets, R = make_sets(shapes, seed, torch, device)
    xs = [torch.randn((M, K), device=device).to(torch.float16) for _, N, K, M, _ in shapes]
    descs = [z.MmDesc(K, N, M, 64, BITS, 1, int(f32)) for _, N, K, M, f32 in shapes]
    stream = torch.cuda.Stream(device)

    def one_pass():
        for one in sets:
            for (W, s, b, y), x, d in zip(one, xs, descs):
                ctx.int4_matmul(d, y, x, s, W, b, stream)

    with torch.cuda.stream(stream):
        one_pass()
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            one_pass()
        for _ in range(warmup):
            graph.replay()
        stream.synchronize()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record(stream)
        for _ in range(steps):
            graph.replay()
        ev1.record(stream)
        stream.synchronize()
    ms = ev0.elapsed_time(ev1) / steps
    nbytes = R * sum(algorithmic_bytes(N, K, M, out_bytes=4 if f32 else 2) for _, N, K, M, f32 in shapes)
    gbs = nbytes / (ms * 1e-3) / 1e9
    peak = measured_peaks()["hbm"]
    del sets, graph
    torch.cuda.empty_cache()
    return {"workload": workload, "value": gbs, "unit": "GB/s", "frac": gbs / peak, "peak": peak,
            "avg_launch_us": ms * 1e3 / (R * len(shapes)), "launches": int(steps * R * len(shapes))}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="prefill_gemm_m512")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-decode", action="store_true", help="default workload: skip the M = 1 rates reported beside it")
    ap.add_argument("--m-rows", type=int, default=1, help="activation rows of layer_set_nshard")
    ap.add_argument("--tokens", type=int, default=2048, help="tokens of moe_ep: per rank (weak) or whole job (strong)")
    ap.add_argument("--ep-scaling", default="weak", choices=["weak", "strong"])
    ap.add_argument("--nshard-gather", default="fused", choices=["fused", "nccl"],
                    help="layer_set_nshard: shards meet by peer stores from the GEMV + a barrier, or by NCCL all-gather")
    args = ap.parse_args()
    args.warmup = max(3, args.warmup)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference_arm(args, rank)
        return

    if args.workload in ("layer_set_nshard", "moe_ep"):
        run_sharded(args, rank, world, local)
        return

    import torch
    import zero_tvm_b200 as z
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)
    ctx = z.Context(local)

    shapes = workload_shapes(args.workload)
    if BITS != 4:
        args.no_cpu_baseline = True     # the CPU sample is the 4-bit reference-order matmul
    is_gemm = shapes[0][3] > 8
    sets, R = make_sets(shapes, 1234 + rank, torch, device)
    xs = [torch.randn((M, K), device=device).to(torch.float16) for _, N, K, M, _ in shapes]
    descs = [z.MmDesc(K, N, M, 64, BITS, 1, int(f32)) for _, N, K, M, f32 in shapes]
    stream = torch.cuda.Stream(device)

    def one_pass():
        for one in sets:
            for (W, s, b, y), x, d in zip(one, xs, descs):
                ctx.int4_matmul(d, y, x, s, W, b, stream)

    launches_per_matmul = [1 for _ in shapes]   # one kernel per matmul: GEMV for M <= 8, tcgen05 GEMM above
    with torch.cuda.stream(stream):
        one_pass()                      # sets function attributes outside of capture
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            one_pass()
        for _ in range(args.warmup):
            graph.replay()
        stream.synchronize()
        # A step is `passes` replays of the rotation, sized so that the timed region lasts long enough for the clock
        # sampler to see it (a single rotation of the GEMV workloads is a fraction of a millisecond).
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record(stream)
        graph.replay()
        ev1.record(stream)
        stream.synchronize()
        passes = int(min(256, max(1, np.ceil(12.0 / max(ev0.elapsed_time(ev1), 1e-3)))))
        if world > 1:
            pt = torch.tensor([passes], device=device)
            dist.all_reduce(pt, op=dist.ReduceOp.MAX)
            passes = int(pt.item())
            dist.barrier()
        torch.cuda.synchronize()
        with ClockSampler(local) as clocks:
            ev0.record(stream)
            for _ in range(args.steps * passes):
                graph.replay()
            ev1.record(stream)
            stream.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
    ms = ev0.elapsed_time(ev1)
    if world > 1:
        t = torch.tensor([ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ms_per_step = ms / args.steps
    R_rot = R
    R = R * passes                      # weight sets visited per step
    n_launch_step = R * sum(launches_per_matmul)

    flops_step = R * sum(2.0 * M * N * K for _, N, K, M, _ in shapes)
    bytes_step = R * sum(algorithmic_bytes(N, K, M, out_bytes=4 if f32 else 2) for _, N, K, M, f32 in shapes)
    peaks = measured_peaks()
    if is_gemm:
        value = world * flops_step / (ms_per_step * 1e-3) / 1e12
        unit = "TFLOP/s"
        peak = peaks["tf_sustained"] or peaks["tf_burst"]
        roof = {"bound": "tensor", "achieved": flops_step / (ms_per_step * 1e-3) / 1e12, "peak": peak,
                "unit": "TFLOP/s", "peak_kind": f"{peaks['src']} sustained bf16 (kernel timed inside a long step)"}
    else:
        value = world * bytes_step / (ms_per_step * 1e-3) / 1e9
        unit = "GB/s"
        roof = {"bound": "hbm", "achieved": bytes_step / (ms_per_step * 1e-3) / 1e9, "peak": peaks["hbm"],
                "unit": "GB/s", "peak_kind": f"{peaks['src']} copy bandwidth"}
    roof["frac"] = roof["achieved"] / roof["peak"]
    roof["traffic"] = None
    roof["avg_launch_us"] = ms_per_step * 1e3 / (R * len(shapes))

    # ---- correctness of the timed configuration (a skipped dispatch always looks like a fast one) ----
    W, s, b, y = sets[0][0]
    label, N, K, M, f32 = shapes[0]
    torch.cuda.synchronize()
    yh = y.float().cpu().numpy()
    verified = None
    if rank == 0:
        from oracle import ztvm_oracle_c as zc
        zc.build()
        rows = min(M, 4)
        y64 = zc.matmul_f64(xs[0][:rows].cpu().numpy(), W.cpu().numpy().view(np.uint32), s.cpu().numpy(),
                            b.cpu().numpy(), 64, BITS, w16=is_gemm)
        floor = (1e-2 if is_gemm else 1e-3) * float(np.sqrt(np.mean(y64 * y64)))
        err = float(np.max(np.abs(yh[:rows] - y64) / np.maximum(np.abs(y64), floor)))
        verified = {"rows": rows, "max_rel_err": err, "ok": bool(err <= 2e-3 and np.abs(yh).max() > 0)}

    # ---- end to end through the host-buffer entry point: pinned x in, y out, every launch ----
    d0 = descs[0]
    xh = torch.randn((M, K)).to(torch.float16).pin_memory()
    yh_t = torch.empty((M, N), dtype=torch.float32 if f32 else torch.float16).pin_memory()
    e2e_sets = [one[0] for one in sets]
    for (W, s, b, _y) in e2e_sets[:3]:
        ctx.int4_matmul_host(d0, yh_t, xh, s, W, b)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e2e_steps = max(1, min(args.steps, 5))
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        for (W, s, b, _y) in e2e_sets:
            ctx.int4_matmul_host(d0, yh_t, xh, s, W, b)
    torch.cuda.synchronize()
    e2e_s = (time.perf_counter() - t0) / e2e_steps
    if world > 1:
        t = torch.tensor([e2e_s], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    if is_gemm:
        e2e_val = world * R_rot * 2.0 * M * N * K / e2e_s / 1e12
    else:
        e2e_val = world * R_rot * algorithmic_bytes(N, K, M, out_bytes=4 if f32 else 2) / e2e_s / 1e9
    e2e = {"value": e2e_val, "unit": unit, "h2d_bytes_per_step": R_rot * M * K * 2,
           "d2h_bytes_per_step": R_rot * M * N * (4 if f32 else 2), "launches_per_step": R_rot,
           "what": "ztvm_int4_matmul_host per launch: pinned x -> device, kernel, y -> host, sync; weights resident"}

    # ---- the decode half of the metric (M = 1, GB/s against the measured copy bandwidth), rank 0 of the default run ----
    decode = None
    if args.workload == "prefill_gemm_m512" and rank == 0 and not args.no_decode:
        del sets, graph, e2e_sets
        torch.cuda.empty_cache()
        decode = [quick_device_rate(ctx, torch, device, z, w, max(3, args.steps // 2), args.warmup)
                  for w in ("decode_gemv", "decode_layer_set", "shape:151936x4096x1xf32")]

    out = {
        "metric": METRIC, "value": value, "unit": unit, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f16 x int4 -> f32 accumulate", "data": "synthetic",
        "config": {"workload": args.workload, "shapes": [s_[0] for s_ in shapes], "group": 64, "bits": BITS,
                   "rotation_sets": R_rot, "passes_per_step": passes, "rotation_bytes": int(bytes_step // passes),
                   "l2": "inputs larger than L2: weight sets rotate, 4x L2 per step",
                   "parallelism": "replicas" if world > 1 else "single"},
        "roofline": roof, "e2e": e2e, "gpu_launches": int(args.steps * n_launch_step),
        "clocks": clocks.summary(), "verified": verified,
        "decode": decode,
    }
    if rank == 0:
        if not args.no_cpu_baseline:
            cb = cpu_baseline(shapes)
            if is_gemm:
                v = 2.0 * cb["rows"] * cb["N"] * cb["K"] / cb["seconds_per_sample"] / 1e12
            else:
                v = algorithmic_bytes(cb["N"], cb["K"], cb["rows"]) / cb["seconds_per_sample"] / 1e9
            out["cpu_baseline"] = {"value": v, "unit": unit, "cores": cb["cores"], "kind": "port", "sample": cb["sample"]}
        print(json.dumps(out))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
