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
                     over the ranks, dispatch / combine between them (TFLOP/s); --tokens T per rank (--ep-scaling weak,
                     default) or in total (--ep-scaling strong)

With N > 1 the first three workloads run as independent replicas, one per rank, on their own weight sets (a single
GEMM / GEMV does not shard); value is the aggregate over ranks divided by the slowest rank's device time. The default
line also carries `sharded`: the two forms of the path that DO shard (row-sharded layer set, expert-parallel MoE),
measured in the same process group at every N, each with its own roofline and a check against the oracle.
"""
from __future__ import annotations

import os
import sys

# The CPU arm uses every host core. A launcher that starts one process per GPU usually pins OMP_NUM_THREADS to 1 in
# each of them; only rank 0 runs the CPU arm, so it takes the machine (must happen before numpy loads its BLAS).
if "reference" in sys.argv[1:] and any(a.startswith("--impl") for a in sys.argv[1:]):
    for _v in ("OMP_NUM_THREADS", "OPENBLAS_NUM_THREADS", "MKL_NUM_THREADS"):
        os.environ[_v] = str(os.cpu_count() or 1)

import argparse  # noqa: E402
import json  # noqa: E402
import subprocess  # noqa: E402
import threading  # noqa: E402
import time  # noqa: E402

import numpy as np  # noqa: E402

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "int4 matmul HBM GB/s (decode M=1) and TFLOP/s (prefill M=512) vs roofline"
L2_BYTES = 126 * 1024 * 1024
NVLINK_GBS = 770.0      # measured peer copy per direction per GPU on this pool (900 nominal)
DTYPE = "f16 x int4 -> f32 accumulate"

BITS = 4   # code width of the timed workload: 3 for shape:...xq3, else 4

# DRAM bytes per launch of the dominant kernel (dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture; the
# summaries under profiles/ hold the captures): workload -> (bytes, where from)
TRAFFIC = {
    "prefill_gemm_m512": (11.58e6, "profiles/gemm_w4_m512_8192x2048.md: the f16 output is still in L2 when the launch ends"),
    "shape:151936x4096x1xf32": (354.2e6, "profiles/gemv_tc_m1_151936x4096.md"),
}


def algorithmic_bytes(N, K, M, bits=None, group=64, affine=True, out_bytes=2):
    """weights + scales (+ biases) + activations + outputs, each touched once."""
    bits = BITS if bits is None else bits
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
        self.rows, self.proc, self.index, self.skip = [], None, index, 0

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
            # nvidia-smi takes its time to produce the first row (seconds when eight ranks start one each): the timed
            # region begins only once sampling is live, and rows from before it are not counted
            t0 = time.perf_counter()
            while not self.rows and time.perf_counter() - t0 < 8.0 and self.proc.poll() is None:
                time.sleep(0.01)
            self.skip = len(self.rows)
        except OSError:
            self.proc = None
        return self

    def mark(self):
        """The timed region starts now: rows read so far do not count."""
        self.skip = len(self.rows)

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
        ok = [r for r in self.rows[self.skip:] if len(r) >= 8 and r[0].isdigit()]
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
    global BITS
    BITS = 4
    if name == "prefill_gemm_m512":
        return [("W[8192,2048] M=512", 8192, 2048, 512, False)]
    if name == "decode_gemv":
        return [("W[8192,2048] M=1", 8192, 2048, 1, False)]
    if name in ("decode_layer_set", "decode_layer_set_m4"):
        M = 4 if name.endswith("_m4") else 1
        return [(n, N, K, M, f32) for n, N, K, f32 in z.synth.DENSE_LAYER_SET]
    if name in ("decode_layer_set_fused", ):      # as the engine dispatches them: q|k|v and gate|up as one projection each
        return [(n, N, K, 1, f32) for n, N, K, f32 in z.synth.DENSE_LAYER_SET_FUSED]
    if name.startswith("shape:"):      # shape:NxKxM (f16 out) or shape:NxKxMxf32 — any one projection, e.g. for profiling
        parts = name[6:].split("x")
        N, K, M = (int(v) for v in parts[:3])
        f32 = "f32" in parts[3:]
        BITS = 3 if "q3" in parts[3:] else 4
        return [(f"W{'3' if BITS == 3 else ''}[{N},{K}] M={M}", N, K, M, f32)]
    raise SystemExit(f"unknown workload {name}")


def config_for(workload, shapes, world):
    """The workload description both arms print (the same dict, so the two lines can be matched)."""
    return {"workload": workload, "shapes": [s_[0] for s_ in shapes], "group": 64, "bits": BITS,
            "l2": "inputs larger than L2: distinct weight sets rotate, 4x L2 per step",
            "parallelism": "replicas" if world > 1 else "single"}


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


# ---- CPU arms -----------------------------------------------------------------------------------------------------
def cpu_port(shapes, limit_s=12.0):
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
    return dict(seconds_per_sample=per, rows=Ms, N=N, K=K, cores=zc.num_threads(), kind="port",
                sample=f"{n} x ({label.split()[0]} with M={Ms} of {M} rows), reference word order, C/OpenMP")


def cpu_reference(shapes, steps, warmup):
    """The reference project's own CPU code for this path: its numpy `dequant_from` (compiled into oracle/_ref/ from
    scripts/make-dsv2-layer-ref.py:102-116) followed by a float32 x @ W.T, the way its reference scripts multiply.
    One step = the WHOLE first matmul of the workload (all M rows), dequant and matmul timed separately.
    Returns None when oracle/_ref/ is not there."""
    from oracle.make_ref import load_dequant_from
    dq = load_dequant_from()
    if dq is None or BITS != 4:
        return None
    import zero_tvm_b200 as z
    label, N, K, M, f32 = shapes[0]
    p = z.synth.projection(N, K, M=M, seed=0)
    x32 = p["x"].astype(np.float32)
    t_dq, t_mm = [], []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        Wd = dq(p["W"], p["scales"], p["biases"], group=64, bits=4)
        t1 = time.perf_counter()
        y = x32 @ Wd.T
        t2 = time.perf_counter()
        if i >= warmup:
            t_dq.append(t1 - t0)
            t_mm.append(t2 - t1)
    assert y.shape == (M, N) and np.isfinite(y).all()
    try:
        import threadpoolctl
        blas = max([i.get("num_threads", 1) for i in threadpoolctl.threadpool_info()] or [1])
    except Exception:
        blas = os.cpu_count() or 1
    return dict(seconds_per_sample=float(np.median(t_dq) + np.median(t_mm)), dequant_s=float(np.median(t_dq)),
                matmul_s=float(np.median(t_mm)), rows=M, N=N, K=K, cores=blas, host_cores=os.cpu_count(), kind="reference",
                step_seconds=[a + b for a, b in zip(t_dq, t_mm)],
                sample=f"{steps} x the whole {label}: the reference's numpy dequant_from ({dq.reference_location}; one thread), "
                       f"then float32 x @ W.T on {blas} BLAS threads")


def rate_of(cb, shapes):
    label, N, K, M, f32 = shapes[0]
    if M > 8:
        return 2.0 * cb["rows"] * cb["N"] * cb["K"] / cb["seconds_per_sample"] / 1e12, "TFLOP/s"
    return algorithmic_bytes(cb["N"], cb["K"], cb["rows"], out_bytes=4 if f32 else 2) / cb["seconds_per_sample"] / 1e9, "GB/s"


def run_reference_arm(args, rank, world):
    """The reference's CPU-side code for this path (its WGSL cannot run without WebGPU), all host cores, rank 0 only."""
    if rank != 0:
        return
    shapes = workload_shapes(args.workload)
    cb = cpu_reference(shapes, max(1, args.steps), max(0, min(args.warmup, 2)))
    if cb is None:      # oracle/_ref/ missing: the oracle's C restatement of the reference word order
        cb = cpu_port(shapes, limit_s=20.0)
    v, unit = rate_of(cb, shapes)
    extra = {k: cb[k] for k in ("dequant_s", "matmul_s", "host_cores") if k in cb}
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": v, "unit": unit, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": cb["seconds_per_sample"] * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": DTYPE, "data": "synthetic",
        "config": config_for(args.workload, shapes, world),
        "cpu_baseline": {"value": v, "unit": unit, "cores": cb["cores"], "kind": cb["kind"], "sample": cb["sample"], **extra},
        "e2e": {"value": v, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ---- the forms that shard -----------------------------------------------------------------------------------------
class ShardedBench:
    """Row-sharded layer set and expert-parallel MoE block, measured in the caller's process group."""

    def __init__(self, torch, dist, z, rank, world, local, steps, warmup):
        from zero_tvm_b200 import sharded
        self.torch, self.dist, self.z, self.sharded = torch, dist, z, sharded
        self.rank, self.world, self.local = rank, world, local
        self.steps, self.warmup = max(4, steps), max(3, warmup)
        self.device = torch.device("cuda", local)
        self.be = z.backend.CudaMatmulBackend(local)
        self.k = sharded.CudaKernels(self.be)
        self.peaks = measured_peaks()

    def close(self):
        self.be.close()

    def _rand_w(self, g, lead, N, K):
        torch, device = self.torch, self.device
        W = torch.randint(-2**31, 2**31 - 1, (*lead, N, K // 8), dtype=torch.int32, device=device, generator=g)
        sc = (torch.randn((*lead, N, K // 64), device=device, generator=g) * 0.01).abs().to(torch.float16)
        b = (torch.randn((*lead, N, K // 64), device=device, generator=g) * 0.05).to(torch.float16)
        return W, sc, b

    def _time(self, step, graph_steps=0):
        """Device time per step, max over ranks. graph_steps > 0: replay a CUDA graph holding that many steps."""
        torch, dist, world = self.torch, self.dist, self.world
        for _ in range(self.warmup):
            step()
        torch.cuda.synchronize()
        replay, per_replay = None, 1
        if graph_steps:
            side = torch.cuda.Stream(self.device)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for _ in range(graph_steps):
                    step()
                side.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=side):
                    for _ in range(graph_steps):
                        step()
                side.synchronize()
            replay, per_replay = graph, graph_steps
            for _ in range(2):
                replay.replay()
            torch.cuda.synchronize()
        n = -(-self.steps // per_replay)
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler(self.local) as clocks:      # sampling is live when this returns; the ranks meet after that
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            clocks.mark()
            ev0.record()
            for _ in range(n):
                if replay is not None:
                    replay.replay()
                else:
                    step()
            ev1.record()
            torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        ms = ev0.elapsed_time(ev1)
        if world > 1:
            t = torch.tensor([ms], device=self.device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms / (n * per_replay), clocks.summary(), ("CUDA graph of %d steps" % per_replay if replay is not None else "eager")

    # -- output rows of the dense layer set over the ranks ---------------------------------------------------------
    def layer_set(self, M, gather):
        torch, z, sharded, world, rank = self.torch, self.z, self.sharded, self.world, self.rank
        g = torch.Generator(device=self.device)
        g.manual_seed(99)          # same weights on every rank, each keeps its shard
        fused = gather == "fused"
        projs, xs, total_bytes, verified = [], [], 0, None
        for name, N, K, f32 in z.synth.DENSE_LAYER_SET:
            W, sc, b = self._rand_w(g, (), N, K)
            lo, hi = sharded.shard_rows(N, world, rank)
            pj = sharded.NShardedProjection(self.k, W[lo:hi].contiguous(), sc[lo:hi].contiguous(), b[lo:hi].contiguous(),
                                            N, K, out_f32=f32, fused=fused, max_m=max(1, M))
            x = torch.randn((M, K), device=self.device, generator=g).to(torch.float16)
            projs.append(pj)
            xs.append(x)
            total_bytes += algorithmic_bytes(N, K, M, bits=4, out_bytes=4 if f32 else 2)
            if name == "k_proj":      # one projection of the timed configuration against the oracle, on every rank's copy
                y = pj.forward(x, M)
                torch.cuda.synchronize()
                if rank == 0:
                    from oracle import ztvm_oracle as zo, ztvm_oracle_c as zc
                    y64 = zc.matmul_f64(x.cpu().numpy(), W.cpu().numpy().view(np.uint32), sc.cpu().numpy(), b.cpu().numpy(), 64)
                    got = y.float().cpu().numpy()
                    err = zo.rel_err_scaled(got, y64, 1e-3)
                    verified = {"projection": name, "max_rel_err": err, "max_rel_err_pure": zo.rel_err(got, y64),
                                "ok": bool(err <= 2e-3 and np.abs(got).max() > 0)}
            del W, sc, b

        def step():
            for pj, x in zip(projs, xs):
                pj.forward(x, M)
        graph_ok = world == 1 or fused      # the NCCL form runs eagerly (eight small collectives per step)
        ms, clocks, how = self._time(step, graph_steps=3 if graph_ok and fused and world > 1 else (2 if graph_ok else 0))
        gbs = total_bytes / (ms * 1e-3) / 1e9
        # bound: every rank streams its 1/world of the weights; each output row crosses NVLink to world - 1 peers
        out_bytes = sum(M * N * (4 if f32 else 2) for _, N, K, f32 in z.synth.DENSE_LAYER_SET)
        t_hbm = total_bytes / world / (self.peaks["hbm"] * 1e9)
        t_nv = out_bytes * (world - 1) / world / (NVLINK_GBS * 1e9) if world > 1 else 0.0
        t_roof = max(t_hbm, t_nv)
        return {"workload": "layer_set_nshard", "M": M, "gather": ("peer stores from the GEMV + barrier" if fused else "NCCL all-gather") if world > 1 else "none (one rank)",
                "scaling": "strong", "ms_per_step": ms, "value": gbs, "unit": "GB/s", "launch": how,
                "roofline": {"bound": "hbm" if t_hbm >= t_nv else "nvlink", "achieved": gbs, "peak": self.peaks["hbm"] * world,
                             "unit": "GB/s", "frac": t_roof / (ms * 1e-3), "roof_us": t_roof * 1e6, "traffic": None,
                             "peak_kind": f"{self.peaks['src']} copy bandwidth x ranks; NVLink {NVLINK_GBS:.0f} GB/s per direction"},
                "clocks": clocks, "verified": verified}

    # -- experts over the ranks ---------------------------------------------------------------------------------------
    def moe_ep(self, tokens, scaling, one_call=False):
        torch, sharded, world, rank = self.torch, self.sharded, self.world, self.rank
        E, top_k, d, ffn = 256, 8, 2048, 512
        epr = E // world
        g = torch.Generator(device=self.device)
        g.manual_seed(77)
        sel = torch.tensor(list(range(rank * epr, (rank + 1) * epr)) + [E], device=self.device)
        stacks, full = [], []
        for N, K in ((ffn, d), (ffn, d), (d, ffn)):
            W, sc, b = self._rand_w(g, (E + 1,), N, K)
            stacks.append((W[sel].contiguous(), sc[sel].contiguous(), b[sel].contiguous()))
            full.append((W, sc, b) if rank == 0 else None)
            del W, sc, b
        moe = sharded.ExpertParallelMoE(self.k, *stacks, E=E, top_k=top_k, d=d, ffn=ffn, max_tokens=None, one_call=one_call)
        tl = tokens if scaling == "weak" else max(1, tokens // world)
        # the same token stream on every rank; each takes its slice (so rank 0 can check its slice against the oracle)
        gx = torch.Generator(device=self.device)
        gx.manual_seed(1234)
        x_all = torch.randn((tl * world, d), device=self.device, generator=gx).to(torch.float16)
        l_all = torch.randn((tl * world, E + 1), device=self.device, generator=gx)
        x, logits = x_all[rank * tl:(rank + 1) * tl].contiguous(), l_all[rank * tl:(rank + 1) * tl].contiguous()
        del x_all, l_all

        out = moe.forward(x, logits)
        torch.cuda.synchronize()
        verified = None
        if rank == 0:       # a sample of this rank's tokens through the oracle's whole block (f16 stores where the engine has them)
            from oracle import ztvm_oracle as zo
            ns = min(tl, 6)
            fw = [tuple(a.cpu().numpy().view(np.uint32) if a.dtype == torch.int32 else a.cpu().numpy() for a in st) for st in full]
            ref = zo.moe_block(x[:ns].cpu().numpy(), logits[:ns].cpu().numpy(), fw[0], fw[1], fw[2], E, top_k, ffn)["y"]
            got = out[:ns].float().cpu().numpy()
            ref64 = ref.astype(np.float64)
            err = float(np.abs(got - ref64).max() / np.abs(ref64).max())
            verified = {"tokens_checked": ns, "max_err_over_max_ref": err, "max_rel_err_pure": zo.rel_err(got, ref64),
                        "tolerance": 5e-3, "note": "whole block (router, three chained expert matmuls with f16 stores between, "
                        "combine) against the oracle's block; the reference's own whole-block bound, max|y - ref| <= 0.005 max|ref|",
                        "ok": bool(err <= 5e-3 and np.abs(got).max() > 0)}
            del fw
        del full

        def step():
            moe.forward(x, logits)
        ms, clocks, how = self._time(step, graph_steps=2 if moe.capturable else 0)
        T_total = tl * world
        pairs = T_total * (top_k + 1)
        flops = pairs * 3 * 2.0 * ffn * d
        tf = flops / (ms * 1e-3) / 1e12
        per_expert = 3 * (ffn * d // 2 + 2 * (ffn * d // 64) * 2)
        act_experts = min(E, T_total * top_k)
        w_bytes_rank = (act_experts / world + 1) * per_expert
        t_hbm = w_bytes_rank / (self.peaks["hbm"] * 1e9)
        t_tc = flops / world / (self.peaks["tf_burst"] * 1e12)
        # rows that leave a rank: (world-1)/world of its routed pairs, x out (d f16) and y back (d f16), per direction
        t_nv = (tl * top_k * (world - 1) / world) * d * 2 / (NVLINK_GBS * 1e9) if world > 1 else 0.0
        t_roof = max(t_hbm, t_tc, t_nv)
        bound = "hbm" if t_roof == t_hbm else "tensor" if t_roof == t_tc else "nvlink"
        return {"workload": "moe_ep", "tokens": T_total, "tokens_per_rank": tl, "scaling": scaling, "experts": E, "top_k": top_k,
                "hidden": d, "ffn": ffn, "ms_per_step": ms, "value": tf, "unit": "TFLOP/s", "launch": how,
                "form": moe.form + (" (one ztvm_moe_ffn_ep call per step, the library's device-side barrier)" if moe.one_call else ""),
                "roofline": {"bound": bound, "achieved": tf, "peak": self.peaks["tf_burst"] * world, "unit": "TFLOP/s",
                             "frac": t_roof / (ms * 1e-3), "roof_us": t_roof * 1e6,
                             "hbm_us": t_hbm * 1e6, "tensor_us": t_tc * 1e6, "nvlink_us": t_nv * 1e6, "traffic": None,
                             "peak_kind": f"max of weights / {self.peaks['src']} copy bandwidth, flops / {self.peaks['src']} burst bf16, "
                                          f"rows over NVLink at {NVLINK_GBS:.0f} GB/s per direction; per rank"},
                "clocks": clocks, "verified": verified}


def run_sharded_only(args, rank, world, local):
    """--workload layer_set_nshard | moe_ep: one sharded form as the whole line."""
    import torch
    import torch.distributed as dist
    import zero_tvm_b200 as z
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    sb = ShardedBench(torch, dist, z, rank, world, local, args.steps, args.warmup)
    if args.workload == "layer_set_nshard":
        r = sb.layer_set(args.m_rows, args.nshard_gather)
    else:
        r = sb.moe_ep(args.tokens, args.ep_scaling)
    out = {"metric": METRIC, "value": r["value"], "unit": r["unit"], "n_gpus": world, "steps": args.steps,
           "warmup": args.warmup, "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": r["scaling"],
           "vs_baseline": None, "dtype": DTYPE, "data": "synthetic",
           "config": {k: v for k, v in r.items() if k not in ("roofline", "clocks", "verified", "value", "unit", "ms_per_step")},
           "roofline": r["roofline"], "gpu_launches": None, "clocks": r["clocks"], "verified": r["verified"]}
    if rank == 0:
        print(json.dumps(out))
    sb.close()
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
    # the timed configuration's first projection against the oracle (a skipped launch always looks like a fast one)
    from oracle import ztvm_oracle as zo, ztvm_oracle_c as zc
    W, s, b, y = sets[0][0]
    stream.synchronize()
    y64 = zc.matmul_f64(xs[0].cpu().numpy(), W.cpu().numpy().view(np.uint32), s.cpu().numpy(), b.cpu().numpy(), 64, BITS)
    got = y.float().cpu().numpy()
    err = zo.rel_err_scaled(got, y64, 1e-3)
    del sets, graph
    torch.cuda.empty_cache()
    return {"workload": workload, "value": gbs, "unit": "GB/s", "frac": gbs / peak, "peak": peak,
            "avg_launch_us": ms * 1e3 / (R * len(shapes)), "launches": int(steps * R * len(shapes)),
            "traffic": TRAFFIC.get(workload, (None, None))[0],
            "verified": {"max_rel_err": err, "max_rel_err_pure": zo.rel_err(got, y64), "ok": bool(err <= 2e-3 and np.abs(got).max() > 0)}}


def fused_ffn_rate(ctx, torch, device, z, steps, warmup, ffn=12288, K=4096, seed=777):
    """FFN front half of the dense decode layer (gate and up over hidden 4096 -> 12288, SiLU * up) as ONE call of
    ztvm_fused_ffn against the engine's affine path (the [2 ffn, K] matmul, then silu_mul): same method as the other
    decode rates (rotating weight sets >= 4x L2, graph replay, events on the launching stream), verified against the oracle."""
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    N = 2 * ffn
    per_set = algorithmic_bytes(N, K, 1)
    R = max(2, int(np.ceil(4 * L2_BYTES / per_set)))
    sets = []
    for _ in range(R):
        W = torch.randint(-2**31, 2**31 - 1, (N, K // 8), dtype=torch.int32, device=device, generator=g)
        s = (torch.randn((N, K // 64), device=device, generator=g) * 0.01).abs().to(torch.float16)
        b = (torch.randn((N, K // 64), device=device, generator=g) * 0.05).to(torch.float16)
        sets.append((W, s, b))
    x = torch.randn((1, K), device=device).to(torch.float16)
    h = torch.empty((1, ffn), dtype=torch.float16, device=device)
    gu = torch.empty((1, N), dtype=torch.float16, device=device)
    stream = torch.cuda.Stream(device)
    d_f, d_u = z.MmDesc(K, ffn, 1, 64, 4, 1, 0), z.MmDesc(K, N, 1, 64, 4, 1, 0)

    def fused():
        for W, s, b in sets:
            ctx.fused_ffn(d_f, h, x, s, W, b, stream)

    def unfused():
        for W, s, b in sets:
            ctx.int4_matmul(d_u, gu, x, s, W, b, stream)
            ctx.silu_mul(1, ffn, h, gu, stream)

    out = {}
    with torch.cuda.stream(stream):
        for name, fn in (("fused", fused), ("unfused", unfused)):
            fn()
            stream.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                fn()
            for _ in range(warmup):
                graph.replay()
            stream.synchronize()
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ev0.record(stream)
            for _ in range(steps):
                graph.replay()
            ev1.record(stream)
            stream.synchronize()
            out[name] = ev0.elapsed_time(ev1) * 1e3 / (steps * R)      # us per FFN front half
            del graph
    from oracle import ztvm_oracle as zo
    W, s, b = sets[-1]
    with torch.cuda.stream(stream):
        ctx.fused_ffn(d_f, h, x, s, W, b, stream)
        stream.synchronize()
    rows = slice(0, 256)          # the anchor over a slice of the outputs (gate rows 0..255 and their up rows)
    Wn, sn, bn = (t.cpu().numpy() for t in (W, s, b))
    sel = np.r_[0:256, ffn:ffn + 256]
    ref = zo.fused_ffn_f64(x.cpu().numpy(), Wn[sel].view(np.uint32), sn[sel], bn[sel], 256)
    got = h[:, rows].float().cpu().numpy()
    err = zo.rel_err_scaled(got, ref, 1e-3)
    peak = measured_peaks()["hbm"]
    nbytes = per_set - N * 2 + ffn * 2          # the fused call writes ffn outputs, not 2 ffn
    del sets
    torch.cuda.empty_cache()
    return {"workload": "ffn_gate_up_silu_m1", "value": nbytes / (out["fused"] * 1e-6) / 1e9, "unit": "GB/s",
            "frac": nbytes / (out["fused"] * 1e-6) / 1e9 / peak, "peak": peak, "avg_launch_us": out["fused"], "launches": int(steps * R),
            "unfused_us": out["unfused"], "unfused_launches_per_call": 2, "traffic": None,
            "verified": {"max_rel_err": err, "max_rel_err_pure": zo.rel_err(got, ref), "ok": bool(err <= 2e-3 and np.abs(got).max() > 0)}}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="prefill_gemm_m512")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-decode", action="store_true", help="default workload: skip the M = 1 rates reported beside it")
    ap.add_argument("--no-sharded", action="store_true", help="default workload: skip the sharded forms reported beside it")
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
        run_reference_arm(args, rank, world)
        return

    if args.workload in ("layer_set_nshard", "moe_ep"):
        run_sharded_only(args, rank, world, local)
        return

    import torch
    import zero_tvm_b200 as z
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)
    ctx = z.Context(local)

    shapes = workload_shapes(args.workload)
    if BITS != 4:
        args.no_cpu_baseline = True     # the CPU sample is the 4-bit reference-order matmul
    is_gemm = shapes[0][3] > 16      # up to 16 rows the library runs GEMV slabs (f32 weights)
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
        with ClockSampler(local) as clocks:      # sampling is live when this returns; the ranks meet after that
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            clocks.mark()
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
        # the timed region is a fraction of a second at near-boost clocks: the burst figure is the fair denominator
        # (the sustained one, taken over seconds under the power cap, is given beside it)
        value = world * flops_step / (ms_per_step * 1e-3) / 1e12
        unit = "TFLOP/s"
        ach = flops_step / (ms_per_step * 1e-3) / 1e12
        roof = {"bound": "tensor", "achieved": ach, "peak": peaks["tf_burst"], "unit": "TFLOP/s",
                "peak_kind": f"{peaks['src']} burst bf16", "peak_sustained": peaks["tf_sustained"],
                "frac_of_sustained": ach / peaks["tf_sustained"] if peaks["tf_sustained"] else None}
    else:
        value = world * bytes_step / (ms_per_step * 1e-3) / 1e9
        unit = "GB/s"
        roof = {"bound": "hbm", "achieved": bytes_step / (ms_per_step * 1e-3) / 1e9, "peak": peaks["hbm"],
                "unit": "GB/s", "peak_kind": f"{peaks['src']} copy bandwidth"}
    roof["frac"] = roof["achieved"] / roof["peak"]
    tr = TRAFFIC.get(args.workload)
    roof["traffic"] = tr[0] if tr else None
    if tr:
        roof["traffic_source"] = tr[1]
    roof["algorithmic_bytes_per_launch"] = int(bytes_step // R) if len(shapes) == 1 else None
    roof["avg_launch_us"] = ms_per_step * 1e3 / (R * len(shapes))

    # ---- correctness of the timed configuration (a skipped dispatch always looks like a fast one) ----
    W, s, b, y = sets[0][0]
    label, N, K, M, f32 = shapes[0]
    torch.cuda.synchronize()
    yh = y.float().cpu().numpy()
    verified = None
    if rank == 0:
        from oracle import ztvm_oracle as zo, ztvm_oracle_c as zc
        zc.build()
        rows = min(M, 4)
        y64 = zc.matmul_f64(xs[0][:rows].cpu().numpy(), W.cpu().numpy().view(np.uint32), s.cpu().numpy(),
                            b.cpu().numpy(), 64, BITS, w16=is_gemm)
        err = zo.rel_err_scaled(yh[:rows], y64, 1e-2 if is_gemm else 1e-3)
        verified = {"rows": rows, "max_rel_err": err, "max_rel_err_pure": zo.rel_err(yh[:rows], y64),
                    "floor": "1e-2 x rms(y_ref)" if is_gemm else "1e-3 x rms(y_ref)", "ok": bool(err <= 2e-3 and np.abs(yh).max() > 0)}

    # ---- end to end through the host-buffer entry point: pinned x in, y out, every launch ----
    d0 = descs[0]
    xh = torch.randn((M, K)).to(torch.float16).pin_memory()
    yh_t = torch.empty((M, N), dtype=torch.float32 if f32 else torch.float16).pin_memory()
    e2e_sets = [one[0] for one in sets]
    # three result buffers: the queued calls of the pipelined form each need their own while they are in flight
    yh_ring = [yh_t] + [torch.empty_like(yh_t).pin_memory() for _ in range(2)]
    for (W, s, b, _y) in e2e_sets[:3]:
        ctx.int4_matmul_host(d0, yh_t, xh, s, W, b)
    for i, (W, s, b, _y) in enumerate(e2e_sets[:3]):
        ctx.int4_matmul_host_async(d0, yh_ring[i % 3], xh, s, W, b)
    ctx.host_wait()
    torch.cuda.synchronize()
    e2e_steps = max(1, min(args.steps, 5))

    def e2e_time(run_step):
        if world > 1:
            dist.barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            run_step()
        torch.cuda.synchronize()
        sec = (time.perf_counter() - t0) / e2e_steps
        if world > 1:
            t = torch.tensor([sec], device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            sec = float(t.item())
        return sec

    def step_sync():
        for (W, s, b, _y) in e2e_sets:
            ctx.int4_matmul_host(d0, yh_t, xh, s, W, b)

    def step_pipelined():      # every launch still copies its x in and its y out; the wait closes the step
        for i, (W, s, b, _y) in enumerate(e2e_sets):
            ctx.int4_matmul_host_async(d0, yh_ring[i % 3], xh, s, W, b)
        ctx.host_wait()

    def rate(sec):
        if is_gemm:
            return world * R_rot * 2.0 * M * N * K / sec / 1e12
        return world * R_rot * algorithmic_bytes(N, K, M, out_bytes=4 if f32 else 2) / sec / 1e9

    e2e_sync_s = e2e_time(step_sync)
    e2e_s = e2e_time(step_pipelined)
    # the pipelined form must deliver what the synchronous one does (same weights: the last set of the rotation)
    Wl, sl, bl, _ = e2e_sets[-1]
    ctx.int4_matmul_host(d0, yh_t, xh, sl, Wl, bl)
    same = bool(torch.equal(yh_t, yh_ring[(len(e2e_sets) - 1) % 3])) if len(e2e_sets) % 3 != 1 else True
    e2e = {"value": rate(e2e_s), "unit": unit, "h2d_bytes_per_step": R_rot * M * K * 2,
           "d2h_bytes_per_step": R_rot * M * N * (4 if f32 else 2), "launches_per_step": R_rot,
           "what": "ztvm_int4_matmul_host_async per launch (pinned x -> device, kernel, y -> host on three lanes, so the two "
                   "copy directions and the kernels of neighbouring launches overlap), ztvm_host_wait at the end of the step; "
                   "weights resident",
           "synchronous_value": rate(e2e_sync_s), "synchronous_what": "ztvm_int4_matmul_host: copy, kernel, copy, wait, per launch",
           "pipelined_equals_synchronous": same}

    del sets, graph, e2e_sets
    torch.cuda.empty_cache()
    # ---- the decode half of the metric (M = 1, GB/s against the measured copy bandwidth), rank 0 of the default run ----
    decode = None
    if args.workload == "prefill_gemm_m512" and not args.no_decode:
        if rank == 0:
            decode = [quick_device_rate(ctx, torch, device, z, w, max(3, args.steps // 2), args.warmup)
                      for w in ("decode_gemv", "decode_layer_set", "decode_layer_set_fused", "shape:151936x4096x1xf32",
                                "shape:12288x4096x1xq3")]
            decode.append(fused_ffn_rate(ctx, torch, device, z, max(3, args.steps // 2), args.warmup))
            workload_shapes(args.workload)      # back to the main workload's code width
        if world > 1:
            dist.barrier()

    # ---- the forms of the path that shard, in this same process group (one rank: their single-GPU form) ----
    sharded_list = None
    if args.workload == "prefill_gemm_m512" and not args.no_sharded:
        sb = ShardedBench(torch, dist, z, rank, world, local, min(args.steps, 20), args.warmup)
        sharded_list = []
        for fn, a in ((sb.moe_ep, (2048, "strong")), (sb.moe_ep, (256, "strong")), (sb.moe_ep, (2048, "weak")),
                      (sb.moe_ep, (2048, "strong", True)),
                      (sb.layer_set, (1, "fused")), (sb.layer_set, (4, "fused")), (sb.layer_set, (1, "nccl"))):
            if world == 1 and a == (1, "nccl"):
                continue                      # one rank: no gather of either kind
            if world == 1 and a in ((2048, "weak"), (2048, "strong", True)):
                continue                      # one rank: weak and strong are the same run; nothing to dispatch
            try:
                sharded_list.append(fn(*a))
            except Exception as e:            # a form that fails must not take the headline line with it
                sharded_list.append({"workload": fn.__name__, "args": list(a), "error": f"{type(e).__name__}: {e}"[:300]})
            torch.cuda.empty_cache()
        sb.close()

    out = {
        "metric": METRIC, "value": value, "unit": unit, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": DTYPE, "data": "synthetic",
        "config": config_for(args.workload, shapes, world),
        "timing": {"rotation_sets": R_rot, "passes_per_step": passes, "rotation_bytes": int(bytes_step // passes)},
        "roofline": roof, "e2e": e2e, "gpu_launches": int(args.steps * n_launch_step),
        "clocks": clocks.summary(), "verified": verified,
        "decode": decode, "sharded": sharded_list,
    }
    if rank == 0:
        if not args.no_cpu_baseline and world == 1:
            cb = cpu_reference(shapes, 3, 1) or cpu_port(shapes)
            v, _u = rate_of(cb, shapes)
            out["cpu_baseline"] = {"value": v, "unit": unit, "cores": cb["cores"], "kind": cb["kind"], "sample": cb["sample"],
                                   **{k: cb[k] for k in ("dequant_s", "matmul_s", "host_cores") if k in cb}}
            if cb["kind"] == "reference":     # the oracle's C restatement of the reference word order, beside it
                pb = cpu_port(shapes, limit_s=6.0)
                out["cpu_baseline_port"] = {"value": rate_of(pb, shapes)[0], "unit": unit, "cores": pb["cores"], "kind": "port",
                                            "sample": pb["sample"]}
        print(json.dumps(out))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
