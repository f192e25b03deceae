"""Worker of test_gpu_multi.py: one process per GPU (NCCL for the rendezvous, the data moves by the library's own peer
stores). Every rank checks its own results against the oracle and exits non-zero on a mismatch.

  row-sharded projection, fused form: a consumer kernel reads the output of forward n AFTER forward n+1 has been
    issued (the longest lifetime the class promises), while the ranks are deliberately driven out of step, so a
    buffer that a fast peer overwrites too early shows up as a wrong sum;
  expert-parallel MoE block, peer-store form: eager and as a replayed CUDA graph against the oracle's whole block,
    through the separate calls (torch's symmetric-memory barrier) and through ztvm_moe_ffn_ep (the library's barrier).
"""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import zero_tvm_b200 as z                      # noqa: E402
from zero_tvm_b200 import sharded              # noqa: E402
from oracle import ztvm_oracle as zo, ztvm_oracle_c as zc   # noqa: E402


def rand_w(g, dev, lead, N, K):
    W = torch.randint(-2**31, 2**31 - 1, (*lead, N, K // 8), dtype=torch.int32, device=dev, generator=g)
    sc = (torch.randn((*lead, N, K // 64), device=dev, generator=g) * 0.01).abs().to(torch.float16)
    b = (torch.randn((*lead, N, K // 64), device=dev, generator=g) * 0.05).to(torch.float16)
    return W, sc, b


def np_w(t):
    return tuple(a.cpu().numpy().view(np.uint32) if a.dtype == torch.int32 else a.cpu().numpy() for a in t)


def projection_with_a_late_consumer(k, dev, rank, world, one_call=False):
    N, K, M, steps = 1536, 512, 4, 24
    g = torch.Generator(device=dev)
    g.manual_seed(5)
    W, sc, b = rand_w(g, dev, (), N, K)
    lo, hi = sharded.shard_rows(N, world, rank)
    pj = sharded.NShardedProjection(k, W[lo:hi].contiguous(), sc[lo:hi].contiguous(), b[lo:hi].contiguous(), N, K,
                                    fused=True, max_m=M, one_call=one_call)
    xs = torch.randn((steps, M, K), device=dev, generator=g).to(torch.float16)
    consumed = torch.zeros((steps, M, N), dtype=torch.float32, device=dev)
    prev = None
    for n in range(steps):
        # ranks take turns being slow: the sleeping rank's consumer of forward n-1 runs long after its peers moved on
        if n % world == rank:
            torch.cuda._sleep(3_000_000)
        y = pj.forward(xs[n], M)
        if prev is not None:
            consumed[n - 1].copy_(prev)          # reads forward n-1 after forward n was issued
        prev = y
    consumed[steps - 1].copy_(prev)
    torch.cuda.synchronize()
    Wn, sn, bn = np_w((W, sc, b))
    worst = 0.0
    for n in range(steps):
        ref = zc.matmul_f64(xs[n].cpu().numpy(), Wn, sn, bn, 64)
        err = zo.rel_err_scaled(consumed[n].cpu().numpy(), ref, 1e-3)
        worst = max(worst, err)
    assert worst <= 2e-3, f"rank {rank}: consumed outputs differ from the oracle: {worst:.3e}"
    return worst


def moe_block_by_peer_stores(k, dev, rank, world, one_call=False):
    E, top_k, d, ffn, tl = 16, 4, 256, 128, 40
    epr = E // world
    g = torch.Generator(device=dev)
    g.manual_seed(7)
    sel = torch.tensor(list(range(rank * epr, (rank + 1) * epr)) + [E], device=dev)
    stacks, full = [], []
    for N, K in ((ffn, d), (ffn, d), (d, ffn)):
        t = rand_w(g, dev, (E + 1,), N, K)
        stacks.append(tuple(a[sel].contiguous() for a in t))
        full.append(np_w(t))
    moe = sharded.ExpertParallelMoE(k, *stacks, E=E, top_k=top_k, d=d, ffn=ffn, one_call=one_call)
    x_all = torch.randn((tl * world, d), device=dev, generator=g).to(torch.float16)
    l_all = torch.randn((tl * world, E + 1), device=dev, generator=g)
    x, logits = x_all[rank * tl:(rank + 1) * tl].contiguous(), l_all[rank * tl:(rank + 1) * tl].contiguous()
    ref = zo.moe_block(x.cpu().numpy(), logits.cpu().numpy(), full[0], full[1], full[2], E, top_k, ffn)["y"].astype(np.float64)

    def check(out, what):
        got = out.float().cpu().numpy()
        err = float(np.abs(got - ref).max() / np.abs(ref).max())
        assert np.isfinite(got).all() and err <= 5e-3, f"rank {rank}: {what}: {err:.3e}"
        return err

    assert "peer" in moe.form, moe.form
    e0 = check(moe.forward(x, logits), "eager")
    e1 = e0
    if moe.capturable:
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            moe.forward(x, logits)
            side.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                out = moe.forward(x, logits)
            side.synchronize()
        for _ in range(3):
            out.zero_()
            torch.cuda.synchronize()
            dist.barrier()
            graph.replay()
            torch.cuda.synchronize()
            e1 = max(e1, check(out, "graph replay"))
    return max(e0, e1)


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    be = z.backend.CudaMatmulBackend(local)
    k = sharded.CudaKernels(be)
    a = projection_with_a_late_consumer(k, dev, rank, world)
    a = max(a, projection_with_a_late_consumer(k, dev, rank, world, one_call=True))      # ztvm_int4_matmul_nshard
    b = moe_block_by_peer_stores(k, dev, rank, world)
    # the same step as ONE library call per rank (ztvm_moe_ffn_ep) with the library's own device-side barrier
    c = moe_block_by_peer_stores(k, dev, rank, world, one_call=True)
    b = max(b, c)
    assert be.ctx.device_errors() == 0
    print(f"rank {rank}: projection {a:.3e} moe {b:.3e} ok", flush=True)
    be.close()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
