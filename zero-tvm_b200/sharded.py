"""Sharded forms of the path over one process per GPU (torch.distributed is the plumbing; NCCL on GPUs).

The reference runs every matmul whole on one device; the two sharded forms here are the natural partitions of
the path: output rows of a dense projection (each workgroup owns rows: src/compiler/shaders/int4_matmul.gen.ts:243)
and experts of a MoE block (experts never mix tokens: src/zero-tvm/engine-core.ts:4444-4450).

  NShardedProjection   rank r owns rows [r*N/G, (r+1)*N/G) of W / scales / biases, x is replicated; the output
                       shards meet in one all-gather.
  ExpertParallelMoE    rank r owns routed experts [r*E/G, (r+1)*E/G) plus a replica of the shared expert; tokens
                       are sharded T/G; (token, slot) pairs travel to the owner of their expert in one all-to-all,
                       the expert FFN runs there, results travel back in a second all-to-all, and the weighted
                       combine runs where the token lives.

Both classes take a `kernels` object with the per-projection calls (`CudaKernels` below binds them to the C ABI).
The planning code (bucket, sort, permute) is device-agnostic tensor code, so the multi-rank logic is also tested on
CPU ranks over gloo with a checker standing in for `kernels`.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist

from .backend import moe_down_pod_args, moe_gate_pod_args, pod_args, resolve_matmul


def shard_rows(N: int, world: int, rank: int) -> tuple[int, int]:
    """Row range of rank `rank`: contiguous, sizes differ by at most one multiple of 16 rows."""
    per = -(-N // world)
    per = -(-per // 16) * 16
    lo = min(N, rank * per)
    return lo, min(N, lo + per)


class CudaKernels:
    """The per-projection calls of the sharded forms, bound to libztvm_b200.so on this rank's GPU.

    Every call is issued on torch's CURRENT stream, the one the surrounding tensor code and the NCCL collectives
    are ordered on; the library's own stream is non-blocking and would race with them.
    """

    def __init__(self, backend):
        self.be = backend

    @staticmethod
    def _stream() -> int:
        h = torch.cuda.current_stream().cuda_stream
        return h if h else 1      # 0 would mean "the library's stream" to the C ABI; 1 is the legacy default stream

    def matmul(self, y, x, W, s, b, N, K, M, out_f32=False):
        entry = resolve_matmul(affine=True, K=K, out_f32=out_f32) if M == 1 else "int4_matmul_batched_dyn_affine"
        self.be.dispatch(entry, [y, x, s, W, pod_args(K, N, m_rows=None if M == 1 else M), b], stream=self._stream())

    def matmul_multi(self, y_dsts, y_row_stride, x, W, s, b, N, K, M, out_f32=False):
        """The decode matmul with its [M, N] result stored into every address of `y_dsts` (ztvm_int4_matmul_multi)."""
        from .capi import MmDesc
        self.be.ctx.int4_matmul_multi(MmDesc(K, N, M, 64, 4, 1, int(out_f32)), y_dsts, y_row_stride, x, s, W, b,
                                      stream=self._stream())

    def dispatch_plan(self, ids_routed, experts_per_rank, world):
        """ids_routed: an int32 [T, K] view (row stride allowed) of routed expert ids -> (order i64, local expert i32,
        pairs per destination rank i64), all on the device."""
        T, K = ids_routed.shape
        assert ids_routed.stride(1) == 1
        dev = ids_routed.device
        order = torch.empty((T * K,), dtype=torch.int64, device=dev)
        local_expert = torch.empty((T * K,), dtype=torch.int32, device=dev)
        send = torch.empty((world,), dtype=torch.int64, device=dev)
        self.be.ctx.moe_dispatch_plan(ids_routed, T, K, ids_routed.stride(0), experts_per_rank * world, experts_per_rank,
                                      world, order, local_expert, send, stream=self._stream())
        return order, local_expert, send

    def route_topk(self, ids, scores, logits, E, K, tokens):
        self.be.moe_router_topk(ids, scores, logits, E, K, True, True, tokens, stream=self._stream())

    def expert_ffn(self, y_rows, x_rows, local_ids, gate, up, down, d, ffn, rows):
        """y_rows[r] = down_e(silu(gate_e x_r) * up_e x_r) with e = local_ids[r]; one slot per row."""
        if rows == 0:
            return
        st = self._stream()
        gu = torch.empty((rows, 1, 2 * ffn), dtype=torch.float16, device=x_rows.device)
        h = torch.empty((rows, 1, ffn), dtype=torch.float16, device=x_rows.device)
        ent_g = resolve_matmul(affine=True, K=d, moe=True)
        ent_d = resolve_matmul(affine=True, K=ffn, moe=True)
        self.be.dispatch(ent_g, [gu, x_rows, gate[1], gate[0], moe_gate_pod_args(d, ffn, 1), gate[2], local_ids],
                         (ffn // 4, rows, 1), stream=st)
        self.be.dispatch(ent_g, [gu.view(-1)[ffn:], x_rows, up[1], up[0], moe_gate_pod_args(d, ffn, 1), up[2], local_ids],
                         (ffn // 4, rows, 1), stream=st)
        self.be.silu_mul(h, gu, rows, ffn, stream=st)
        self.be.dispatch(ent_d, [y_rows, h, down[1], down[0], moe_down_pod_args(d, ffn, 1), down[2], local_ids],
                         (d // 4, rows, 1), stream=st)

    def block_ffn(self, y_slots, gu, h, x, ids, gate, up, down, d, ffn, tokens, slots):
        """The engine's own sequence over an id list [tokens, slots]: gate and up into the halves of gu, SiLU, down."""
        st = self._stream()
        ent_g = resolve_matmul(affine=True, K=d, moe=True)
        ent_d = resolve_matmul(affine=True, K=ffn, moe=True)
        grid = (ffn // 4, tokens, slots)
        # the three matmuls walk one id list, which nothing writes in between: its expert-sorted plan is built once
        self.be.ctx.moe_plan_reuse(True)
        try:
            self.be.dispatch(ent_g, [gu, x, gate[1], gate[0], moe_gate_pod_args(d, ffn, slots), gate[2], ids], grid, stream=st)
            self.be.dispatch(ent_g, [gu.view(-1)[ffn:], x, up[1], up[0], moe_gate_pod_args(d, ffn, slots), up[2], ids], grid, stream=st)
            self.be.silu_mul(h, gu, tokens * slots, ffn, stream=st)
            self.be.dispatch(ent_d, [y_slots, h, down[1], down[0], moe_down_pod_args(d, ffn, slots), down[2], ids],
                             (d // 4, tokens, slots), stream=st)
        finally:
            self.be.ctx.moe_plan_reuse(False)

    # -- expert-parallel step without the host in it (rows travel by peer stores; see ExpertParallelMoE) ------------
    def ep_dispatch(self, layout, ids, tokens, top_k, x, d):
        self.be.ctx.moe_ep_dispatch(layout, ids, tokens, top_k, True, ids.stride(0), x, d, x.stride(0), stream=self._stream())

    def ep_matmul(self, desc, rows, y, x, stack, ids):
        self.be.ctx.int4_matmul_moe_ep(desc, rows, y, x, stack[1], stack[0], stack[2], ids, stream=self._stream())

    def ep_silu(self, rows, ffn, h, gu):
        self.be.ctx.silu_mul_rows(rows, ffn, h, gu, stream=self._stream())

    def dense_ffn(self, x, gate, up, down, e, d, ffn, rows):
        """down_e(silu(gate_e x) * up_e x) for every row of x with ONE expert e of the stacks: plain projections."""
        dev = x.device
        gu = torch.empty((rows, 2 * ffn), dtype=torch.float16, device=dev)
        g = torch.empty((rows, ffn), dtype=torch.float16, device=dev)
        u = torch.empty((rows, ffn), dtype=torch.float16, device=dev)
        for m0 in range(0, rows, 4096):                      # the batched entry takes at most 65535 rows per call
            m = min(4096, rows - m0)
            self.matmul(g[m0:m0 + m], x[m0:m0 + m], gate[0][e], gate[1][e], gate[2][e], ffn, d, m)
            self.matmul(u[m0:m0 + m], x[m0:m0 + m], up[0][e], up[1][e], up[2][e], ffn, d, m)
        gu[:, :ffn] = g
        gu[:, ffn:] = u
        h = torch.empty((rows, ffn), dtype=torch.float16, device=dev)
        self.be.silu_mul(h, gu, rows, ffn, stream=self._stream())
        y = torch.empty((rows, d), dtype=torch.float16, device=dev)
        for m0 in range(0, rows, 4096):
            m = min(4096, rows - m0)
            self.matmul(y[m0:m0 + m], h[m0:m0 + m], down[0][e], down[1][e], down[2][e], d, ffn, m)
        return y

    def combine(self, out, y_slots, scores, tokens, slots, d):
        self.be.moe_combine(out, y_slots, scores, tokens, slots, d, stream=self._stream())


class NShardedProjection:
    """One dense projection with its output rows split over the ranks of `group`.

    Two ways for the shards to meet:
      fused=False  each rank computes its [M, per] block, one NCCL all-gather assembles the rows (any M);
      fused=True   decode form (M <= max_m <= 8): every rank holds the full output in symmetric memory and the GEMV of
                   rank r stores its shard into ALL ranks' outputs from inside the kernel (peer stores over NVLink),
                   followed by one symmetric-memory barrier. No collective kernel, no staging copy. The outputs rotate
                   over THREE buffers: a rank that has passed the barrier of forward n+1 may already be storing forward
                   n+2 into its peers, and that lands in buffer (n+2) % 3, never in the one a slower peer is still
                   reading from forward n. The tensor returned by forward() therefore stays valid until this rank's
                   second forward() after it (it is overwritten by the third): consume it, in stream order, before then.
    """

    def __init__(self, kernels, W, scales, biases, N_total: int, K: int, *, out_f32: bool = False, group=None,
                 fused: bool = False, max_m: int = 8, one_call: bool = False):
        self.k, self.group = kernels, group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.N_total, self.K, self.out_f32 = N_total, K, out_f32
        self.lo, self.hi = shard_rows(N_total, self.world, self.rank)
        self.per = shard_rows(N_total, self.world, 0)[1]
        assert W.shape[0] == self.hi - self.lo, "pass this rank's row shard"
        self.W, self.s, self.b = W, scales, biases
        self.fused = bool(fused) and self.world > 1
        if self.fused:
            import torch.distributed._symmetric_memory as symm
            assert 1 <= max_m <= 8
            dt = torch.float32 if out_f32 else torch.float16
            self.max_m, self._flip = max_m, 0
            self._out = symm.empty((3, max_m, N_total), dtype=dt, device=W.device)
            g = group if group is not None else dist.group.WORLD
            self._hdl = symm.rendezvous(self._out, g.group_name)
            esz = 4 if out_f32 else 2
            # address of (buffer b, row 0, column lo) inside every rank's copy
            self._dst = [[int(base) + (bi * max_m * N_total + self.lo) * esz for base in self._hdl.buffer_ptrs]
                         for bi in range(3)]
            # one_call: ztvm_int4_matmul_nshard (the GEMV's peer stores + the library's own device-side barrier) instead of
            # the GEMV followed by torch's symmetric-memory barrier; the flag words are a symmetric allocation of their own
            self.one_call = bool(one_call)
            if self.one_call:
                self._flag_buf = symm.empty((64,), dtype=torch.int32, device=W.device)
                self._flag_buf.zero_()
                self._flags = [int(p) for p in symm.rendezvous(self._flag_buf, g.group_name).buffer_ptrs]
                dist.barrier(group=group)          # every rank's flag words are zero before anyone's first store

    def forward(self, x: torch.Tensor, M: int) -> torch.Tensor:
        """x f16 [M, K] (replicated) -> y [M, N_total], every rank holding the whole output."""
        if self.fused:
            assert M <= self.max_m
            bi = self._flip
            self._flip = (bi + 1) % 3
            if self.one_call:
                from .capi import MmDesc
                self.k.be.ctx.int4_matmul_nshard(MmDesc(self.K, self.hi - self.lo, M, 64, 4, 1, int(self.out_f32)), self._dst[bi],
                                                 self.world, self.rank, self.N_total, x, self.s, self.W, self.b, self._flags,
                                                 stream=self.k._stream())
                return self._out[bi, :M]
            if self.hi > self.lo:
                self.k.matmul_multi(self._dst[bi], self.N_total, x, self.W, self.s, self.b, self.hi - self.lo, self.K, M,
                                    self.out_f32)
            self._hdl.barrier(channel=bi)          # every shard has landed everywhere (runs on the current stream)
            return self._out[bi, :M]
        dt = torch.float32 if self.out_f32 else torch.float16
        n_loc = self.hi - self.lo
        # every rank contributes a [M, per] block (the last shard may be short: padded, trimmed after the gather)
        y_loc = torch.zeros((M, self.per), dtype=dt, device=x.device)
        if n_loc:
            if n_loc == self.per:
                self.k.matmul(y_loc, x, self.W, self.s, self.b, n_loc, self.K, M, self.out_f32)
            else:
                tmp = torch.empty((M, n_loc), dtype=dt, device=x.device)
                self.k.matmul(tmp, x, self.W, self.s, self.b, n_loc, self.K, M, self.out_f32)
                y_loc[:, :n_loc] = tmp
        if self.world == 1:
            return y_loc[:, :self.N_total]
        buf = torch.empty((self.world * M, self.per), dtype=dt, device=x.device)   # rank-major concatenation
        dist.all_gather_into_tensor(buf, y_loc, group=self.group)
        return buf.view(self.world, M, self.per).permute(1, 0, 2).reshape(M, self.world * self.per)[:, :self.N_total]


@dataclass
class DispatchPlan:
    order: torch.Tensor        # [P] pair indices (token*K + slot) sorted by destination rank
    send_counts: list          # pairs per destination rank
    recv_counts: list          # pairs arriving from each source rank
    local_expert: torch.Tensor  # [P] expert index inside the destination's stack, in send order


def plan_dispatch(ids_routed: torch.Tensor, experts_per_rank: int, world: int, group=None, kernels=None) -> DispatchPlan:
    """Buckets the routed (token, slot) pairs by the rank that owns their expert.

    `kernels.dispatch_plan`, when the kernels object has one, does the sort on the device in one call
    (ztvm_moe_dispatch_plan); otherwise the same plan is built from tensor ops (any device: the CPU ranks of the tests).
    Either way the split sizes have to reach the host: one device-to-host copy per step.
    """
    if kernels is not None and hasattr(kernels, "dispatch_plan"):
        order, local_expert, send = kernels.dispatch_plan(ids_routed, experts_per_rank, world)
    else:
        flat = ids_routed.reshape(-1).to(torch.int64)
        dest = torch.div(flat, experts_per_rank, rounding_mode="floor")
        order = torch.argsort(dest, stable=True)
        send = torch.bincount(dest, minlength=world)[:world]
        local_expert = (flat[order] % experts_per_rank).to(torch.int32)
    if world > 1:
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=group)
    else:
        recv = send.clone()
    return DispatchPlan(order, send.tolist(), recv.tolist(), local_expert)


class ExpertParallelMoE:
    """Expert-parallel form of the block the engine runs as seven dispatches (engine-core.ts:2342-2349)."""

    def __init__(self, kernels, gate, up, down, *, E: int, top_k: int, d: int, ffn: int, group=None, max_tokens=None,
                 peer: bool = True, world: int | None = None, rank: int | None = None, one_call: bool = False):
        """gate / up / down: (W, scales, biases) stacks of THIS rank: E/G routed experts followed by the shared one.
        world / rank: only to stand in for a process group (tests that run several ranks' steps from one process).
        one_call: the peer-store step through ztvm_moe_ffn_ep (dispatch, the library's own device-side barrier, the
        three projections, barrier) instead of the separate calls with torch's symmetric-memory barrier."""
        self.k, self.group = kernels, group
        self.world = world if world is not None else (dist.get_world_size(group) if dist.is_initialized() else 1)
        self.rank = rank if rank is not None else (dist.get_rank(group) if dist.is_initialized() else 0)
        assert E % self.world == 0
        self.E, self.top_k, self.d, self.ffn = E, top_k, d, ffn
        self.epr = E // self.world
        self.gate, self.up, self.down = gate, up, down
        self.max_tokens = max_tokens
        # One rank: there is nothing to dispatch, the block is the engine's own sequence of dispatches over the id list.
        # Several ranks, CUDA kernels: rows travel by peer stores from inside the kernels (symmetric memory), counts stay
        # on the device. Otherwise (CPU ranks of the tests, or peer=False): two all-to-alls with host-read split sizes.
        self.peer = bool(peer) and self.world > 1 and hasattr(kernels, "ep_dispatch")
        self.form = ("one rank: router, gate, up, SiLU, down, combine over the id list" if self.world == 1 else
                     "peer stores: dispatch kernel -> barrier -> grouped expert matmuls over the receive buffer, the down "
                     "projection storing each result row to its source rank -> barrier -> combine" if self.peer else
                     "all-to-all of counts, rows and results (host reads the split sizes)")
        self.capturable = self.world == 1 or self.peer      # no host round trip inside a step
        self.one_call = bool(one_call) and self.peer
        self._bufs = {}

    def _local_block(self, x: torch.Tensor, logits: torch.Tensor) -> torch.Tensor:
        """world == 1: the shared expert is just slot K of every token (its id is E), as the engine runs it."""
        T, K, d, ffn = x.shape[0], self.top_k, self.d, self.ffn
        if T not in self._bufs:         # buffers are kept per token count, so a step can be replayed from a CUDA graph
            dev = x.device
            self._bufs[T] = dict(ids=torch.empty((T, K + 1), dtype=torch.int32, device=dev),
                                 scores=torch.empty((T, K + 1), dtype=torch.float32, device=dev),
                                 gu=torch.empty((T, K + 1, 2 * ffn), dtype=torch.float16, device=dev),
                                 h=torch.empty((T, K + 1, ffn), dtype=torch.float16, device=dev),
                                 y=torch.empty((T, K + 1, d), dtype=torch.float16, device=dev),
                                 out=torch.empty((T, d), dtype=torch.float16, device=dev))
        b = self._bufs[T]
        self.k.route_topk(b["ids"], b["scores"], logits, self.E, K, T)
        self.k.block_ffn(b["y"], b["gu"], b["h"], x, b["ids"], self.gate, self.up, self.down, d, ffn, T, K + 1)
        self.k.combine(b["out"], b["y"], b["scores"], T, K + 1, d)
        return b["out"]

    def peer_bytes(self, T: int):
        """Size and offsets of one rank's symmetric allocation for T local tokens."""
        G, K, d = self.world, self.top_k, self.d
        cap = max(T * K, T)
        R = (G + 1) * cap
        al = lambda n: (n + 255) // 256 * 256
        off_x, off_ids = 0, al(R * d * 2)
        off_src = off_ids + al(R * 4)
        off_cnt = off_src + al(R * 4)
        off_y = off_cnt + 256          # recv_cnt takes 64 bytes of its 256; the barrier's flag words the next 64
        return off_y + al(T * (K + 1) * d * 2), (off_x, off_ids, off_src, off_cnt, off_y), cap, R

    def _peer_state(self, T: int, dev, buf=None, ptrs=None):
        """Symmetric receive buffers + result slots for T local tokens (one allocation, one rendezvous).
        buf / ptrs: an allocation made by the caller and every rank's base address (tests without a process group)."""
        if ("peer", T) in self._bufs:
            return self._bufs[("peer", T)]
        from .capi import MoeDesc, MmDesc, MoeEpLayout, MoeEpRows
        G, K, d, ffn = self.world, self.top_k, self.d, self.ffn
        total, (off_x, off_ids, off_src, off_cnt, off_y), cap, R = self.peer_bytes(T)
        regions = G + 1
        hdl = None
        if buf is None:
            import torch.distributed._symmetric_memory as symm
            buf = symm.empty((total,), dtype=torch.uint8, device=dev)
            buf.zero_()
            g = self.group if self.group is not None else dist.group.WORLD
            hdl = symm.rendezvous(buf, g.group_name)
            ptrs = [int(p) for p in hdl.buffer_ptrs]
        st = dict(hdl=hdl, buf=buf, cap=cap, R=R)
        view = lambda off, n, dt, shape: buf[off:off + n].view(dt).view(shape)
        st["recv_x"] = view(off_x, R * d * 2, torch.float16, (R, d))
        st["recv_ids"] = view(off_ids, R * 4, torch.int32, (R,))
        st["recv_src"] = view(off_src, R * 4, torch.int32, (R,))
        st["recv_cnt"] = view(off_cnt, 64, torch.int32, (16,))
        st["y_slots"] = view(off_y, T * (K + 1) * d * 2, torch.float16, (T, K + 1, d))
        L = MoeEpLayout()
        L.world, L.rank, L.experts_per_rank, L.seg_cap = G, self.rank, self.epr, cap
        for r in range(G):
            L.recv_x[r], L.recv_ids[r], L.recv_src[r], L.recv_cnt[r] = ptrs[r] + off_x, ptrs[r] + off_ids, ptrs[r] + off_src, ptrs[r] + off_cnt
        st["cursors"] = torch.zeros((G + 2,), dtype=torch.int32, device=dev)
        L.cursors = st["cursors"].data_ptr()
        st["layout"] = L

        def rows(dst: bool, reuse: bool):
            r = MoeEpRows()
            r.seg_counts, r.seg_cap, r.segments, r.reuse_plan = st["recv_cnt"].data_ptr(), cap, regions, int(reuse)
            if dst:
                r.dst_index = st["recv_src"].data_ptr()
                for i in range(G):
                    r.y_seg[i] = ptrs[i] + off_y
                r.y_seg[G] = ptrs[self.rank] + off_y          # the local region's rows belong to this rank's own tokens
            return r
        st["rows_first"], st["rows_again"], st["rows_down"] = rows(False, False), rows(False, True), rows(True, True)
        mm = lambda Kd, N: MmDesc(Kd, N, 1, 64, 4, 1, 0)
        E1 = self.epr + 1
        st["desc_gu"] = MoeDesc(mm(d, ffn), E1, 1, R, 0, 2 * ffn, d, 2 * ffn, 1)
        st["desc_down"] = MoeDesc(mm(ffn, d), E1, 1, R, 0, d, ffn, d, 1)
        st["ids"] = torch.empty((T, K + 1), dtype=torch.int32, device=dev)
        st["scores"] = torch.empty((T, K + 1), dtype=torch.float32, device=dev)
        st["gu"] = torch.empty((R, 2 * ffn), dtype=torch.float16, device=dev)
        st["h"] = torch.empty((R, ffn), dtype=torch.float16, device=dev)
        st["out"] = torch.empty((T, d), dtype=torch.float16, device=dev)
        if self.one_call:
            from .capi import MoeFfnEpArgs
            a = MoeFfnEpArgs()
            a.layout = L
            a.tokens, a.top_k, a.has_shared, a.ids_stride, a.d, a.ffn, a.x_tok_stride = T, K, 1, K + 1, d, ffn, d
            a.ids = st["ids"].data_ptr()
            for nm, stack in (("gate", self.gate), ("up", self.up), ("down", self.down)):
                setattr(a, nm + "_w", stack[0].data_ptr())
                setattr(a, nm + "_scales", stack[1].data_ptr())
                setattr(a, nm + "_biases", stack[2].data_ptr())
            a.gate_up, a.h = st["gu"].data_ptr(), st["h"].data_ptr()
            for r in range(G):
                a.y_slots[r] = ptrs[r] + off_y
                a.flags[r] = ptrs[r] + off_cnt + 64
            st["args"] = a
        self._bufs[("peer", T)] = st
        return st

    def _peer_block(self, x: torch.Tensor, logits: torch.Tensor) -> torch.Tensor:
        """One step with no host round trip: every launch below is ordered on the current stream, the two barriers are
        device-side (symmetric-memory signal pads), so the whole step can be replayed from a CUDA graph."""
        T, K, d, ffn = x.shape[0], self.top_k, self.d, self.ffn
        st = self._peer_state(T, x.device)
        self.k.route_topk(st["ids"], st["scores"], logits, self.E, K, T)
        if self.one_call:
            st["args"].x = x.data_ptr()
            self.k.be.ctx.moe_ffn_ep(st["args"], stream=self.k._stream())
        else:
            self.k.ep_dispatch(st["layout"], st["ids"], T, K, x, d)
            st["hdl"].barrier(channel=0)                   # every rank's rows and counts have landed here
            self._peer_ffn(st)
            st["hdl"].barrier(channel=1)                   # every result row is back where its token lives
        self.k.combine(st["out"], st["y_slots"], st["scores"], T, K + 1, d)
        return st["out"]

    def _peer_ffn(self, st):
        """Expert FFN over everything that arrived; the down projection returns each row to its source rank."""
        ffn = self.ffn
        self.k.ep_matmul(st["desc_gu"], st["rows_first"], st["gu"], st["recv_x"], self.gate, st["recv_ids"])
        self.k.ep_matmul(st["desc_gu"], st["rows_again"], st["gu"].view(-1)[ffn:], st["recv_x"], self.up, st["recv_ids"])
        self.k.ep_silu(st["rows_first"], ffn, st["h"], st["gu"])
        self.k.ep_matmul(st["desc_down"], st["rows_down"], st["y_slots"], st["h"], self.down, st["recv_ids"])

    def _a2a(self, send: torch.Tensor, send_counts, recv_counts) -> torch.Tensor:
        out = torch.empty((sum(recv_counts),) + tuple(send.shape[1:]), dtype=send.dtype, device=send.device)
        if self.world == 1:
            out.copy_(send)
        else:
            dist.all_to_all_single(out, send, output_split_sizes=recv_counts, input_split_sizes=send_counts, group=self.group)
        return out

    def forward(self, x: torch.Tensor, logits: torch.Tensor) -> torch.Tensor:
        """x f16 [T_local, d], logits f32 [T_local, E+1] -> y f16 [T_local, d] (overwritten by the next forward)."""
        if self.world == 1:
            return self._local_block(x, logits)
        if self.peer:
            return self._peer_block(x, logits)
        T, K, d = x.shape[0], self.top_k, self.d
        dev = x.device
        ids = torch.empty((T, K + 1), dtype=torch.int32, device=dev)
        scores = torch.empty((T, K + 1), dtype=torch.float32, device=dev)
        self.k.route_topk(ids, scores, logits, self.E, K, T)
        plan = plan_dispatch(ids[:, :K], self.epr, self.world, self.group, kernels=self.k)
        # ids outside the expert range are left out by the device-side plan: only the filled prefix is a plan
        n_sent = sum(plan.send_counts)
        plan.order, plan.local_expert = plan.order[:n_sent], plan.local_expert[:n_sent]
        # dispatch: activation rows and their local expert index, in destination order
        tok_of_pair = torch.div(plan.order, K, rounding_mode="floor")
        x_send = x.index_select(0, tok_of_pair)
        x_recv = self._a2a(x_send, plan.send_counts, plan.recv_counts)
        e_recv = self._a2a(plan.local_expert.reshape(-1, 1), plan.send_counts, plan.recv_counts)
        # expert FFN on what arrived
        R = x_recv.shape[0]
        y_recv = torch.empty((R, d), dtype=torch.float16, device=dev)
        self.k.expert_ffn(y_recv, x_recv, e_recv.contiguous(), self.gate, self.up, self.down, d, self.ffn, R)
        # combine: results travel back and are un-permuted into [T, K+1, d]
        y_back = self._a2a(y_recv, plan.recv_counts, plan.send_counts)
        y_slots = torch.empty((T, K + 1, d), dtype=torch.float16, device=dev)
        routed = torch.zeros((T * K, d), dtype=torch.float16, device=dev)     # a dropped pair contributes nothing
        routed.index_copy_(0, plan.order, y_back)
        y_slots[:, :K] = routed.view(T, K, d)
        # the shared expert is replicated and sees every local token: three dense projections (GEMM / GEMV by T), no ids
        y_slots[:, K] = self.k.dense_ffn(x, self.gate, self.up, self.down, self.epr, d, self.ffn, T)
        out = torch.empty((T, d), dtype=torch.float16, device=dev)
        self.k.combine(out, y_slots, scores, T, K + 1, d)
        return out
