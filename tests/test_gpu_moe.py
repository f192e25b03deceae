"""GPU parity of the MoE path: router top-k, ids-indirect expert matmuls, SiLU*up, weighted combine,
composed exactly like the engine's seven dispatches (src/zero-tvm/engine-core.ts:2342-2349)."""
import numpy as np
import pytest

import zero_tvm_b200 as z
from oracle import ztvm_oracle as zo
from conftest import record_parity
from zero_tvm_b200.backend import moe_down_pod_args, moe_gate_pod_args, resolve_matmul

pytestmark = pytest.mark.gpu
TOL = 2e-3   # with the scale-tied floor of oracle.rel_err_scaled (1e-3 of the output rms)


def moe_kernel_kind(pairs, experts, K, N, bits):
    """Which kernel ztvm_int4_matmul_moe picks (mirrors moe_pick in ztvm_api.cu): 'pair', 'stream' or 'tiles'."""
    if bits != 4 or pairs < 128 or experts > 1024:
        return "pair"
    tiles_ok = K % 64 == 0 and N % 8 == 0
    stream_ok = K % 256 == 0 and K <= 4096 and N % 16 == 0
    if stream_ok and (pairs < 10 * experts or not tiles_ok):
        return "stream"
    return "tiles" if tiles_ok else "pair"


def run_block(backend, dev, mb, K_top=8, bits=4):
    """router -> gate, up -> silu -> down -> combine with the engine's buffers and PODArgs."""
    T, E, d, ffn = mb["T"], mb["E"], mb["hidden"], mb["ffn"]
    slots = K_top + int(mb["has_shared"])
    x, logits = dev.put(mb["x"]), dev.put(mb["logits"])
    ids = dev.empty((T, slots), np.uint32, fill=0x7FFFFFFF)
    scores = dev.empty((T, slots), np.float32, fill=-999.0)
    backend.moe_router_topk(ids, scores, logits, E, K_top, True, mb["has_shared"], T)
    gate_up = dev.empty((T, slots, 2 * ffn), np.float16, fill=float("nan"))
    ent_g = resolve_matmul(affine=True, K=d, moe=True, q3=bits == 3)
    ent_d = resolve_matmul(affine=True, K=ffn, moe=True, q3=bits == 3)
    gw, gs, gb = (dev.put(a) for a in mb["gate"])
    uw, us, ub = (dev.put(a) for a in mb["up"])
    dw, ds, db = (dev.put(a) for a in mb["down"])
    grid = (ffn // 4, T, slots)
    backend.dispatch(ent_g, [gate_up, x, gs, gw, moe_gate_pod_args(d, ffn, slots, bits), gb, ids], grid)
    # `up` is the same kernel bound ffn elements into the buffer (engine-core.ts:2036-2043)
    up_view = gate_up.view(-1)[ffn:]
    backend.dispatch(ent_g, [up_view, x, us, uw, moe_gate_pod_args(d, ffn, slots, bits), ub, ids], grid)
    h = dev.empty((T, slots, ffn), np.float16, fill=float("nan"))
    backend.silu_mul(h, gate_up, T * slots, ffn)
    y_slots = dev.empty((T, slots, d), np.float16, fill=float("nan"))
    backend.dispatch(ent_d, [y_slots, h, ds, dw, moe_down_pod_args(d, ffn, slots, bits), db, ids], (d // 4, T, slots))
    y = dev.empty((T, d), np.float16, fill=float("nan"))
    backend.moe_combine(y, y_slots, scores, T, slots, d)
    assert backend.ctx.device_errors() == 0
    return dict(ids=dev.get(ids, np.uint32), scores=dev.get(scores), gate_up=dev.get(gate_up), h=dev.get(h),
                y_slots=dev.get(y_slots), y=dev.get(y))


def check_block(got, mb, oracle_c, K_top=8, bits=4, pairs_run=None):
    """pairs_run: (token, slot) pairs of the launch that produced `got`, when `mb` is only a sample of its tokens."""
    T, E, d, ffn = mb["T"], mb["E"], mb["hidden"], mb["ffn"]
    ids_ref, sc_ref = oracle_c.router_topk(mb["logits"], E, K_top, True, mb["has_shared"])
    # routing: indices exact, scores 2e-6 (tests/kernels/run.mjs:333-336)
    assert np.array_equal(got["ids"], ids_ref)
    assert np.abs(got["scores"] - sc_ref).max() < 2e-6
    # each stage against the f64 anchor computed from the GPU's own (already checked) inputs. The anchor follows the
    # kernel that ran: the tensor-core tiles multiply f16 weights (anchor over W16, GEMM floor), the per-pair GEMV and
    # the streaming grouped kernel multiply the codes exactly (anchor over fl32(s*q+b), GEMV floor).
    experts = E + int(mb["has_shared"])
    def anchor(x_in, proj, N, K, per_slot):
        tiles = moe_kernel_kind(pairs_run or ids_ref.size, experts, K, N, bits) == "tiles"
        ref = oracle_c.moe_matmul_f64(x_in, *mb[proj], ids_ref, N, K, 64, bits, in_per_slot=per_slot, w16=tiles)
        return ref, (1e-2 if tiles else 1e-3)
    def graded(y, ref, frac=1e-3):
        err = zo.rel_err_scaled(y, ref, frac)
        record_parity(err, zo.rel_err(y, ref))
        return err
    g64, fr = anchor(mb["x"], "gate", ffn, d, False)
    assert graded(got["gate_up"][..., :ffn], g64, fr) <= TOL
    u64, fr = anchor(mb["x"], "up", ffn, d, False)
    assert graded(got["gate_up"][..., ffn:], u64, fr) <= TOL
    h_ref = oracle_c.silu_mul(got["gate_up"], ffn)
    assert graded(got["h"], h_ref.astype(np.float64)) <= TOL
    d64, fr = anchor(got["h"], "down", d, ffn, True)
    assert graded(got["y_slots"], d64, fr) <= TOL
    y_ref = oracle_c.moe_combine(got["y_slots"], got["scores"])
    assert np.array_equal(got["y"].view(np.uint16), y_ref.view(np.uint16))
    assert np.isfinite(got["y"].astype(np.float32)).all()


@pytest.mark.parametrize("E,K,norm,shared", [(256, 8, True, True), (128, 8, True, False), (64, 6, False, True),
                                              (257, 8, True, False), (1000, 32, True, True), (8, 8, True, False)])
def test_router_topk(E, K, norm, shared, backend, dev, oracle_c):
    """makeMoeTopkTest (tests/kernels/run.mjs:284-345): logits uniform in [-4,4), indices exact, scores 2e-6,
    and on the no-shared path the slot past K stays untouched (poisoned here, as there)."""
    rng = np.random.default_rng(E + K)
    T = 37
    logits = (rng.random((T, E + int(shared)), dtype=np.float32) * 8 - 4).astype(np.float32)
    logits[0, 5 % E] = logits[0, 1]                      # exact tie: lower index first
    S = K + int(shared)
    ids = dev.empty((T * S + 1,), np.uint32, fill=0x5EADBEEF)
    sc = dev.empty((T * S + 1,), np.float32, fill=-999.0)
    backend.moe_router_topk(ids, sc, dev.put(logits), E, K, norm, shared, T)
    gi, gs = dev.get(ids, np.uint32), dev.get(sc)
    assert gi[-1] == 0x5EADBEEF and gs[-1] == -999.0     # nothing written past the block
    ri, rs = oracle_c.router_topk(logits, E, K, norm, shared)
    assert np.array_equal(gi[:-1].reshape(T, S), ri)
    assert np.abs(gs[:-1].reshape(T, S) - rs).max() < 2e-6
    if norm:
        assert np.abs(gs[:-1].reshape(T, S)[:, :K].sum(1) - 1).max() < 1e-5


@pytest.mark.parametrize("T", [1, 3, 16])
def test_small_block(T, backend, dev, oracle_c):
    mb = z.synth.moe_block(T, E=16, hidden=256, ffn=128, seed=T)
    got = run_block(backend, dev, mb, K_top=4)
    check_block(got, mb, oracle_c, K_top=4)
    # and against the whole-block numpy restatement (f16 intermediates where the engine stores f16)
    r = zo.moe_block(mb["x"], mb["logits"], mb["gate"], mb["up"], mb["down"], 16, 4, 128)
    # whole-block bound of the reference's real-weight test: 0.005 of max|ref| (tests/kernels/real-weights.mjs:72-73)
    ref = r["y"].astype(np.float64)
    assert np.abs(got["y"].astype(np.float64) - ref).max() <= 5e-3 * np.abs(ref).max()


@pytest.mark.parametrize("T", [1, 16, 256])
def test_qwen36_class_block(T, backend, dev, oracle_c):
    """256 experts + shared, hidden 2048, expert ffn 512, top-8, int4 group 64."""
    mb = z.synth.moe_block(T, seed=0)
    got = run_block(backend, dev, mb)
    check_block(got, mb, oracle_c)


def test_q3_block(backend, dev, oracle_c):
    """3-bit experts (int4_matmul_tiled_affine_q3_moe)."""
    mb = z.synth.moe_block(5, E=32, hidden=512, ffn=256, bits=3, seed=3)
    got = run_block(backend, dev, mb, K_top=4, bits=3)
    check_block(got, mb, oracle_c, K_top=4, bits=3)


def test_full_size_block_properties(backend, dev, oracle_c):
    """T = 2048 at full size: routing exact; a sample of (token, slot) pairs against the f64 anchor;
    and token-permutation invariance (each token's output depends on that token only), bit for bit."""
    T = 2048
    mb = z.synth.moe_block(T, seed=0)
    got = run_block(backend, dev, mb)
    ids_ref, sc_ref = oracle_c.router_topk(mb["logits"], 256, 8, True, True)
    assert np.array_equal(got["ids"], ids_ref)
    sel = np.random.default_rng(1).choice(T, 24, replace=False)
    sub = dict(mb, T=len(sel), x=mb["x"][sel], logits=mb["logits"][sel])
    sub_got = {k: v[sel] for k, v in got.items()}
    check_block(sub_got, sub, oracle_c, pairs_run=ids_ref.size)
    perm = np.random.default_rng(2).permutation(T)
    got_p = run_block(backend, dev, dict(mb, x=mb["x"][perm], logits=mb["logits"][perm]))
    assert np.array_equal(got_p["y"].view(np.uint16), got["y"][perm].view(np.uint16))


def test_bad_expert_id_is_counted_not_followed(backend, dev):
    """An id outside the stack must not be dereferenced: the pair is skipped and counted."""
    mb = z.synth.moe_block(2, E=8, hidden=256, ffn=128, seed=1)
    slots = 3
    ids = np.array([[0, 99, 8], [1, 2, 3]], dtype=np.uint32)      # 99 is out of range (stack has 9 rows)
    out = dev.empty((2, slots, 2 * 128), np.float16, fill=7.0)
    gw, gs, gb = (dev.put(a) for a in mb["gate"])
    backend.dispatch("int4_matmul_tiled_affine_moe",
                     [out, dev.put(mb["x"]), gs, gw, moe_gate_pod_args(256, 128, slots), gb, dev.put(ids)],
                     (32, 2, slots))
    assert backend.ctx.device_errors() == 1
    got = dev.get(out)
    assert (got[0, 1, :128] == 7.0).all()          # skipped pair untouched
    assert (got[0, 0, :128] != 7.0).any()
    assert backend.ctx.device_errors() == 0        # counter resets


def test_grouped_path_handles_bad_ids_and_matches_per_pair_path(backend, dev, oracle_c):
    """160 pairs go through the grouped GEMM: an out-of-range id is counted and its row left untouched; every other
    row agrees with the f64 anchor."""
    mb = z.synth.moe_block(32, E=8, hidden=256, ffn=128, seed=6)
    slots = 5
    rng = np.random.default_rng(0)
    ids = rng.integers(0, 9, size=(32, slots), dtype=np.uint32)
    ids[3, 2] = 77                                     # out of range
    out = dev.empty((32, slots, 2 * 128), np.float16, fill=7.0)
    gw, gs, gb = (dev.put(a) for a in mb["gate"])
    backend.dispatch("int4_matmul_tiled_vec4h_affine_moe",
                     [out, dev.put(mb["x"]), gs, gw, moe_gate_pod_args(256, 128, slots), gb, dev.put(ids)], (32, 32, slots))
    assert backend.ctx.device_errors() == 1
    got = dev.get(out)
    assert (got[3, 2, :128] == 7.0).all() and (got[..., 128:] == 7.0).all()
    ids_ok = ids.copy(); ids_ok[3, 2] = 0
    tiles = moe_kernel_kind(ids.size, 9, 256, 128, 4) == "tiles"
    ref = oracle_c.moe_matmul_f64(mb["x"], *mb["gate"], ids_ok, 128, 256, 64, 4, in_per_slot=False, w16=tiles)
    mask = np.ones((32, slots), bool); mask[3, 2] = False
    assert zo.rel_err_scaled(got[..., :128][mask], ref[mask], 1e-2 if tiles else 1e-3) <= TOL


@pytest.mark.parametrize("forced,kind,tiles_env", [("2", "stream", ""), ("1", "tiles", ""), ("1", "tiles", "sm")])
def test_forced_grouped_kernels_on_uneven_expert_loads(forced, kind, tiles_env, dev, oracle_c, monkeypatch):
    """Each grouped kernel on a skewed routing: one expert takes a third of 300 pairs (many 8-pair chunks for the
    streaming kernel, a full and a ragged 128-pair tile for the tensor-core ones), some experts take none."""
    monkeypatch.setenv("ZTVM_MOE_GROUPED", forced)
    monkeypatch.setenv("ZTVM_MOE_TILES", tiles_env)
    be = z.backend.CudaMatmulBackend(0)
    mb = z.synth.moe_block(100, E=12, hidden=512, ffn=256, seed=21)
    slots = 3
    rng = np.random.default_rng(9)
    ids = rng.choice(np.array([0, 2, 3, 5, 7, 11, 12], dtype=np.uint32), size=(100, slots)).astype(np.uint32)
    ids[rng.random((100, slots)) < 0.34] = 5
    out = dev.empty((100, slots, 2 * 256), np.float16, fill=7.0)
    gw, gs, gb = (dev.put(a) for a in mb["gate"])
    be.dispatch("int4_matmul_tiled_vec4h_affine_moe",
                [out, dev.put(mb["x"]), gs, gw, moe_gate_pod_args(512, 256, slots), gb, dev.put(ids)], (64, 100, slots))
    assert be.ctx.device_errors() == 0
    got = dev.get(out)
    assert (got[..., 256:] == 7.0).all()
    got = got[..., :256]
    tiles = kind == "tiles"
    ref = oracle_c.moe_matmul_f64(mb["x"], *mb["gate"], ids, 256, 512, 64, 4, in_per_slot=False, w16=tiles)
    err = zo.rel_err_scaled(got, ref, 1e-2 if tiles else 1e-3)
    record_parity(err, zo.rel_err(got, ref))
    assert err <= TOL
    be.close()


@pytest.mark.parametrize("T,E,d,ffn,slots", [(700, 3, 256, 200, 2), (40, 5, 192, 72, 4), (1500, 2, 512, 384, 1)])
def test_tensor_memory_tiles_on_ragged_shapes(T, E, d, ffn, slots, dev, oracle_c, monkeypatch):
    """The tiles with the weights in tensor memory on shapes that are no multiple of anything convenient: N not a
    multiple of 128 (a short last row block), K of 3 k blocks, experts with several 128-pair tiles and ragged last
    tiles, more units than SMs (every CTA walks several units: both accumulator sets and every ring wrap)."""
    monkeypatch.setenv("ZTVM_MOE_GROUPED", "1")
    monkeypatch.setenv("ZTVM_MOE_TILES", "")
    be = z.backend.CudaMatmulBackend(0)
    mb = z.synth.moe_block(T, E=E, hidden=d, ffn=ffn, seed=41)
    ids = np.random.default_rng(5).integers(0, E + 1, size=(T, slots), dtype=np.uint32)
    out = dev.empty((T, slots, ffn), np.float16, fill=7.0)
    gw, gs, gb = (dev.put(a) for a in mb["gate"])
    desc = z.MoeDesc(z.MmDesc(d, ffn, 1, 64, 4, 1, 0), E + 1, slots, T, 0, ffn, d, slots * ffn, slots)
    for rep in range(2):
        be.ctx.int4_matmul_moe(desc, out, dev.put(mb["x"]), gs, gw, gb, dev.put(ids))
    assert be.ctx.device_errors() == 0
    got = dev.get(out)
    ref = oracle_c.moe_matmul_f64(mb["x"], *mb["gate"], ids, ffn, d, 64, 4, in_per_slot=False, w16=True)
    err = zo.rel_err_scaled(got, ref, 1e-2)
    record_parity(err, zo.rel_err(got, ref))
    assert err <= TOL
    be.close()


def test_plan_reuse_across_the_matmuls_of_one_step(backend, dev, oracle_c):
    """With ztvm_moe_plan_reuse on, gate / up / down over one id list build the expert-sorted plan once: same bits as
    without it; a new id list written by the router at the same address must not meet the old plan."""
    import torch
    mb = z.synth.moe_block(64, E=16, hidden=512, ffn=256, seed=61)
    slots = 5
    gw, gs, gb = (dev.put(a) for a in mb["gate"])
    uw, us, ub = (dev.put(a) for a in mb["up"])
    x = dev.put(mb["x"])
    logits = [dev.put(mb["logits"]), dev.put(np.ascontiguousarray(mb["logits"][::-1]))]
    ids = dev.empty((64, slots), np.uint32, fill=0)
    scores = dev.empty((64, slots), np.float32, fill=0.0)
    desc = z.MoeDesc(z.MmDesc(512, 256, 1, 64, 4, 1, 0), 17, slots, 64, 0, 256, 512, slots * 256, slots)
    outs = {}
    for reuse in (False, True):
        backend.ctx.moe_plan_reuse(reuse)
        for li in (0, 1):                       # the second routing overwrites ids in place
            backend.moe_router_topk(ids, scores, logits[li], 16, 4, True, True, 64)
            yg = dev.empty((64, slots, 256), np.float16, fill=3.0)
            yu = dev.empty((64, slots, 256), np.float16, fill=3.0)
            backend.ctx.int4_matmul_moe(desc, yg, x, gs, gw, gb, ids)
            backend.ctx.int4_matmul_moe(desc, yu, x, us, uw, ub, ids)
            outs[(reuse, li)] = (dev.get(yg).view(np.uint16), dev.get(yu).view(np.uint16), dev.get(ids, np.uint32).copy())
    backend.ctx.moe_plan_reuse(False)
    assert backend.ctx.device_errors() == 0
    for li in (0, 1):
        assert np.array_equal(outs[(False, li)][0], outs[(True, li)][0])
        assert np.array_equal(outs[(False, li)][1], outs[(True, li)][1])
        idn = outs[(True, li)][2]
        tiles = moe_kernel_kind(64 * slots, 17, 512, 256, 4) == "tiles"
        ref = oracle_c.moe_matmul_f64(mb["x"], *mb["up"], idn, 256, 512, 64, 4, in_per_slot=False, w16=tiles)
        err = zo.rel_err_scaled(outs[(True, li)][1].view(np.float16), ref, 1e-2 if tiles else 1e-3)
        record_parity(err, zo.rel_err(outs[(True, li)][1].view(np.float16), ref))
        assert err <= TOL
    assert not np.array_equal(outs[(True, 0)][2], outs[(True, 1)][2])


def test_moe_argument_errors(backend, dev):
    mb = z.synth.moe_block(2, E=8, hidden=256, ffn=128, seed=1)
    gw, gs, gb = (dev.put(a) for a in mb["gate"])
    out = dev.empty((2, 3, 256), np.float16)
    ids = dev.put(np.zeros((2, 3), dtype=np.uint32))
    x = dev.put(mb["x"])
    def call(**kw):
        base = dict(K=256, N=128, M=1, group=64, bits=4, affine=1, out_f32=0, experts=9, slots=3, tokens=2,
                    in_slot=0, out_slot=256, in_tok=256, out_tok=768, ids_stride=3)
        base.update(kw)
        d = z.MoeDesc(z.MmDesc(base["K"], base["N"], base["M"], base["group"], base["bits"], base["affine"],
                               base["out_f32"]), base["experts"], base["slots"], base["tokens"], base["in_slot"],
                      base["out_slot"], base["in_tok"], base["out_tok"], base["ids_stride"])
        backend.ctx.int4_matmul_moe(d, out, x, gs, gw, gb, ids)
    call()
    for kw, code in ((dict(affine=0), z.capi.ERR_UNSUPPORTED), (dict(M=4), z.capi.ERR_BAD_DIMS),
                     (dict(ids_stride=2), z.capi.ERR_BAD_DIMS), (dict(in_tok=252), z.capi.ERR_ALIGNMENT),
                     (dict(slots=0), z.capi.ERR_BAD_DIMS), (dict(out_f32=1), z.capi.ERR_UNSUPPORTED)):
        with pytest.raises(z.ZtvmError) as e:
            call(**kw)
        assert e.value.status == code, (kw, e.value)
    call(tokens=0)   # empty token list is a no-op, not an error


@pytest.mark.parametrize("T", [3, 200])
def test_expert_parallel_form_on_one_rank_matches_the_seven_dispatches(T, backend, dev):
    """sharded.ExpertParallelMoE with the CUDA kernels and a single rank (no process group): same block, other
    kernels (sorted pairs, dense shared expert), so agreement is to the whole-block bound, not bit for bit."""
    import torch
    from zero_tvm_b200 import sharded
    mb = z.synth.moe_block(T, E=16, hidden=512, ffn=256, seed=31)
    ref = run_block(backend, dev, mb, K_top=4)["y"].astype(np.float64)
    stacks = [tuple(dev.put(a) for a in mb[n]) for n in ("gate", "up", "down")]
    moe = sharded.ExpertParallelMoE(sharded.CudaKernels(backend), *stacks, E=16, top_k=4, d=512, ffn=256)
    y = moe.forward(dev.put(mb["x"]), dev.put(mb["logits"]))
    torch.cuda.synchronize()
    got = y.cpu().numpy().astype(np.float64)
    assert np.abs(got - ref).max() <= 5e-3 * np.abs(ref).max()


@pytest.mark.parametrize("T,G,E,d,ffn,top_k", [(24, 2, 8, 256, 128, 2), (300, 4, 16, 512, 256, 4), (64, 8, 64, 256, 128, 8)])
def test_peer_store_expert_parallel_step_with_ranks_emulated_on_one_gpu(T, G, E, d, ffn, top_k, backend, dev):
    """The expert-parallel step whose rows travel by stores into the owners' receive buffers, with G ranks emulated
    from one process on one GPU: every rank's buffers are plain allocations here and the kernels of the ranks run one
    after the other (dispatch of all ranks, then every rank's expert matmuls, then every combine), which is the order
    the two barriers enforce between real ranks. The result must be the block the engine's own sequence of dispatches
    computes on all tokens at once (whole-block bound: different kernels, same arithmetic)."""
    import torch
    from zero_tvm_b200 import sharded
    mb = z.synth.moe_block(T, E=E, hidden=d, ffn=ffn, seed=51)
    ref = run_block(backend, dev, mb, K_top=top_k)["y"].astype(np.float64)
    epr, tl = E // G, T // G
    k = sharded.CudaKernels(backend)
    moes, states, xs, ls = [], [], [], []
    for r in range(G):
        sel = list(range(r * epr, (r + 1) * epr)) + [E]
        stacks = [tuple(dev.put(a[sel]) for a in mb[n]) for n in ("gate", "up", "down")]
        moes.append(sharded.ExpertParallelMoE(k, *stacks, E=E, top_k=top_k, d=d, ffn=ffn, world=G, rank=r))
        xs.append(dev.put(mb["x"][r * tl:(r + 1) * tl]))
        ls.append(dev.put(mb["logits"][r * tl:(r + 1) * tl]))
    total = moes[0].peer_bytes(tl)[0]
    bufs = [torch.zeros((total,), dtype=torch.uint8, device="cuda") for _ in range(G)]
    ptrs = [b.data_ptr() for b in bufs]
    for r in range(G):
        states.append(moes[r]._peer_state(tl, xs[r].device, buf=bufs[r], ptrs=ptrs))
    for step in range(2):                      # twice: cursors and counts must come back to a clean state
        for b in (st["y_slots"] for st in states):
            b.fill_(float("nan"))
        torch.cuda.synchronize()
        for r in range(G):
            st = states[r]
            k.route_topk(st["ids"], st["scores"], ls[r], E, top_k, tl)
            k.ep_dispatch(st["layout"], st["ids"], tl, top_k, xs[r], d)
        torch.cuda.synchronize()
        counts = np.stack([st["recv_cnt"].cpu().numpy()[:G + 1] for st in states])
        assert counts[:, :G].sum() == T * top_k and (counts[:, G] == tl).all()
        for r in range(G):
            moes[r]._peer_ffn(states[r])
        torch.cuda.synchronize()
        outs = []
        for r in range(G):
            st = states[r]
            k.combine(st["out"], st["y_slots"], st["scores"], tl, top_k + 1, d)
            outs.append(st["out"])
        torch.cuda.synchronize()
        assert backend.ctx.device_errors() == 0
        got = torch.cat(outs).cpu().numpy().astype(np.float64)
        assert np.isfinite(got).all()
        assert np.abs(got - ref).max() <= 5e-3 * np.abs(ref).max(), f"step {step}"


@pytest.mark.parametrize("T", [300, 640, 4200])
def test_dispatch_plan_on_the_device_matches_the_tensor_op_plan(backend, dev, T):
    """ztvm_moe_dispatch_plan against the plan recomputed on the host: same pairs per destination, a
    permutation of all pairs in destination order, the right local expert for every pair. The sizes sit on both
    sides of the pair counts where the planner changes kernels (one block up to 32768 pairs, several above)."""
    import torch
    from zero_tvm_b200 import sharded
    K, E, world = 8, 64, 4
    epr = E // world
    rng = np.random.default_rng(17)
    ids_full = np.stack([rng.permutation(E)[:K + 1] for _ in range(T)]).astype(np.uint32)   # K routed + one more column
    ids_full[:, K] = E
    t = dev.put(ids_full)
    k = sharded.CudaKernels(backend)
    order, local, send = k.dispatch_plan(t[:, :K], epr, world)
    torch.cuda.synchronize()
    assert backend.ctx.device_errors() == 0
    order, local, send = order.cpu().numpy(), local.cpu().numpy(), send.cpu().numpy()
    flat = ids_full[:, :K].reshape(-1).astype(np.int64)
    assert np.array_equal(send, np.bincount(flat // epr, minlength=world))
    assert np.array_equal(np.sort(order), np.arange(T * K))
    dest = flat[order] // epr
    assert (np.diff(dest) >= 0).all()
    assert np.array_equal(local, (flat[order] % epr).astype(np.int32))


def test_peer_barrier_alone_and_with_a_rank_that_never_arrives(backend, dev):
    """One rank: the barrier passes at once, the epoch counts calls. Two ranks of which the second never calls: the wait
    is bounded (about a second), the expiry is reported, and the context goes on working afterwards."""
    import time
    import torch
    mine = torch.zeros(16, dtype=torch.int32, device="cuda")
    for n in range(3):
        backend.ctx.peer_barrier([mine.data_ptr()], 1, 0)
    backend.ctx.sync()
    assert backend.ctx.device_errors() == 0
    assert mine[0].item() == 3 and mine[1].item() == 3          # word 0: rank 0's arrival, word 1 (= world): the epoch
    absent = torch.zeros(16, dtype=torch.int32, device="cuda")  # the flag words of a rank that never shows up
    mine.zero_()
    t0 = time.perf_counter()
    backend.ctx.peer_barrier([mine.data_ptr(), absent.data_ptr()], 2, 0)
    with pytest.raises(z.ZtvmError) as e:
        backend.ctx.device_errors()
    waited = time.perf_counter() - t0
    assert "barrier" in str(e.value) and 0.3 < waited < 10.0, (str(e.value), waited)
    assert absent[0].item() == 1                                # this rank did announce itself to the other one
    # the status is cleared by reading it, and ordinary work still runs
    assert backend.ctx.device_errors() == 0
    p = z.synth.projection(64, 256, M=1, seed=1)
    y = dev.empty((1, 64), np.float16)
    backend.ctx.int4_matmul(z.MmDesc(256, 64, 1, 64, 4, 1, 0), y, dev.put(p["x"]), dev.put(p["scales"]), dev.put(p["W"]),
                            dev.put(p["biases"]))
    backend.ctx.sync()
    assert np.isfinite(dev.get(y)).all()


def _golden(name):
    import os
    return np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", name))


@pytest.mark.parametrize("name", ["router_ref_e64_k6_raw.npz", "router_ref_e256_k8_norm.npz", "router_ref_e16_k4_norm.npz"])
def test_router_kernel_against_the_reference_numpy_router(name, backend, dev):
    """ztvm_moe_route_topk on the vectors the reference's own numpy routing produced (see tests/golden/make_golden.py):
    the same experts in the same slots, exact ties included, and the same weights."""
    g = _golden(name)
    logits, ids, w, norm = g["logits"], g["ids"], g["weights"], bool(g["norm"])
    T, E = logits.shape
    K = ids.shape[1]
    d_ids = dev.empty((T, K), np.uint32, fill=0)
    d_w = dev.empty((T, K), np.float32, fill=0.0)
    backend.moe_router_topk(d_ids, d_w, dev.put(logits), E, K, norm, False, T)
    backend.ctx.sync()
    assert np.array_equal(dev.get(d_ids, np.uint32), ids)
    assert np.allclose(dev.get(d_w), w, rtol=3e-6, atol=1e-9)


def test_silu_kernel_against_the_reference_numpy_function(backend, dev):
    """ztvm_silu_mul on the inputs of the reference's numpy silu_mul: its f32 value rounded to f16, at most one f16 step
    away where the kernel's order of the three operations rounds differently."""
    g = _golden("silu_mul_ref.npz")
    gate, up, h = g["gate"], g["up"], g["h"]
    rows, ffn = gate.shape
    out = dev.empty((rows, ffn), np.float16, fill=float("nan"))
    backend.silu_mul(out, dev.put(np.ascontiguousarray(np.concatenate([gate, up], axis=1))), rows, ffn)
    backend.ctx.sync()
    got, want = dev.get(out), h.astype(np.float16)
    steps = np.abs(got.view(np.int16).astype(np.int32) - want.view(np.int16).astype(np.int32))
    assert steps.max() <= 1 and (steps == 0).mean() >= 0.99, (steps.max(), (steps == 0).mean())
