"""GPU parity of the dense matmul path, called through the C ABI the way the engine dispatches it
(entry name + bind group + PODArgs). Codes and dequantised weights are bit-exact against the oracle;
outputs sit within 2e-3 of an fp64 dot product over the dequantised weights, graded as the reference
grades (relative error with a small floor: tests/kernels/run.mjs:153 uses |ref|+1e-3)."""
import glob
import os

import numpy as np
import pytest

import zero_tvm_b200 as z
from oracle import ztvm_oracle as zo
from zero_tvm_b200.backend import pod_args, resolve_matmul
from conftest import record_parity

pytestmark = pytest.mark.gpu
TOL = 2e-3       # the path's stated tolerance, graded with oracle.rel_err_scaled (floor = 1e-3 of the output rms)
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def run_matmul(backend, dev, p, entry=None, out_f32=False, poison=True):
    """Dispatch one projection exactly like the engine: [out, in, scales, weights, PODArgs, biases?]."""
    M, N, K = p["M"], p["N"], p["K"]
    entry = entry or resolve_matmul(affine=p["affine"], K=K, out_f32=out_f32, q3=p["bits"] == 3)
    info = z.backend.parse_entry(entry)
    y = dev.empty((M, N), np.float32 if info.out_f32 else np.float16, fill=float("nan") if poison else None)
    pod = pod_args(K, N, bits=p["bits"], group=p["group"], m_rows=M if info.has_m_rows else None)
    bind = [y, dev.put(p["x"]), dev.put(p["scales"]), dev.put(p["W"]), pod]
    if p["affine"]:
        bind.append(dev.put(p["biases"]))
    backend.dispatch(entry, bind, grid=((N + 3) // 4, 1, 1))
    return dev.get(y)


def check_y(y, p, oracle_c, w16=None, tol=TOL):
    """M <= 8 runs the GEMV (f32 weights, fp64 anchor over W32, floor 1e-3 of the output rms); more rows of 4-bit
    weights run the tensor-core GEMM (f16 weights: anchor over W16, graded with the GEMM floor of 1e-2 rms)."""
    if w16 is None:
        w16 = y.shape[0] > 16 and p["bits"] == 4
    y64 = oracle_c.matmul_f64(p["x"], p["W"], p["scales"], p["biases"], p["group"], p["bits"], p["affine"], w16=w16)
    assert np.isfinite(y).all(), "output holds NaN/inf (poison not overwritten?)"
    assert np.abs(y).max() > 0
    err = zo.rel_err_scaled(y, y64, 1e-2 if w16 else 1e-3)
    record_parity(err, zo.rel_err(y, y64))     # floored and pure-relative error, listed at the end of the run
    assert err <= tol, f"rel err {err:.3e} (pure relative {zo.rel_err(y, y64):.3e})"
    return err


# ---- bit-exact hooks ------------------------------------------------------------------------------
@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(GOLDEN, "dequant_from_*.npz"))))
def test_dequant_hook_matches_reference_vectors(path, backend, dev):
    g = np.load(path)
    N, KP = g["W"].shape
    d = z.MmDesc(KP * 8, N, 1, 64, 4, 1, 0)
    W, s, b = dev.put(g["W"]), dev.put(g["scales"]), dev.put(g["biases"])
    out16 = dev.empty((N, KP * 8), np.float16)
    backend.ctx.dequant(d, out16, True, s, W, b)
    assert np.array_equal(dev.get(out16).view(np.uint16), g["w16"].view(np.uint16))
    out32 = dev.empty((N, KP * 8), np.float32)
    backend.ctx.dequant(d, out32, False, s, W, b)
    w32 = zo.dequant_w32(zo.unpack_codes(g["W"], 4), g["scales"], g["biases"], 64)
    assert np.array_equal(dev.get(out32).view(np.uint32), w32.view(np.uint32))


@pytest.mark.parametrize("bits,group,affine,N,K", [
    (4, 64, True, 8192, 2048),     # the decode GEMV configuration
    (3, 64, True, 12288, 4096),    # the 3-bit configuration
    (4, 32, False, 1000, 1408),    # symmetric, ragged
    (3, 64, True, 13, 256),
])
def test_codes_and_dequant_bit_exact(bits, group, affine, N, K, backend, dev, oracle_c):
    p = z.synth.projection(N, K, bits=bits, group=group, affine=affine, seed=0)
    d = z.MmDesc(K, N, 1, group, bits, int(affine), 0)
    W, s = dev.put(p["W"]), dev.put(p["scales"])
    b = dev.put(p["biases"]) if affine else None
    codes = dev.empty((N, K), np.uint8, fill=255)
    backend.ctx.unpack_codes(d, codes, W)
    assert np.array_equal(dev.get(codes), p["q"])
    # the in-place subnormal codes the streaming matrix-unit kernels multiply with (their own mask functions)
    codes_s = dev.empty((N, K), np.uint8, fill=255)
    backend.ctx.unpack_codes_streamed(d, codes_s, W)
    assert np.array_equal(dev.get(codes_s), p["q"])
    for as_f16 in (False, True):
        out = dev.empty((N, K), np.float16 if as_f16 else np.float32)
        backend.ctx.dequant(d, out, as_f16, s, W, b)
        ref = oracle_c.dequant(p["W"], p["scales"], p["biases"], group, bits, affine, out_f16=as_f16)
        got = dev.get(out)
        assert np.array_equal(got.view(np.uint16 if as_f16 else np.uint32), ref.view(np.uint16 if as_f16 else np.uint32))


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(GOLDEN, "kernel_ref_*.npz"))))
def test_kernel_ref_vectors(path, backend, dev):
    """Vectors produced by the reference's own numpy statements (scripts/make-kernel-ref.py:55-66): both code hooks
    bit-exact against its unpack (4-bit nibbles, 3-bit bit stream), the GEMV within 2e-3 of its factored y."""
    g = np.load(path)
    bits = int(g["bits"])
    N, K = g["codes"].shape
    d = z.MmDesc(K, N, 1, 64, bits, 1, 0)
    W = dev.put(g["W"])
    for hook in (backend.ctx.unpack_codes, backend.ctx.unpack_codes_streamed):
        codes = dev.empty((N, K), np.uint8, fill=255)
        hook(d, codes, W)
        assert np.array_equal(dev.get(codes), g["codes"]), hook.__name__
    p = dict(x=g["x"].reshape(1, K), W=g["W"], scales=g["scales"], biases=g["biases"], N=N, K=K, M=1, bits=bits,
             group=64, affine=True)
    y = run_matmul(backend, dev, p, out_f32=True)[0]
    err = zo.rel_err_scaled(y, g["y"], 1e-3)
    record_parity(err, zo.rel_err(y, g["y"]))
    assert err <= TOL, f"rel err {err:.3e} against the reference's factored y"


# ---- the reference's own kernel tests ----------------------------------------------------------------
@pytest.mark.parametrize("K", [512, 768, 1024, 1408])
@pytest.mark.parametrize("entry,flavour", [
    ("int4_matmul", "symmetric"), ("int4_matmul_sg", "symmetric"), ("int4_matmul_tiled", "symmetric"),
    ("int4_matmul_f32_tiled8", "symmetric"), ("int4_matmul_affine", "affine"),
    ("int4_matmul_tiled_affine", "affine"), ("int4_matmul_f32_tiled_affine", "affine"),
    ("int4_matmul_affine_q3", "affine_q3"), ("int4_matmul_tiled_affine_q3", "affine_q3"),
])
def test_reference_kernel_cases(K, entry, flavour, backend, dev):
    """makeInt4MatmulTest (tests/kernels/run.mjs:77-157): 8 rows, seeded inputs, f64 reference loop,
    pass when max |got-ref|/(|ref|+1e-3) < 0.02. Same inputs, same metric; we also hold our own 2e-3."""
    case = zo.reference_test_case(K, affine=flavour != "symmetric", q3=flavour == "affine_q3")
    p = dict(x=case["x"][None], W=case["W"], scales=case["scales"], biases=case["biases"], M=1, N=8, K=K,
             bits=case["bits"], group=case["group"], affine=case["affine"])
    y = run_matmul(backend, dev, p, entry=entry)[0].astype(np.float64)
    ref = zo.reference_test_expected(case)
    ref = ref if "_f32" in entry else zo.to_f16(ref).astype(np.float64)
    err = np.max(np.abs(y - ref) / (np.abs(ref) + 1e-3))
    assert err < TOL, err


@pytest.mark.parametrize("K", [512, 1024])
@pytest.mark.parametrize("wide,flavour", [("_vec4", "symmetric"), ("_vec4h", "symmetric"), ("_vec4h", "affine")])
def test_reference_wide_load_cases(K, wide, flavour, backend, dev):
    """The wide-load rungs (run.mjs:1131-1198): different WGSL, same arithmetic, same CUDA kernel."""
    case = zo.reference_test_case(K, affine=flavour == "affine")
    entry = "int4_matmul_tiled" + wide + ("_affine" if flavour == "affine" else "")
    p = dict(x=case["x"][None], W=case["W"], scales=case["scales"], biases=case["biases"], M=1, N=8, K=K,
             bits=4, group=case["group"], affine=case["affine"])
    y = run_matmul(backend, dev, p, entry=entry)[0].astype(np.float64)
    ref = zo.to_f16(zo.reference_test_expected(case)).astype(np.float64)
    assert np.max(np.abs(y - ref) / (np.abs(ref) + 1e-3)) < TOL


# ---- the benchmark configurations ----------------------------------------------------------------------
def test_decode_gemv_config(backend, dev, oracle_c):
    """x[1,2048] times W[8192,2048], affine group 64, seed 0, f16 out."""
    p = z.synth.projection(8192, 2048, seed=0)
    y = run_matmul(backend, dev, p)
    check_y(y, p, oracle_c)
    # the reference-order f32 GEMV on the CPU lands on (almost always) the same f16 values
    yref = oracle_c.gemv_ref(p["x"], p["W"], p["scales"], p["biases"], 64)
    assert zo.rel_err_scaled(y, yref.astype(np.float64)) < TOL


def test_int3_gemv_config(backend, dev, oracle_c):
    """x[1,4096] times W[12288,4096] in 3-bit codes, group 64."""
    p = z.synth.projection(12288, 4096, bits=3, seed=0)
    y = run_matmul(backend, dev, p)
    check_y(y, p, oracle_c)


@pytest.mark.parametrize("N,K", [(13, 256), (100, 768), (301, 8192), (2000, 12288)])
def test_int3_streaming_kernel_shapes(N, K, backend, dev, oracle_c):
    """The 3-bit streaming GEMV over one, three and more than sixteen K slices (the last two run several K tiles
    with their running sums in shared memory), rows that do not fill the 16-row tiles."""
    p = z.synth.projection(N, K, bits=3, seed=N)
    check_y(run_matmul(backend, dev, p), p, oracle_c)
    check_y(run_matmul(backend, dev, p, out_f32=True), p, oracle_c)


@pytest.mark.parametrize("name,N,K,f32", z.synth.DENSE_LAYER_SET)
@pytest.mark.parametrize("M", [1, 4])
def test_dense_layer_set(name, N, K, f32, M, backend, dev, oracle_c):
    if name == "up_proj":
        pytest.skip("same shape as gate_proj")
    seed = [n for n, *_ in z.synth.DENSE_LAYER_SET].index(name)
    p = z.synth.projection(N, K, M=M, seed=seed)
    entry = ("int4_matmul_batched_dyn_affine" if M > 1 and not f32 else None)
    if M > 1 and f32:
        # the engine runs the lm_head per row with the f32 GEMV (engine-core.ts:2543-2549)
        ys = []
        for m in range(M):
            pm = dict(p, x=p["x"][m:m + 1], M=1)
            ys.append(run_matmul(backend, dev, pm, out_f32=True))
        y = np.concatenate(ys, 0)
    else:
        y = run_matmul(backend, dev, p, entry=entry, out_f32=f32)
    check_y(y, p, oracle_c)


# ---- shapes the reference tests for raggedness -------------------------------------------------------------
@pytest.mark.parametrize("M", [1, 2, 3, 4, 5, 7, 8, 13])
@pytest.mark.parametrize("N,K", [(96, 128), (13, 768), (1001, 1408), (260, 4096)])
def test_ragged_batched(M, N, K, backend, dev, oracle_c):
    """13 x 96 x 128 is the reference's GEMM gate shape (scripts/gemm-bench.mjs:483-498); rows past M
    must not be written (writes are guarded by M_ROWS, int4_matmul.gen.ts:625-628)."""
    p = z.synth.projection(N, K, M=M, seed=M * 7 + N)
    yfull = dev.empty((M + 3, N), np.float16, fill=-77.0)
    bind = [yfull, dev.put(p["x"]), dev.put(p["scales"]), dev.put(p["W"]), pod_args(K, N, m_rows=M),
            dev.put(p["biases"])]
    backend.dispatch("int4_matmul_batched_dyn_affine", bind)
    got = dev.get(yfull)
    assert (got[M:] == -77.0).all(), "rows past M_ROWS were written"
    check_y(got[:M], p, oracle_c)


def test_batched_m4_fixed(backend, dev, oracle_c):
    """int4_matmul_batched_m4: symmetric, fixed M = 4 (int4_matmul.gen.ts:465-516)."""
    p = z.synth.projection(512, 3072, M=4, group=32, affine=False, seed=3)
    y = run_matmul(backend, dev, p, entry="int4_matmul_batched_m4")
    check_y(y, p, oracle_c)


def test_ragged_unit_count(backend, dev, oracle_c):
    """K = 320 is ten 32-code units: fewer than one unit per lane, the loop must keep the tail
    (the trip-count truncation the reference fixed, tests/kernels/run.mjs:1169-1198)."""
    p = z.synth.projection(40, 320, seed=5)
    check_y(run_matmul(backend, dev, p), p, oracle_c)
    p = z.synth.projection(40, 2112, seed=6)   # 66 units: two full lane rounds plus two
    check_y(run_matmul(backend, dev, p), p, oracle_c)


# ---- size-independent properties at full size -----------------------------------------------------------------
def test_exact_properties_full_size(backend, dev):
    """Zero input gives exact zeros; scaling x by a power of two scales y exactly; permuting weight rows
    permutes the outputs bit for bit. Holds at any size, checked at the lm_head shape."""
    N, K = 151936, 4096
    p = z.synth.projection(N, K, seed=7)
    y1 = run_matmul(backend, dev, p, out_f32=True)
    y2 = run_matmul(backend, dev, dict(p, x=(p["x"].astype(np.float32) * 0.5).astype(np.float16)), out_f32=True)
    assert np.array_equal(y2, y1 * np.float32(0.5))
    y0 = run_matmul(backend, dev, dict(p, x=np.zeros_like(p["x"])), out_f32=True)
    assert (y0 == 0).all()
    perm = np.random.default_rng(0).permutation(N)
    pp = dict(p, W=p["W"][perm], scales=p["scales"][perm], biases=p["biases"][perm])
    yp = run_matmul(backend, dev, pp, out_f32=True)
    assert np.array_equal(yp, y1[:, perm])


def test_mutations_are_caught(backend, dev, oracle_c):
    """The reference's mutation gate (scripts/mutation-gate.mjs): a wrong scale-group shift or a dropped
    bias must turn the parity check red. Here the mutation is applied to the ORACLE's inputs."""
    p = z.synth.projection(256, 1024, seed=11)
    y = run_matmul(backend, dev, p)
    check_y(y, p, oracle_c)
    nobias = dict(p, biases=np.zeros_like(p["biases"]))
    y64 = oracle_c.matmul_f64(nobias["x"], nobias["W"], nobias["scales"], nobias["biases"], 64)
    assert zo.rel_err_scaled(y, y64) > 10 * TOL
    shifted = dict(p, scales=np.roll(p["scales"], 1, axis=1))
    y64 = oracle_c.matmul_f64(shifted["x"], shifted["W"], shifted["scales"], shifted["biases"], 64)
    assert zo.rel_err_scaled(y, y64) > 10 * TOL


# ---- errors come back as codes, before any launch ---------------------------------------------------------------
def test_argument_errors(backend, dev):
    c = backend.ctx
    p = z.synth.projection(64, 256, seed=1)
    y = dev.empty((1, 64), np.float16, fill=5.0)
    x, s, W, b = dev.put(p["x"]), dev.put(p["scales"]), dev.put(p["W"]), dev.put(p["biases"])
    cases = [
        (z.MmDesc(256, 64, 1, 64, 5, 1, 0), z.capi.ERR_UNSUPPORTED),   # bits
        (z.MmDesc(256, 64, 1, 64, 3, 0, 0), z.capi.ERR_UNSUPPORTED),   # 3-bit symmetric
        (z.MmDesc(256, 64, 1, 48, 4, 1, 0), z.capi.ERR_BAD_DIMS),      # group not a power of two
        (z.MmDesc(200, 64, 1, 64, 4, 1, 0), z.capi.ERR_BAD_DIMS),      # K % group
        (z.MmDesc(256, 0, 1, 64, 4, 1, 0), z.capi.ERR_BAD_DIMS),
        (z.MmDesc(256, 64, 0, 64, 4, 1, 0), z.capi.ERR_BAD_DIMS),
    ]
    for d, code in cases:
        with pytest.raises(z.ZtvmError) as e:
            c.int4_matmul(d, y, x, s, W, b)
        assert e.value.status == code, (e.value, code)
    d = z.MmDesc(256, 64, 1, 64, 4, 1, 0)
    with pytest.raises(z.ZtvmError) as e:
        c.int4_matmul(d, y, x, s, W, None)                  # affine without biases
    assert e.value.status == z.capi.ERR_NULL_POINTER
    with pytest.raises(z.ZtvmError) as e:
        c.int4_matmul(d, y, x.data_ptr() + 2, s, W, b)      # misaligned activations
    assert e.value.status == z.capi.ERR_ALIGNMENT
    assert (dev.get(y) == 5.0).all(), "a refused call must not launch"


def test_host_buffer_entry_point(backend, dev, oracle_c):
    p = z.synth.projection(1024, 2048, M=4, seed=2)
    d = z.MmDesc(2048, 1024, 4, 64, 4, 1, 0)
    y = np.empty((4, 1024), dtype=np.float16)
    backend.ctx.int4_matmul_host(d, y, np.ascontiguousarray(p["x"]), dev.put(p["scales"]), dev.put(p["W"]),
                                 dev.put(p["biases"]))
    check_y(y, p, oracle_c)
    # page-locked caller buffers take the direct DMA path (no staging copy): same bits; mixed pinned / pageable too
    import torch
    xp = torch.from_numpy(np.ascontiguousarray(p["x"])).pin_memory()
    yp = torch.zeros((4, 1024), dtype=torch.float16).pin_memory()
    W, s_, b = dev.put(p["W"]), dev.put(p["scales"]), dev.put(p["biases"])
    backend.ctx.int4_matmul_host(d, yp, xp, s_, W, b)
    assert np.array_equal(yp.numpy().view(np.uint16), y.view(np.uint16))
    y2 = np.zeros((4, 1024), dtype=np.float16)
    backend.ctx.int4_matmul_host(d, y2, xp, s_, W, b)
    assert np.array_equal(y2.view(np.uint16), y.view(np.uint16))


def test_multi_destination_matmul_matches_the_single_destination_call(backend, dev, oracle_c):
    """ztvm_int4_matmul_multi: the shard [M, N] lands at a column offset inside three wider outputs (stand-ins for the
    ranks' full outputs), bit-identical to ztvm_int4_matmul, and nothing else in those outputs is touched."""
    N, K, M, N_total, lo = 1024, 2048, 4, 2560, 512
    p = z.synth.projection(N, K, M=M, seed=5)
    W, s, b, x = (dev.put(p[k]) for k in ("W", "scales", "biases", "x"))
    y_ref = dev.empty((M, N), np.float16)
    backend.ctx.int4_matmul(z.MmDesc(K, N, M, 64, 4, 1, 0), y_ref, x, s, W, b)
    outs = [dev.empty((M, N_total), np.float16, fill=3.0) for _ in range(3)]
    backend.ctx.int4_matmul_multi(z.MmDesc(K, N, M, 64, 4, 1, 0), [o.data_ptr() + lo * 2 for o in outs], N_total, x, s, W, b)
    backend.ctx.sync()
    ref = dev.get(y_ref).view(np.uint16)
    for o in outs:
        got = dev.get(o)
        assert np.array_equal(got[:, lo:lo + N].view(np.uint16), ref)
        assert (got[:, :lo] == 3.0).all() and (got[:, lo + N:] == 3.0).all()
    with pytest.raises(z.ZtvmError) as e:   # shapes the persistent GEMV does not take are refused, not rerouted
        backend.ctx.int4_matmul_multi(z.MmDesc(K, N, 16, 64, 4, 1, 0), [outs[0]], N_total, x, s, W, b)
    assert e.value.status == z.capi.ERR_UNSUPPORTED
