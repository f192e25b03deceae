"""GPU parity of the prefill GEMM (M > 8): tcgen05 MMA over weights dequantised to f16 on the fly.
Reference for the outputs: an fp64 dot product over W16 = f16(fl32(s*q+b)), the value the reference's own numpy
dequantiser produces and its matrix-unit GEMMs multiply with; W16 itself is checked bit for bit through the
dequant hook, which calls the same device function the GEMM inlines."""
import numpy as np
import pytest

import zero_tvm_b200 as z
from oracle import ztvm_oracle as zo
from conftest import record_parity
from zero_tvm_b200.backend import pick_chunk_gemm, pod_args

pytestmark = pytest.mark.gpu
TOL = 2e-3
# Tensor-core accumulation is f32 with truncation, a few bits short of a round-to-nearest f32 chain, so outputs that
# cancel to almost nothing sit further from the fp64 anchor in RELATIVE terms. The GEMM is graded like the
# reference grades its GEMMs: relative error with the floor max(1e-2, |ref|) on O(1) outputs
# (scripts/gemm-bench.mjs:516), made scale-free as 1e-2 of the output rms.
FLOOR_FRAC = 1e-2


def run_gemm(backend, dev, p, entry=None, extra_rows=0):
    M, N, K = p["M"], p["N"], p["K"]
    entry = entry or pick_chunk_gemm(None, affine=p["affine"], K=K)
    y = dev.empty((M + extra_rows, N), np.float16, fill=-77.0)
    bind = [y, dev.put(p["x"]), dev.put(p["scales"]), dev.put(p["W"]), pod_args(K, N, group=p["group"], m_rows=M)]
    if p["affine"]:
        bind.append(dev.put(p["biases"]))
    backend.dispatch(entry, bind, grid=((N + 31) // 32, (M + 63) // 64, 1))
    out = dev.get(y)
    assert backend.ctx.device_errors() == 0
    return out


def check(y, p, oracle_c):
    gemm = y.shape[0] > 16     # up to 16 rows the call runs as GEMV slabs: f32 weights, the GEMV floor
    y64 = oracle_c.matmul_f64(p["x"], p["W"], p["scales"], p["biases"], p["group"], 4, p["affine"], w16=gemm)
    assert np.isfinite(y).all()
    err = zo.rel_err_scaled(y, y64, FLOOR_FRAC if gemm else 1e-3)
    record_parity(err, zo.rel_err(y, y64))     # floored and pure-relative error, listed at the end of the run
    assert err <= TOL, f"rel err {err:.3e} (floor 1e-3 rms: {zo.rel_err_scaled(y, y64):.3e})"
    return err


@pytest.mark.parametrize("M", [64, 128, 256, 512, 1024])
def test_prefill_gemm_config(M, backend, dev, oracle_c):
    """X[M,2048] times W[8192,2048], affine group 64, the M sweep of the prefill configuration."""
    w = z.synth.projection(8192, 2048, M=1, seed=0)
    x = z.synth.make_x(np.random.default_rng([0, M]), M, 2048)
    p = dict(w, x=x, M=M)
    y = run_gemm(backend, dev, p)
    check(y, p, oracle_c)


@pytest.mark.parametrize("M,N,K", [(13, 96, 128), (9, 8, 64), (17, 96, 128), (31, 40, 320), (100, 1000, 1408), (129, 72, 192), (300, 4096, 4096),
                                   (257, 130, 768)])
def test_ragged_shapes(M, N, K, backend, dev, oracle_c):
    """13 x 96 x 128 is the reference's own GEMM gate (scripts/gemm-bench.mjs:483-498). Rows past M stay untouched."""
    p = z.synth.projection(N, K, M=M, seed=M + N)
    y = run_gemm(backend, dev, p, extra_rows=2)
    assert (y[M:] == -77.0).all()
    check(y[:M], p, oracle_c)


@pytest.mark.parametrize("entry", ["int4_matmul_sg_e5_affine", "int4_matmul_sg_e1_affine", "int4_matmul_sgmat_affine",
                                   "int4_matmul_tiled_st_affine", "int4_matmul_tiled_m_affine",
                                   "int4_matmul_batched_dyn_affine"])
def test_every_prefill_entry_lands_on_the_gemm(entry, backend, dev, oracle_c):
    p = z.synth.projection(256, 512, M=96, seed=5)
    check(run_gemm(backend, dev, p, entry=entry), p, oracle_c)


def test_symmetric_flavour(backend, dev, oracle_c):
    p = z.synth.projection(512, 1024, M=200, group=32, affine=False, seed=8)
    check(run_gemm(backend, dev, p, entry="int4_matmul_sg_e5"), p, oracle_c)


def test_gemm_agrees_with_gemv_rows(backend, dev):
    """Chunked vs per-token prefill must agree to output precision (the reference's equivalence policy,
    src/zero-tvm/engine-core.ts:3831-3837): row m of the GEMM against the M=1 GEMV of the same row."""
    p = z.synth.projection(1024, 2048, M=64, seed=2)
    y = run_gemm(backend, dev, p).astype(np.float64)
    W, s, b = dev.put(p["W"]), dev.put(p["scales"]), dev.put(p["biases"])
    for m in (0, 31, 63):
        y1 = dev.empty((1, 1024), np.float16)
        backend.dispatch("int4_matmul_tiled_vec4h_affine", [y1, dev.put(p["x"][m:m + 1]), s, W, pod_args(2048, 1024), b])
        # the GEMM multiplies with f16-rounded weights, the GEMV with the f32 ones: a difference of up to 2^-11
        # per weight, so the two agree to a few 1e-4 of the output scale, not to a relative bound per element
        d = np.abs(y[m] - dev.get(y1)[0].astype(np.float64)).max()
        assert d < 4e-3 * np.sqrt(np.mean(y[m] ** 2))   # about one f16 ulp of the largest outputs


def test_exact_properties(backend, dev):
    """Zero activations give exact zeros; doubling x doubles y exactly; permuting tokens permutes rows."""
    p = z.synth.projection(2048, 1024, M=256, seed=4)
    y1 = run_gemm(backend, dev, p)
    y0 = run_gemm(backend, dev, dict(p, x=np.zeros_like(p["x"])))
    assert (y0 == 0).all()
    y2 = run_gemm(backend, dev, dict(p, x=(p["x"].astype(np.float32) * 2).astype(np.float16)))   # doubling is exact
    big = np.abs(y1.astype(np.float32)) > 1e-3          # f16 subnormal outputs round differently before / after doubling
    assert np.array_equal(y2[big], (y1.astype(np.float32) * 2).astype(np.float16)[big])
    perm = np.random.default_rng(0).permutation(256)
    yp = run_gemm(backend, dev, dict(p, x=p["x"][perm]))
    assert np.array_equal(yp.view(np.uint16), y1[perm].view(np.uint16))


@pytest.mark.parametrize("M", [100, 130, 300])
def test_f32_output_through_the_c_abi(M, backend, dev, oracle_c):
    """out_f32 with M > 8 (no reference GEMM entry writes f32, the C ABI allows it): the shared-memory-operand kernel
    (M <= 128) and both tile widths of the weights-in-TMEM kernel, ragged N."""
    N, K = 200, 512
    p = z.synth.projection(N, K, M=M, seed=40 + M)
    y = dev.empty((M + 1, N), np.float32, fill=-77.0)
    backend.ctx.int4_matmul(z.MmDesc(K, N, M, 64, 4, 1, 1), y, dev.put(p["x"]), dev.put(p["scales"]), dev.put(p["W"]),
                            dev.put(p["biases"]))
    backend.ctx.sync()
    out = dev.get(y)
    assert backend.ctx.device_errors() == 0
    assert (out[M:] == -77.0).all()
    check(out[:M], p, oracle_c)


def test_pipelined_host_calls_equal_the_synchronous_one(backend, dev):
    """ztvm_int4_matmul_host_async on its three lanes, more calls than lanes, different activations per call: every result
    equals the synchronous host call's bit for bit; pageable buffers are refused."""
    import torch
    M, N, K = 40, 256, 512
    p = z.synth.projection(N, K, M=M, seed=21)
    s, W, b = dev.put(p["scales"]), dev.put(p["W"]), dev.put(p["biases"])
    d = z.MmDesc(K, N, M, 64, 4, 1, 0)
    rng = np.random.default_rng(4)
    xs = [torch.from_numpy(z.synth.make_x(rng, M, K)).pin_memory() for _ in range(7)]
    ys = [torch.empty((M, N), dtype=torch.float16).pin_memory() for _ in range(7)]
    ref = [torch.empty((M, N), dtype=torch.float16).pin_memory() for _ in range(7)]
    for x, y in zip(xs, ref):
        backend.ctx.int4_matmul_host(d, y, x, s, W, b)
    for x, y in zip(xs, ys):
        backend.ctx.int4_matmul_host_async(d, y, x, s, W, b)
    backend.ctx.host_wait()
    for i in range(7):
        assert torch.equal(ys[i], ref[i]), i
    assert not torch.equal(ref[0], ref[1])
    with pytest.raises(z.ZtvmError) as e:
        backend.ctx.int4_matmul_host_async(d, torch.empty((M, N), dtype=torch.float16), xs[0], s, W, b)
    assert e.value.status == z.capi.ERR_UNSUPPORTED and "page-locked" in str(e.value)
