"""GPU parity of the fused FFN front half (gate and up dot products + SiLU * up in one call): the one-launch paired form
of the persistent GEMV and the two-launch form on the shapes it does not take, against the fp64 anchor and against the
unfused calls of the same library."""
import numpy as np
import pytest

import zero_tvm_b200 as z
from oracle import ztvm_oracle as zo
from conftest import record_parity

pytestmark = pytest.mark.gpu
TOL = 2e-3


def run_fused(backend, dev, p, ffn, M):
    h = dev.empty((M, ffn), np.float16, fill=float("nan"))
    desc = z.MmDesc(p["K"], ffn, M, p["group"], p["bits"], int(p["affine"]), 0)
    backend.ctx.fused_ffn(desc, h, dev.put(p["x"]), dev.put(p["scales"]), dev.put(p["W"]),
                          dev.put(p["biases"]) if p["affine"] else None)
    backend.ctx.sync()
    assert backend.ctx.device_errors() == 0
    return dev.get(h)


# (ffn, K, M): rows that split unevenly over 148 CTAs, a partial last tile, K beyond one K tile (accumulators carried
# between K tiles), one to eight tokens
@pytest.mark.parametrize("ffn,K,M", [(512, 2048, 1), (12288, 4096, 1), (1000, 512, 3), (24, 256, 1), (2048, 8192, 2),
                                     (1536, 2048, 8), (9, 256, 5)])
def test_paired_gemv_against_the_anchor(ffn, K, M, backend, dev):
    p = z.synth.projection(2 * ffn, K, M=M, seed=ffn + K + M)
    got = run_fused(backend, dev, p, ffn, M).astype(np.float64)
    assert np.isfinite(got).all()
    ref = zo.fused_ffn_f64(p["x"], p["W"], p["scales"], p["biases"], ffn)
    err = zo.rel_err_scaled(got, ref, 1e-3)
    record_parity(err, zo.rel_err(got, ref))
    assert err <= TOL, err


def test_paired_gemv_symmetric_flavour(backend, dev):
    """w = s * (q - 7) at group 64 takes the one-launch form too (the reference's fused_ffn is symmetric, at group 32)."""
    ffn, K, M = 640, 1024, 2
    p = z.synth.projection(2 * ffn, K, M=M, seed=91, affine=False)
    got = run_fused(backend, dev, p, ffn, M).astype(np.float64)
    ref = zo.fused_ffn_f64(p["x"], p["W"], p["scales"], p["biases"], ffn, 64, 4, False)
    err = zo.rel_err_scaled(got, ref, 1e-3)
    record_parity(err, zo.rel_err(got, ref))
    assert np.isfinite(got).all() and err <= TOL, err


def test_small_case_matches_the_shader_arithmetic(backend, dev):
    """Against the shader's own order of operations in f32 (word-order dot products, f32 SiLU, one f16 rounding):
    at most one f16 unit in the last place apart on all but a few outputs, none further than 2e-3."""
    ffn, K = 96, 512
    p = z.synth.projection(2 * ffn, K, M=1, seed=77)
    got = run_fused(backend, dev, p, ffn, 1)
    ref = zo.fused_ffn_f32(p["x"], p["W"], p["scales"], p["biases"], ffn)
    ulps = np.abs(got.view(np.int16).astype(np.int32) - ref.view(np.int16).astype(np.int32))
    assert (ulps <= 1).mean() >= 0.97 and zo.rel_err_scaled(got.astype(np.float64), ref.astype(np.float64), 1e-3) <= TOL


@pytest.mark.parametrize("group,bits,affine,M", [(32, 4, False, 1), (128, 4, True, 2), (64, 3, True, 1), (64, 8, True, 1),
                                                 (64, 4, True, 40), (64, 4, True, 300)])
def test_two_launch_form_on_other_shapes(group, bits, affine, M, backend, dev):
    """Symmetric group 32 is the reference's own fused_ffn flavour; 3-bit, 8-bit, group 128 and M > 8 take the same path."""
    ffn, K = 384, 1024 if bits != 3 else 768
    p = z.synth.projection(2 * ffn, K, M=M, seed=group + bits + M, bits=bits, group=group, affine=affine)
    got = run_fused(backend, dev, p, ffn, M).astype(np.float64)
    w16 = M > 16 and bits == 4                     # the tensor-core GEMM multiplies f16-rounded weights
    q = zo.unpack_codes(p["W"], bits)
    Wdq = (zo.dequant_w16 if w16 else zo.dequant_w32)(q, p["scales"], p["biases"], group, affine)
    y = zo.matmul_f64(p["x"], Wdq)
    g, u = y[:, :ffn], y[:, ffn:]
    ref = u * g / (1.0 + np.exp(-g))
    err = zo.rel_err_scaled(got, ref, 1e-2 if w16 else 1e-3)
    record_parity(err, zo.rel_err(got, ref))
    assert err <= TOL, err


def test_fused_equals_unfused_to_output_precision(backend, dev):
    """gate_up matmul + silu_mul (the engine's three-dispatch affine path, f16 between the two) against the fused call:
    same inputs, results agree to the f16 rounding of the intermediate."""
    ffn, K, M = 2048, 2048, 4
    p = z.synth.projection(2 * ffn, K, M=M, seed=5)
    fused = run_fused(backend, dev, p, ffn, M).astype(np.float64)
    gu = dev.empty((M, 2 * ffn), np.float16)
    h = dev.empty((M, ffn), np.float16)
    backend.ctx.int4_matmul(z.MmDesc(K, 2 * ffn, M, 64, 4, 1, 0), gu, dev.put(p["x"]), dev.put(p["scales"]), dev.put(p["W"]),
                            dev.put(p["biases"]))
    backend.ctx.silu_mul(M, ffn, h, gu)
    backend.ctx.sync()
    unfused = dev.get(h).astype(np.float64)
    assert zo.rel_err_scaled(fused, unfused, 1e-3) <= 4e-3


def test_dispatch_names_and_refusals(backend, dev):
    ffn, K = 64, 256
    p = z.synth.projection(2 * ffn, K, M=1, seed=3)
    h = dev.empty((1, ffn), np.float16)
    x, s, w, b = dev.put(p["x"]), dev.put(p["scales"]), dev.put(p["W"]), dev.put(p["biases"])
    backend.dispatch_fused_ffn("fused_ffn_affine", [h, x, s, w, [ffn], b], D=K, ffn=ffn)
    backend.ctx.sync()
    ref = zo.fused_ffn_f64(p["x"], p["W"], p["scales"], p["biases"], ffn)
    assert zo.rel_err_scaled(dev.get(h).astype(np.float64), ref, 1e-3) <= TOL
    with pytest.raises(KeyError):
        backend.dispatch_fused_ffn("fused_ffn_q9", [h, x, s, w, [ffn], b], D=K, ffn=ffn)
    with pytest.raises(ValueError):
        backend.dispatch_fused_ffn("fused_ffn_affine", [h, x, s, w, [ffn]], D=K, ffn=ffn)
    with pytest.raises(z.ZtvmError) as e:
        backend.ctx.fused_ffn(z.MmDesc(K, ffn, 1, 64, 4, 1, 1), h, x, s, w, b)
    assert e.value.status == z.capi.ERR_UNSUPPORTED
