"""GPU parity of the rows next to the matmul path on the same C ABI: router-logit matvec (8-bit, 4-bit, f16), embedding
row gather (4-bit, 8-bit) and the 8-bit twins of the dense matmul, each called the way the engine binds them."""
import numpy as np
import pytest

import zero_tvm_b200 as z
from oracle import ztvm_oracle as zo
from conftest import record_parity
from zero_tvm_b200.backend import pod_args

pytestmark = pytest.mark.gpu
TOL = 2e-3


@pytest.mark.parametrize("bits,entry", [(8, "moe_router_logits"), (4, "moe_router_logits_q4"), (16, "moe_router_logits_f16")])
def test_router_logits_reference_case(bits, entry, backend, dev):
    """The reference's own test inputs and gate: max |got - ref| / (|ref| + 1e-2) < 1e-4 (tests/kernels/run.mjs:268-275)."""
    case = zo.reference_router_case(bits)
    ref = zo.reference_router_expected(case)
    rows, D = 9, 2048
    logits = dev.empty((rows,), np.float32, fill=float("nan"))
    x, w = dev.put(case["x"]), dev.put(case["w"])
    bind = [logits, x, w, [D, rows]] if bits == 16 else [logits, x, w, dev.put(case["scales"]), dev.put(case["biases"]), [D, rows]]
    backend.dispatch_router_logits(entry, bind, grid=(rows, 1, 1))
    got = dev.get(logits)
    err = float(np.max(np.abs(got - ref) / (np.abs(ref) + 1e-2)))
    record_parity(err, zo.rel_err(got, ref))
    assert err < 1e-4, err


@pytest.mark.parametrize("bits", [8, 4, 16])
@pytest.mark.parametrize("T", [1, 5, 64])
def test_router_logits_block_shape(bits, T, backend, dev, oracle_c):
    """257 rows (256 experts + the shared expert's gate) x hidden 2048, T tokens: exact-code f32 accumulation at every T."""
    rng = np.random.default_rng(40 + bits + T)
    D, rows = 2048, 257
    x = z.synth.make_x(rng, T, D)
    logits = dev.empty((T, rows), np.float32, fill=float("nan"))
    if bits == 16:
        w = (rng.standard_normal((rows, D), dtype=np.float32) * np.float32(0.05)).astype(np.float16)
        backend.ctx.moe_router_logits(D, rows, T, 16, logits, dev.put(x), dev.put(w))
        ref = zo.router_logits_f64(x, w, bits=16)
    else:
        _, W, s, b = z.synth.make_weights(rng, rows, D, bits=bits)
        backend.ctx.moe_router_logits(D, rows, T, bits, logits, dev.put(x), dev.put(W), dev.put(s), dev.put(b))
        ref = zo.router_logits_f64(x, W, s, b, bits)
    got = dev.get(logits)
    assert np.isfinite(got).all()
    err = zo.rel_err_scaled(got, ref, 1e-3)
    record_parity(err, zo.rel_err(got, ref))
    assert err <= TOL, err
    # logits feed a softmax: what matters is the absolute error against their spread (f32 accumulation, f32 output)
    assert np.abs(got - ref).max() <= 1e-5 * np.sqrt(np.mean(ref * ref))


@pytest.mark.parametrize("bits,entry", [(4, "embedding_affine"), (8, "embedding_affine_int8")])
def test_embedding_rows_bit_exact(bits, entry, backend, dev):
    rng = np.random.default_rng(50 + bits)
    vocab, D = 300, 512
    _, W, s, b = z.synth.make_weights(rng, vocab, D, bits=bits)
    ids = rng.integers(0, vocab, size=37, dtype=np.int32)
    ids[5] = vocab + 3          # out of range: counted, row untouched
    out = dev.empty((37, D), np.float16, fill=9.0)
    backend.dispatch_embedding(entry, [out, dev.put(ids), dev.put(s), dev.put(W), [37, (37 * D + 255) // 256], dev.put(b)], D)
    assert backend.ctx.device_errors() == 1
    got = dev.get(out)
    ok = np.ones(37, bool); ok[5] = False
    ref = zo.embedding_rows(ids[ok], W, s, b, bits)
    assert np.array_equal(got[ok].view(np.uint16), ref.view(np.uint16))
    assert (got[5] == 9.0).all()


@pytest.mark.parametrize("M,N,K", [(1, 512, 1024), (1, 300, 2048), (3, 256, 768), (8, 128, 4096), (20, 96, 512)])
def test_int8_affine_matmul(M, N, K, backend, dev, oracle_c):
    """int8_affine_matvec / int8_affine_batched: codes and weights bit-exact through the hooks, y within 2e-3 of the f64 anchor."""
    p = z.synth.projection(N, K, M=M, bits=8, seed=70 + M)
    d = z.MmDesc(K, N, 1, 64, 8, 1, 0)
    W, s, b = dev.put(p["W"]), dev.put(p["scales"]), dev.put(p["biases"])
    codes = dev.empty((N, K), np.uint8, fill=1)
    backend.ctx.unpack_codes(d, codes, W)
    assert np.array_equal(dev.get(codes), p["q"])
    for as_f16 in (False, True):
        out = dev.empty((N, K), np.float16 if as_f16 else np.float32)
        backend.ctx.dequant(d, out, as_f16, s, W, b)
        ref = oracle_c.dequant(p["W"], p["scales"], p["biases"], 64, 8, True, out_f16=as_f16)
        assert np.array_equal(dev.get(out).view(np.uint16 if as_f16 else np.uint32), ref.view(np.uint16 if as_f16 else np.uint32))
    entry = "int8_affine_matvec" if M == 1 else "int8_affine_batched"
    y = dev.empty((M, N), np.float16, fill=float("nan"))
    backend.dispatch(entry, [y, dev.put(p["x"]), s, W, pod_args(K, N, bits=8, m_rows=None if M == 1 else M), b], grid=(N, M, 1))
    got = dev.get(y)
    y64 = oracle_c.matmul_f64(p["x"], p["W"], p["scales"], p["biases"], 64, 8, True)
    err = zo.rel_err_scaled(got, y64, 1e-3)
    record_parity(err, zo.rel_err(got, y64))
    assert np.isfinite(got).all() and err <= TOL, err


def test_argument_errors(backend, dev):
    x = dev.empty((1, 256), np.float16, fill=0.0)
    w = dev.empty((4, 64), np.uint32)
    sb = dev.empty((4, 4), np.float16, fill=0.0)
    out = dev.empty((4,), np.float32)
    with pytest.raises(z.ZtvmError) as e:
        backend.ctx.moe_router_logits(256, 4, 1, 5, out, x, w, sb, sb)
    assert e.value.status == z.capi.ERR_UNSUPPORTED
    with pytest.raises(z.ZtvmError) as e:
        backend.ctx.embedding_affine(100, 4, 4, 1, x, dev.put(np.zeros(1, np.int32)), sb, w, sb)
    assert e.value.status == z.capi.ERR_BAD_DIMS
    with pytest.raises(z.ZtvmError) as e:      # 8-bit exists in the affine layout only
        backend.ctx.int4_matmul(z.MmDesc(256, 4, 1, 64, 8, 0, 0), out, x, sb, w, None)
    assert e.value.status == z.capi.ERR_UNSUPPORTED
    with pytest.raises(KeyError):
        backend.dispatch_router_logits("moe_router_logits_q2", [out, x, w, sb, sb, [256, 4]])
