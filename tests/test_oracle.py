"""CPU tests of the oracle itself: golden vectors from the reference's own numpy dequantiser,
agreement of the numpy and C restatements, and the reference's own test cases and tolerance."""
import glob
import os

import numpy as np
import pytest

from oracle import ztvm_oracle as zo

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(GOLDEN, "dequant_from_*.npz"))))
def test_dequant_matches_reference_dequant_from(path, oracle_c):
    """W16 must equal, bit for bit, what scripts/make-dsv2-layer-ref.py:102-116 produced."""
    g = np.load(path)
    q = zo.unpack_codes(g["W"], 4)
    w16 = zo.dequant_w16(q, g["scales"], g["biases"], 64)
    assert w16.dtype == np.float16
    assert np.array_equal(w16.view(np.uint16), g["w16"].view(np.uint16))
    w16c = oracle_c.dequant(g["W"], g["scales"], g["biases"], 64, 4, out_f16=True)
    assert np.array_equal(w16c.view(np.uint16), g["w16"].view(np.uint16))
    # fma and mul+add agree for W32 (s*q is exact in f32)
    w32 = zo.dequant_w32(q, g["scales"], g["biases"], 64)
    w32c = oracle_c.dequant(g["W"], g["scales"], g["biases"], 64, 4)
    assert np.array_equal(w32.view(np.uint32), w32c.view(np.uint32))
    s64 = g["scales"].astype(np.float64).repeat(64, 1)
    b64 = g["biases"].astype(np.float64).repeat(64, 1)
    assert np.array_equal((s64 * q + b64).astype(np.float32), w32)


def test_golden_files_present():
    assert len(glob.glob(os.path.join(GOLDEN, "dequant_from_*.npz"))) >= 4
    assert len(glob.glob(os.path.join(GOLDEN, "kernel_ref_q3_*.npz"))) >= 3
    assert len(glob.glob(os.path.join(GOLDEN, "kernel_ref_q4_*.npz"))) >= 2


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(GOLDEN, "kernel_ref_*.npz"))))
def test_unpack_and_factored_gemv_match_reference_kernel_ref(path, oracle_c):
    """Codes must equal, bit for bit, what the unpack statements of scripts/make-kernel-ref.py:55-63 produced (4-bit
    nibbles, 3-bit LSB-first bit stream); y must sit within 2e-3 of its factored reference
    y = sum_g s_g*dot_g + b_g*xsum_g (lines 64-66), for the f64 anchor and for the reference-order f32 GEMV."""
    g = np.load(path)
    bits = int(g["bits"])
    assert np.array_equal(zo.unpack_codes(g["W"], bits), g["codes"])
    assert np.array_equal(oracle_c.unpack_codes(g["W"], bits), g["codes"])
    if bits == 3:
        assert np.array_equal(zo.unpack_codes_q3_window(g["W"]), g["codes"])
    assert np.array_equal(zo.pack_codes(g["codes"], bits), g["W"])
    x = g["x"].reshape(1, -1)
    w32 = zo.dequant_w32(g["codes"], g["scales"], g["biases"], 64)
    y64 = zo.matmul_f64(x, w32)[0]
    assert zo.rel_err_scaled(g["y"], y64, 1e-3) <= 2e-3
    for got in (zo.gemv_word_order_f32(x, g["W"], g["scales"], g["biases"], 64, bits)[0],
                oracle_c.gemv_ref(x, g["W"], g["scales"], g["biases"], 64, bits, True, out_f32=True)[0],
                oracle_c.matmul_f64(x, g["W"], g["scales"], g["biases"], 64, bits)[0]):
        assert zo.rel_err_scaled(got, g["y"], 1e-3) <= 2e-3


@pytest.mark.parametrize("bits", [16, 8, 4])
def test_router_logits_reference_case(bits, oracle_c):
    """The reference's own router test (tests/kernels/run.mjs:186-283: mulberry32 seed 11 + bits, D 2048, 9 rows, its
    formula in f64) through the oracle: the f64 anchor equals its reference loop, and the shader's word order in f32 sits
    inside its gate max |got - ref| / (|ref| + 1e-2) < 1e-4."""
    case = zo.reference_router_case(bits)
    ref = zo.reference_router_expected(case)
    y64 = zo.router_logits_f64(case["x"], case["w"], case.get("scales"), case.get("biases"), bits)[0]
    assert np.max(np.abs(y64 - ref) / (np.abs(ref) + 1e-2)) < 1e-9
    if bits != 16:
        got = zo.router_logits_word_order_f32(case["x"], case["w"], case["scales"], case["biases"], bits)
        assert np.max(np.abs(got - ref) / (np.abs(ref) + 1e-2)) < 1e-4
        gc = oracle_c.gemv_ref(case["x"].reshape(1, -1), case["w"], case["scales"], case["biases"], 64, bits, True, out_f32=True)[0]
        assert np.max(np.abs(gc - ref) / (np.abs(ref) + 1e-2)) < 1e-4


def test_embedding_rows_are_the_canonical_w16(oracle_c):
    import zero_tvm_b200 as z
    for bits in (4, 8):
        rng = np.random.default_rng(31 + bits)
        q, W, s, b = z.synth.make_weights(rng, 50, 256, bits=bits)
        ids = np.array([3, 49, 0, 3, 17], dtype=np.int32)
        rows = zo.embedding_rows(ids, W, s, b, bits)
        full = oracle_c.dequant(W, s, b, 64, bits, True, out_f16=True)
        assert np.array_equal(rows.view(np.uint16), full[ids].view(np.uint16))
        # f16 arithmetic as the shader writes it (f16(q) * s + b) agrees with it within the reference's 0.005 gate
        sh = (q[ids].astype(np.float16) * s[ids].repeat(64, 1) + b[ids].repeat(64, 1)).astype(np.float64)
        assert np.abs(sh - rows.astype(np.float64)).max() <= 0.005 * np.abs(rows.astype(np.float64)).max()


@pytest.mark.parametrize("bits", [4, 3, 8])
def test_pack_unpack_roundtrip(bits, oracle_c):
    rng = np.random.default_rng(5)
    q = rng.integers(0, 1 << bits, size=(7, 448), dtype=np.uint8)
    W = zo.pack_codes(q, bits)
    assert W.shape == (7, 448 * bits // 32) and W.dtype == np.uint32
    assert np.array_equal(zo.unpack_codes(W, bits), q)
    assert np.array_equal(oracle_c.unpack_codes(W, bits), q)
    if bits == 3:
        assert np.array_equal(zo.unpack_codes_q3_window(W), q)      # the shader's 24-bit window walk
        # bit-serial packing as the reference test writes it (tests/kernels/run.mjs:87-101)
        Wser = np.zeros_like(W)
        for r in range(q.shape[0]):
            for i in range(q.shape[1]):
                bit = 3 * i
                Wser[r, bit >> 5] |= np.uint32((int(q[r, i]) << (bit & 31)) & 0xFFFFFFFF)
                if (bit & 31) > 29:
                    Wser[r, (bit >> 5) + 1] |= np.uint32(int(q[r, i]) >> (32 - (bit & 31)))
        assert np.array_equal(Wser, W)


def test_synth_packing_agrees_with_oracle():
    import zero_tvm_b200 as z
    rng = np.random.default_rng(3)
    for bits in (4, 3):
        q = rng.integers(0, 1 << bits, size=(2, 5, 256), dtype=np.uint8)
        assert np.array_equal(z.synth.pack_codes(q, bits), zo.pack_codes(q, bits))


@pytest.mark.parametrize("K", [512, 768, 1024, 1408])
@pytest.mark.parametrize("flavour", ["symmetric", "affine", "affine_q3"])
def test_reference_test_cases(K, flavour, oracle_c):
    """The inputs and the f64 loop of tests/kernels/run.mjs:77-135, graded with its own metric
    (max |got-ref|/(|ref|+1e-3) < 0.02, run.mjs:153-154); our f32 word-order GEMV sits far inside it."""
    case = zo.reference_test_case(K, affine=flavour != "symmetric", q3=flavour == "affine_q3")
    ref = zo.reference_test_expected(case)
    for impl in (
        lambda: zo.gemv_word_order_f32(case["x"], case["W"], case["scales"], case["biases"], case["group"],
                                       case["bits"], case["affine"])[0],
        lambda: oracle_c.gemv_ref(case["x"], case["W"], case["scales"], case["biases"], case["group"],
                                  case["bits"], case["affine"], out_f32=True)[0],
    ):
        got = impl()
        err = np.max(np.abs(got - ref) / (np.abs(ref) + 1e-3))
        assert err < 1e-4, err
    # and the f64 dot over W32 is the same number as the reference loop (same algebra)
    q = zo.unpack_codes(case["W"], case["bits"])
    w32 = zo.dequant_w32(q, case["scales"], case["biases"], case["group"], case["affine"])
    y64 = zo.matmul_f64(case["x"], w32)[0]
    assert np.max(np.abs(y64 - ref) / (np.abs(ref) + 1e-3)) < 1e-5


def test_c_and_numpy_oracles_agree(oracle_c):
    import zero_tvm_b200 as z
    for bits, group, affine in ((4, 64, True), (3, 64, True), (4, 32, False), (8, 64, True)):
        p = z.synth.projection(48, 768, M=3, bits=bits, group=group, affine=affine, seed=9)
        w32 = zo.dequant_w32(p["q"], p["scales"], p["biases"], group, affine)
        assert np.array_equal(oracle_c.dequant(p["W"], p["scales"], p["biases"], group, bits, affine), w32)
        y64 = zo.matmul_f64(p["x"], w32)
        assert np.allclose(oracle_c.matmul_f64(p["x"], p["W"], p["scales"], p["biases"], group, bits, affine), y64,
                           rtol=1e-13, atol=1e-13)
        y64h = zo.matmul_f64(p["x"], w32.astype(np.float16))
        assert np.allclose(oracle_c.matmul_f64(p["x"], p["W"], p["scales"], p["biases"], group, bits, affine,
                                               w16=True), y64h, rtol=1e-13, atol=1e-13)
        yw = zo.gemv_word_order_f32(p["x"], p["W"], p["scales"], p["biases"], group, bits, affine)
        ywc = oracle_c.gemv_ref(p["x"], p["W"], p["scales"], p["biases"], group, bits, affine, out_f32=True)
        assert np.array_equal(yw, ywc)
        assert zo.rel_err(ywc, y64, 1e-3) < 1e-4


def test_router_topk(oracle_c):
    """Indices exact against a brute-force sort, scores within 2e-6 (tests/kernels/run.mjs:284-345)."""
    rng = np.random.default_rng(7)
    for E, K, norm, shared in ((256, 8, True, True), (128, 8, True, False), (64, 4, False, True), (8, 8, True, False)):
        logits = (rng.random((5, E + int(shared)), dtype=np.float32) * 8 - 4).astype(np.float32)
        logits[0, 3] = logits[0, 1]  # a tie: the lower index must win
        ids, sc = zo.router_topk(logits, E, K, norm, shared)
        idc, scc = oracle_c.router_topk(logits, E, K, norm, shared)
        for t in range(logits.shape[0]):
            ex = np.exp(logits[t, :E].astype(np.float64) - logits[t, :E].max())
            order = sorted(range(E), key=lambda i: (-ex[i], i))[:K]
            ref_sc = ex[order] / (ex[order].sum() if norm else ex.sum())
            assert list(ids[t, :K]) == order and list(idc[t, :K]) == order
            assert np.abs(sc[t, :K] - ref_sc).max() < 2e-6 and np.abs(scc[t, :K] - ref_sc).max() < 2e-6
            if shared:
                assert ids[t, K] == E and idc[t, K] == E
                sg = 1 / (1 + np.exp(-float(logits[t, E])))
                assert abs(sc[t, K] - sg) < 2e-6 and abs(scc[t, K] - sg) < 2e-6


def test_silu_and_combine(oracle_c):
    rng = np.random.default_rng(2)
    gu = rng.standard_normal((6, 2 * 96), dtype=np.float32).astype(np.float16)
    h = zo.silu_mul(gu, 96)
    hc = oracle_c.silu_mul(gu, 96)
    g, u = gu[:, :96].astype(np.float64), gu[:, 96:].astype(np.float64)
    ref = u * g / (1 + np.exp(-g))
    assert np.abs(h.astype(np.float64) - ref).max() <= np.abs(ref).max() * 1e-3
    assert np.abs(h.astype(np.float32) - hc.astype(np.float32)).max() <= 2e-3 * np.abs(ref).max()
    y = rng.standard_normal((4, 9, 64), dtype=np.float32).astype(np.float16)
    sc = rng.random((4, 9), dtype=np.float32)
    out = zo.moe_combine(y, sc)
    outc = oracle_c.moe_combine(y, sc)
    assert np.array_equal(out.view(np.uint16), outc.view(np.uint16))
    ref = (sc[:, :, None].astype(np.float64) * y.astype(np.float64)).sum(1)
    assert np.abs(out.astype(np.float64) - ref).max() < 4e-3


def test_moe_block_small(oracle_c):
    """The whole block through numpy vs the C twin's pieces (f16 intermediates where the engine stores f16)."""
    import zero_tvm_b200 as z
    mb = z.synth.moe_block(3, E=16, hidden=256, ffn=128, seed=4)
    r = zo.moe_block(mb["x"], mb["logits"], mb["gate"], mb["up"], mb["down"], 16, 4, 128)
    ids, sc = oracle_c.router_topk(mb["logits"], 16, 4, True, True)
    assert np.array_equal(ids, r["ids"])
    g = oracle_c.moe_matmul_f64(mb["x"], *mb["gate"], ids, 128, 256, 64, 4, in_per_slot=False)
    assert np.allclose(g, zo.moe_matmul_f64(mb["x"], *mb["gate"], ids, 64, 4, in_per_slot=False), rtol=1e-12)
    # reference-order f32 GEMV agrees with the f64 anchor within the path's tolerance
    out = np.zeros((3, 5, 256), dtype=np.float16)
    oracle_c.moe_gemv_ref(mb["x"], *mb["gate"], ids, 128, 256, 64, 4, 0, 256, 256, 5 * 256, out.reshape(-1))
    assert zo.rel_err(out[..., :128], g, 1e-3) < 2e-3
    assert r["y"].shape == (3, 256) and np.isfinite(r["y"].astype(np.float32)).all()


def test_fused_ffn_restatements_agree():
    """fused_ffn.wgsl:63-131 restated twice (f64 anchor, the shader's f32 order): they agree to the output tolerance, and
    the anchor is the plain matmul anchor followed by the activation."""
    import zero_tvm_b200 as z
    for affine, group in ((True, 64), (False, 32)):
        p = z.synth.projection(96, 512, M=3, seed=8, group=group, affine=affine)
        a = zo.fused_ffn_f64(p["x"], p["W"], p["scales"], p["biases"], 48, group, 4, affine)
        b = zo.fused_ffn_f32(p["x"], p["W"], p["scales"], p["biases"], 48, group, 4, affine)
        assert a.shape == b.shape == (3, 48)
        assert zo.rel_err_scaled(b.astype(np.float64), a, 1e-3) <= 2e-3
        y = zo.matmul_f64(p["x"], zo.dequant_w32(zo.unpack_codes(p["W"], 4), p["scales"], p["biases"], group, affine))
        assert np.allclose(a, y[:, 48:] * y[:, :48] / (1 + np.exp(-y[:, :48])), rtol=1e-12)


def _golden(name):
    import os
    return np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", name))


@pytest.mark.parametrize("name", ["router_ref_e64_k6_raw.npz", "router_ref_e256_k8_norm.npz", "router_ref_e16_k4_norm.npz"])
def test_router_against_the_reference_numpy_router(name):
    """Vectors made by the reference's own numpy routing statements (scripts/make-dsv2-layer-ref.py:327-345; extracted
    with ast by tests/golden/make_golden.py): same experts in the same slot order -- ties to the lower index included --
    and the same weights, with and without renormalisation, from both restatements."""
    from oracle import ztvm_oracle_c as zc
    g = _golden(name)
    logits, ids, w, norm = g["logits"], g["ids"], g["weights"], bool(g["norm"])
    T, E = logits.shape
    K = ids.shape[1]
    for fn in (zo.router_topk, zc.router_topk):
        got_ids, got_w = fn(logits, E, K, norm, False)
        assert np.array_equal(np.asarray(got_ids, dtype=np.uint32), ids), fn.__module__
        assert np.allclose(got_w, w, rtol=2e-6, atol=1e-9), fn.__module__


def test_silu_mul_against_the_reference_numpy_function():
    """silu_mul of scripts/make-dsv2-layer-ref.py:283-284 run on f32 copies of f16 inputs: the restatements round its
    value to f16; another order of the same three operations may land one f16 step away on a few outputs."""
    from oracle import ztvm_oracle_c as zc
    g = _golden("silu_mul_ref.npz")
    gate, up, h = g["gate"], g["up"], g["h"]
    want = h.astype(np.float16)
    gu = np.concatenate([gate, up], axis=1)
    for fn in (zo.silu_mul, zc.silu_mul):
        got = np.asarray(fn(gu, gate.shape[1]), dtype=np.float16)
        steps = np.abs(got.view(np.int16).astype(np.int32) - want.view(np.int16).astype(np.int32))
        assert steps.max() <= 1 and (steps == 0).mean() >= 0.99, (fn.__module__, steps.max(), (steps == 0).mean())
