"""CPU oracle for the int4/int3 group-quantised dequant-matmul family (numpy).

TEST INFRASTRUCTURE ONLY. This module restates, on the CPU, the arithmetic of
the Zero-TVM kernels that the CUDA library replaces. Nothing in the shipped
package imports it; only the test-suite, the smoke check and the CPU-baseline
leg of the benchmark do, and always as the checker, never as the thing being
measured or shipped.

Parity status. Pinned against output of the reference's own numpy code, run on
seeded inputs and committed as fixtures in tests/golden/ (made by
tests/golden/make_golden.py, which extracts the pieces with `ast`): the 4-bit
affine dequantiser (`dequant_from`, scripts/make-dsv2-layer-ref.py:102-116), the
3-bit and 4-bit unpack and the factored GEMV reference
(scripts/make-kernel-ref.py:55-66), the routing of one token (softmax, top-k
order with ties to the lower index, raw or renormalised weights:
scripts/make-dsv2-layer-ref.py:327-345) and `silu_mul` (:283-284). Everything
else (the symmetric flavour, the GEMV word order, the shared-expert slot, combine,
router logits, embedding, fused FFN) follows the reference's formulas, but the
reference ships no stored vectors for them and its JavaScript/WGSL cannot run
here: for those functions parity is pinned by formula only ("parity unpinned"
against executed reference output).

Every function cites the reference file:line it follows (paths are relative to
the reference project's root).
"""
from __future__ import annotations

import numpy as np

F16 = np.float16
F32 = np.float32
F64 = np.float64


# --------------------------------------------------------------------------
# number formats
# --------------------------------------------------------------------------
def to_f16(a) -> np.ndarray:
    """f64/f32 -> f16, round-to-nearest-even, subnormals kept.

    tests/kernels/half.mjs:13-36 does f64 -> f32 -> f16; numpy's astype chain
    performs the same two IEEE roundings.
    """
    return np.asarray(a).astype(F32).astype(F16)


# --------------------------------------------------------------------------
# packing / unpacking of codes
# --------------------------------------------------------------------------
def words_per_row(K: int, bits: int) -> int:
    """u32 words per weight row: K*bits/32 (engine-core.ts:1047-1049)."""
    assert (K * bits) % 32 == 0
    return K * bits // 32


def pack_codes(q: np.ndarray, bits: int) -> np.ndarray:
    """codes u8 [..., K] -> packed u32 [..., K*bits/32].

    4-bit: code i of a word sits at bits [4i, 4i+4) (int4_matmul.gen.ts:157-167).
    3-bit: code i of a ROW sits at bit 3i of the row's LSB-first bitstream,
    straddling word edges freely (int4_matmul.gen.ts:115-131,
    tests/kernels/run.mjs:87-101).
    """
    q = np.asarray(q, dtype=np.uint8)
    K = q.shape[-1]
    lead = q.shape[:-1]
    if bits == 4:
        q32 = q.reshape(*lead, K // 8, 8).astype(np.uint32)
        shifts = (np.arange(8, dtype=np.uint32) * 4)
        return (q32 << shifts).sum(axis=-1, dtype=np.uint32)
    if bits == 8:   # four bytes per word, little end first (int8_affine_matvec.wgsl, moe_router_logits.wgsl: word >> 8n)
        return np.ascontiguousarray(q).view("<u4").reshape(*lead, K // 4)
    if bits == 3:
        b = np.stack([(q >> j) & 1 for j in range(3)], axis=-1).reshape(*lead, K * 3)
        by = np.packbits(b.astype(np.uint8), axis=-1, bitorder="little")
        return np.ascontiguousarray(by).view("<u4").reshape(*lead, K * 3 // 32)
    raise ValueError("bits must be 3, 4 or 8")


def unpack_codes(W: np.ndarray, bits: int) -> np.ndarray:
    """packed u32 [..., KP] -> codes u8 [..., K] (inverse of pack_codes).

    4-bit: q[k] = (W[k>>3] >> 4(k&7)) & 15 (int4_matmul.gen.ts:157-167).
    3-bit: bits 3k..3k+2 of the little-endian row bitstream
    (scripts/make-kernel-ref.py:59-63 uses the same unpackbits formulation).
    """
    W = np.ascontiguousarray(np.asarray(W, dtype=np.uint32))
    lead, KP = W.shape[:-1], W.shape[-1]
    if bits == 4:
        shifts = (np.arange(8, dtype=np.uint32) * 4)
        return ((W[..., None] >> shifts) & 15).astype(np.uint8).reshape(*lead, KP * 8)
    if bits == 8:
        return W.view(np.uint8).reshape(*lead, KP * 4).copy()
    if bits == 3:
        K = KP * 32 // 3
        bitsarr = np.unpackbits(W.view(np.uint8).reshape(*lead, KP * 4), axis=-1, bitorder="little")
        return (bitsarr[..., 0::3][..., :K] + 2 * bitsarr[..., 1::3][..., :K]
                + 4 * bitsarr[..., 2::3][..., :K]).astype(np.uint8)
    raise ValueError("bits must be 3, 4 or 8")


def unpack_codes_q3_window(W: np.ndarray) -> np.ndarray:
    """3-bit unpack the way the shader walks it: 24-bit windows of 8 codes.

    int4_matmul.gen.ts:409-448: block j starts at bit 24j, sh = bit & 31,
    win = W[bit>>5] >> sh, OR'ed with W[+1] << (32-sh) when sh > 8.
    Pure-Python loops; for small cases (cross-check of unpack_codes).
    """
    W = np.asarray(W, dtype=np.uint32)
    N, KP = W.shape
    K = KP * 32 // 3
    out = np.zeros((N, K), dtype=np.uint8)
    for n in range(N):
        for blk in range(K // 8):
            bit = blk * 24
            sh = bit & 31
            win = int(W[n, bit >> 5]) >> sh
            if sh > 8:
                win |= (int(W[n, (bit >> 5) + 1]) << (32 - sh)) & 0xFFFFFFFF
            for j in range(8):
                out[n, blk * 8 + j] = (win >> (3 * j)) & 7
    return out


# --------------------------------------------------------------------------
# dequantisation (the two canonical definitions)
# --------------------------------------------------------------------------
def dequant_w32(q, scales, biases, group: int, affine: bool = True) -> np.ndarray:
    """f32 dequantised weights, the GEMV / staged-f32 semantics.

    affine  : W32 = fl32(fl32(s)*q + fl32(b))      (int4_matmul.gen.ts:1001)
    symmetric: W32 = fl32(fl32(s)*(q-7))            (int4_matmul.gen.ts:1002, :17-22)
    s has an 11-bit significand and q <= 15, so s*q is exact in f32 and the
    add is the only rounding: FMA and mul+add agree bit for bit.
    """
    q = np.asarray(q)
    s = np.asarray(scales, dtype=F16).astype(F32).repeat(group, axis=-1)
    if affine:
        b = np.asarray(biases, dtype=F16).astype(F32).repeat(group, axis=-1)
        return (q.astype(F32) * s + b).astype(F32)
    return ((q.astype(F32) - F32(7.0)) * s).astype(F32)


def dequant_w16(q, scales, biases, group: int, affine: bool = True) -> np.ndarray:
    """f16 dequantised weights, the tensor-core semantics: W16 = f16_rne(W32).

    Same value as the reference's numpy dequant_from output
    (scripts/make-dsv2-layer-ref.py:108-116), which that file documents as
    bit-identical to mx.dequantize.
    """
    return dequant_w32(q, scales, biases, group, affine).astype(F16)


# --------------------------------------------------------------------------
# matmul references
# --------------------------------------------------------------------------
def matmul_f64(x, Wdq) -> np.ndarray:
    """y_ref[m,n] = sum_k f64(x[m,k]) * f64(Wdq[n,k]) — the tolerance anchor."""
    x = np.atleast_2d(np.asarray(x)).astype(F64)
    return x @ np.asarray(Wdq).astype(F64).T


def gemv_word_order_f32(x, W, scales, biases, group: int, bits: int, affine: bool = True,
                        lanes: int = 32) -> np.ndarray:
    """GEMV in the shader's own order of operations, all in f32.

    int4_matmul.gen.ts:388-408,449-464 (+ :409-448 for 3-bit): lane t walks
    8-code blocks t, t+lanes, ...; per block
        acc += s * (sum_i x_i * q_i) + b * (sum_i x_i)      (affine)
        acc += s * (sum_i x_i * (q_i - 7))                  (symmetric)
    with the 8 products paired (x0q0+x1q1)+(x2q2+x3q3)+... (gen.ts:164-166),
    then the lane sums are added (subgroupAdd; a pairwise tree here).
    Returns f32 [M, N] before the output cast.
    """
    x = np.atleast_2d(np.asarray(x, dtype=F16)).astype(F32)
    q = unpack_codes(W, bits).astype(F32)
    N, K = q.shape
    M = x.shape[0]
    nblk = K // 8
    spb = group // 8                      # blocks per scale group
    s = np.asarray(scales, dtype=F16).astype(F32)
    b = np.asarray(biases, dtype=F16).astype(F32) if affine else None
    qb = q.reshape(N, nblk, 8)
    if not affine:
        qb = qb - F32(7.0)
    out = np.zeros((M, N), dtype=F32)
    for m in range(M):
        xb = x[m].reshape(nblk, 8)
        p = (xb[None] * qb).astype(F32)                       # [N, nblk, 8]
        pair = (p[..., 0::2] + p[..., 1::2]).astype(F32)      # 4 pairs
        dot = ((pair[..., 0] + pair[..., 1]).astype(F32) + pair[..., 2]).astype(F32)
        dot = (dot + pair[..., 3]).astype(F32)                # [N, nblk]
        sg = s.repeat(spb, axis=1)[:, :nblk]
        term = (sg * dot).astype(F32)
        if affine:
            xs = xb[:, 0]
            for i in range(1, 8):
                xs = (xs + xb[:, i]).astype(F32)
            term = (term + (b.repeat(spb, axis=1)[:, :nblk] * xs[None]).astype(F32)).astype(F32)
        # lane-strided accumulation
        acc = np.zeros((N, lanes), dtype=F32)
        for blk0 in range(0, nblk, lanes):
            chunk = term[:, blk0:blk0 + lanes]
            acc[:, :chunk.shape[1]] = (acc[:, :chunk.shape[1]] + chunk).astype(F32)
        w = lanes
        while w > 1:
            w //= 2
            acc = (acc[:, :w] + acc[:, w:2 * w]).astype(F32)
        out[m] = acc[:, 0]
    return out


def rel_err(y, y_ref, floor: float = 0.0) -> float:
    """max |y - y_ref| / max(|y_ref|, floor).

    The reference always grades with a floor: +1e-3 (tests/kernels/run.mjs:153),
    max(1e-2, .) (scripts/gemm-bench.mjs:516). floor=0 is the pure relative error.
    """
    y = np.asarray(y).astype(F64)
    y_ref = np.asarray(y_ref).astype(F64)
    den = np.maximum(np.abs(y_ref), floor) if floor > 0 else np.abs(y_ref)
    with np.errstate(divide="ignore", invalid="ignore"):
        r = np.abs(y - y_ref) / den
    r = np.where(np.isnan(r), np.where(y == y_ref, 0.0, np.inf), r)
    return float(r.max()) if r.size else 0.0


def rel_err_scaled(y, y_ref, frac: float = 1e-3) -> float:
    """rel_err with the floor tied to the output scale: floor = frac * rms(y_ref).

    An f32 accumulation carries an absolute error proportional to the size of the
    partial sums, so outputs that cancel to almost nothing cannot be held to a pure
    relative bound by any f32 kernel (the reference's own f32 word order misses 2e-3
    pure-relative on the 8192x2048 decode case). The reference grades with an absolute
    floor of 1e-3 on O(1) outputs; this is the same floor made scale-free, so it also
    fits the MoE down projection whose outputs are O(30).
    """
    y_ref = np.asarray(y_ref).astype(F64)
    rms = float(np.sqrt(np.mean(y_ref * y_ref))) if y_ref.size else 0.0
    return rel_err(y, y_ref, max(frac * rms, 1e-30))


# --------------------------------------------------------------------------
# router logits and embedding rows
# --------------------------------------------------------------------------
def router_logits_f64(x, w, scales=None, biases=None, bits: int = 8) -> np.ndarray:
    """logits[t, e] as an f64 dot over the dequantised router (f32-exact weights; bits 16: the f16 weights themselves).

    moe_router_logits.wgsl:44-140 / run.mjs:186-283: logit = sum_g (s_g * sum x q + b_g * sum x), q unsigned, no offset;
    moe_router_logits_f16.wgsl: plain f16 weights. x f16 [T, D] -> f64 [T, rows].
    """
    x = np.atleast_2d(np.asarray(x, dtype=F16)).astype(F64)
    if bits == 16:
        return x @ np.asarray(w, dtype=F16).astype(F64).T
    q = unpack_codes(w, bits)
    return x @ dequant_w32(q, scales, biases, 64, True).astype(F64).T


def router_logits_word_order_f32(x, w, scales, biases, bits: int) -> np.ndarray:
    """The shader's own order for one token (moe_router_logits.wgsl:68-99): thread tid of 64 takes words tid, tid+64, ...;
    per word acc += s*dot + b*xs in f32; then the pairwise tree over the 64 threads. Pure-Python; small cases only."""
    x = np.asarray(x, dtype=F16).astype(F32).reshape(-1)
    W = np.asarray(w, dtype=np.uint32)
    rows, WPR = W.shape
    per = 32 // bits
    out = np.zeros(rows, dtype=F32)
    for e in range(rows):
        acc = np.zeros(64, dtype=F32)
        for wi in range(WPR):
            g = wi * per // 64
            s_, b_ = F32(np.asarray(scales, dtype=F16)[e, g]), F32(np.asarray(biases, dtype=F16)[e, g])
            dot, xs = F32(0), F32(0)
            for n in range(per):
                v = x[wi * per + n]
                dot = F32(dot + v * F32((int(W[e, wi]) >> (bits * n)) & ((1 << bits) - 1)))
                xs = F32(xs + v)
            t = wi % 64
            acc[t] = F32(acc[t] + F32(F32(s_ * dot) + F32(b_ * xs)))
        st = 32
        while st > 0:
            acc[:st] = (acc[:st] + acc[st:2 * st]).astype(F32)
            st //= 2
        out[e] = acc[0]
    return out


def embedding_rows(input_ids, W, scales, biases, bits: int = 4) -> np.ndarray:
    """out[t] = dequantised row input_ids[t] as f16 (embedding_affine.wgsl:38-57): the canonical W16 of that row, which is
    what the reference's real-weights test compares the shader with (tests/kernels/real-weights.mjs:721-750, 0.005)."""
    ids = np.asarray(input_ids).astype(np.int64)
    q = unpack_codes(np.asarray(W, dtype=np.uint32)[ids], bits)
    return dequant_w16(q, np.asarray(scales)[ids], np.asarray(biases)[ids], 64, True)


# --------------------------------------------------------------------------
# MoE glue
# --------------------------------------------------------------------------
def router_topk(logits, E: int, K: int, norm_topk: bool, has_shared: bool):
    """softmax over the E routed experts, K arg-max rounds, renormalise.

    moe_router_topk.wgsl:83-135 (f32 arithmetic): peak = max, p = exp(l-peak),
    denom = sum p; K rounds of arg-max with ties to the LOWER index (:113-114);
    score = p * (1/sum_top if normTopk else 1/denom) (:125); slots in
    descending score order; slot K = expert E with sigmoid(logit[E]) when the
    checkpoint has a shared expert (:131-134).
    logits f32 [T, E+has_shared] -> ids u32 [T, K+has_shared], scores f32 same.
    """
    logits = np.atleast_2d(np.asarray(logits, dtype=F32))
    T = logits.shape[0]
    S = K + (1 if has_shared else 0)
    ids = np.zeros((T, S), dtype=np.uint32)
    scores = np.zeros((T, S), dtype=F32)
    for t in range(T):
        l = logits[t, :E]
        peak = l.max()
        p = np.exp((l - peak).astype(F32)).astype(F32)
        denom = F32(p.sum(dtype=F32))
        # stable sort on -p keeps the lower index first among equals
        order = np.argsort(-p, kind="stable")[:K]
        top = p[order]
        total = F32(0.0)
        for v in top:
            total = F32(total + v)
        scale = F32(1.0) / (total if norm_topk else denom)
        ids[t, :K] = order
        scores[t, :K] = (top * scale).astype(F32)
        if has_shared:
            ids[t, K] = E
            g = logits[t, E]
            scores[t, K] = F32(1.0) / (F32(1.0) + np.exp(-g).astype(F32))
    return ids, scores


def silu_mul(gate_up, ffn: int) -> np.ndarray:
    """h = f16(up * gate * 1/(1+exp(-gate))) in f32 from f16 inputs.

    silu_mul.wgsl:40-43. gate_up f16 [R, 2*ffn] (gate | up) -> f16 [R, ffn].
    """
    gu = np.asarray(gate_up, dtype=F16).astype(F32)
    g, u = gu[..., :ffn], gu[..., ffn:2 * ffn]
    sg = (g * (F32(1.0) / (F32(1.0) + np.exp(-g).astype(F32))).astype(F32)).astype(F32)
    return (u * sg).astype(F32).astype(F16)


def moe_combine(y_slots, scores) -> np.ndarray:
    """out[t] = f16(sum_s score[t,s] * f32(y[t,s])), slots added in order.

    moe_combine.wgsl:39-43. y_slots f16 [T, S, d], scores f32 [T, S].
    """
    y = np.asarray(y_slots, dtype=F16).astype(F32)
    sc = np.asarray(scores, dtype=F32)
    T, S, d = y.shape
    acc = np.zeros((T, d), dtype=F32)
    for s in range(S):
        acc = (acc + (sc[:, s:s + 1] * y[:, s]).astype(F32)).astype(F32)
    return acc.astype(F16)


def moe_matmul_f64(x, Wstack, sstack, bstack, ids, group: int, bits: int,
                   in_per_slot: bool, w16: bool = False) -> np.ndarray:
    """Per-(token, slot) expert matmul, f64 dot over the dequantised weights.

    int4_matmul.gen.ts:229-254: expert = ids[token, slot]; the expert's rows
    come from the [E(+1), N, ...] stacks; the input is shared across slots
    (gate/up: IN_SLOT_STRIDE = 0) or per slot (down).
    x f16 [T, K] or [T, S, K] -> f64 [T, S, N].
    """
    ids = np.asarray(ids)
    T, S = ids.shape
    N = Wstack.shape[1]
    out = np.zeros((T, S, N), dtype=F64)
    x = np.asarray(x, dtype=F16).astype(F64)
    cache = {}
    for e in np.unique(ids):
        qe = unpack_codes(Wstack[e], bits)
        we = dequant_w32(qe, sstack[e], bstack[e], group, True)
        if w16:
            we = we.astype(F16)
        cache[int(e)] = we.astype(F64)
    for e, we in cache.items():
        t_idx, s_idx = np.nonzero(ids == e)
        xin = x[t_idx, s_idx] if in_per_slot else x[t_idx]
        out[t_idx, s_idx] = xin @ we.T
    return out


def moe_block(x, logits, gate, up, down, E: int, K: int, ffn: int, group: int = 64, bits: int = 4,
              norm_topk: bool = True, has_shared: bool = True):
    """Whole expert block as the engine dispatches it, intermediates rounded to f16
    exactly where the reference stores f16.

    engine-core.ts:2342-2349: gate and up matmuls write interleaved halves of a
    [T, S, 2*ffn] f16 buffer (engine-core.ts:2036-2043), silu_mul -> [T, S, ffn]
    f16, down matmul -> [T, S, d] f16, moe_combine -> [T, d] f16. Composition and
    stacking follow scripts/make-kernel-ref.py:136-143,154-178.
    gate/up/down are (W, scales, biases) stacks with the shared expert at index E.
    Returns dict with ids, scores, gate_up, h, y_slots, y.
    """
    ids, scores = router_topk(logits, E, K, norm_topk, has_shared)
    g = moe_matmul_f64(x, *gate, ids, group, bits, in_per_slot=False)
    u = moe_matmul_f64(x, *up, ids, group, bits, in_per_slot=False)
    gate_up = np.concatenate([to_f16(g), to_f16(u)], axis=-1)        # [T, S, 2ffn]
    h = silu_mul(gate_up, ffn)                                        # [T, S, ffn]
    y_slots = to_f16(moe_matmul_f64(h, *down, ids, group, bits, in_per_slot=True))
    y = moe_combine(y_slots, scores)
    return dict(ids=ids, scores=scores, gate_up=gate_up, h=h, y_slots=y_slots, y=y)


# --------------------------------------------------------------------------
# the reference's own test-input generator (tests/kernels/run.mjs)
# --------------------------------------------------------------------------
def mulberry32(seed: int):
    """The seeded PRNG of tests/kernels/run.mjs:44-52 (uniform in [0,1))."""
    state = [seed & 0xFFFFFFFF]

    def imul(a, b):
        return (a * b) & 0xFFFFFFFF

    def nxt():
        state[0] = (state[0] + 0x6D2B79F5) & 0xFFFFFFFF
        s = state[0]
        t = imul(s ^ (s >> 15), 1 | s)
        t = ((t + imul(t ^ (t >> 7), 61 | t)) & 0xFFFFFFFF) ^ t
        return ((t ^ (t >> 14)) & 0xFFFFFFFF) / 4294967296.0
    return nxt


def reference_test_case(K: int = 512, affine: bool = False, q3: bool = False, M: int = 8):
    """Inputs of makeInt4MatmulTest (tests/kernels/run.mjs:77-105), same seed and
    draw order, so the parity tests run on the reference's own test cases.
    Returns dict(x f16[K], scales f16[M,SPR], biases f16[M,SPR]|None, W u32[M,KP], bits, group).
    """
    r = mulberry32(1)
    bits = 3 if q3 else 4
    KP = K * bits // 32
    group = 64 if affine else 32
    SPR = K // group
    x = to_f16(np.array([r() * 2 - 1 for _ in range(K)]))
    scales = to_f16(np.array([r() * 0.05 + 0.01 for _ in range(M * SPR)])).reshape(M, SPR)
    biases = (to_f16(np.array([r() * 0.1 - 0.05 for _ in range(M * SPR)])).reshape(M, SPR)
              if affine else None)
    if q3:
        q = np.array([int(np.floor(r() * 8)) for _ in range(M * K)], dtype=np.uint8).reshape(M, K)
        W = pack_codes(q, 3)
    else:
        W = np.array([int(r() * 0xFFFFFFFF) & 0xFFFFFFFF for _ in range(M * KP)],
                     dtype=np.uint32).reshape(M, KP)
    return dict(x=x, scales=scales, biases=biases, W=W, bits=bits, group=group, affine=affine)


def reference_test_expected(case) -> np.ndarray:
    """The f64 reference loop of tests/kernels/run.mjs:109-135 (per word,
    scale*dot + bias*xs accumulated in double), before the output cast."""
    x = case["x"].astype(F64)
    q = unpack_codes(case["W"], case["bits"]).astype(F64)
    s = case["scales"].astype(F64).repeat(case["group"], axis=1)
    if case["affine"]:
        b = case["biases"].astype(F64).repeat(case["group"], axis=1)
        return (s * q * x[None] + b * x[None]).sum(axis=1)
    return (s * (q - 7.0) * x[None]).sum(axis=1)


def reference_router_case(bits: int, D: int = 2048, rows: int = 9):
    """Inputs of makeRouterLogitsTest (tests/kernels/run.mjs:199-216), same seed (11 + bits) and draw order: x in
    [-1, 1), codes uniform, scales in [0.005, 0.025), biases in [-0.1, 0.1); bits 16 draws f16 weights in [-0.05, 0.05)
    after the (unused) quantised tensors, as the test does. Returns dict(x f16[D], w, scales, biases)."""
    r = mulberry32(11 + bits)
    GPR = D // 64
    maxq = (1 << bits) - 1
    x = to_f16(np.array([r() * 2 - 1 for _ in range(D)]))
    q = np.array([int(np.floor(r() * (maxq + 1))) for _ in range(rows * D)], dtype=np.int64).reshape(rows, D)
    scales = to_f16(np.array([r() * 0.02 + 0.005 for _ in range(rows * GPR)])).reshape(rows, GPR)
    biases = to_f16(np.array([r() * 0.2 - 0.1 for _ in range(rows * GPR)])).reshape(rows, GPR)
    if bits == 16:
        w = to_f16(np.array([r() * 0.1 - 0.05 for _ in range(rows * D)])).reshape(rows, D)
        return dict(x=x, w=w, bits=16)
    return dict(x=x, w=pack_codes(q.astype(np.uint8), bits), scales=scales, biases=biases, bits=bits, q=q)


def reference_router_expected(case) -> np.ndarray:
    """The f64 reference of tests/kernels/run.mjs:217-233: per group, scale * dot + bias * xs, accumulated in double."""
    x = case["x"].astype(F64)
    if case["bits"] == 16:
        return case["w"].astype(F64) @ x
    q = case["q"].astype(F64)
    rows, D = q.shape
    xg = x.reshape(D // 64, 64)
    dot = (q.reshape(rows, D // 64, 64) * xg[None]).sum(axis=2)
    return (case["scales"].astype(F64) * dot + case["biases"].astype(F64) * xg.sum(axis=1)[None]).sum(axis=1)


def fused_ffn_f64(x, W, scales, biases, ffn: int, group: int = 64, bits: int = 4, affine: bool = True) -> np.ndarray:
    """fp64 anchor of the fused FFN front half (src/compiler/shaders/fused_ffn.wgsl:63-131): gate = x . W[i],
    up = x . W[ffn + i] over the f32 dequantised weights, h = up * gate / (1 + exp(-gate)); nothing is rounded."""
    q = unpack_codes(W, bits)
    Wdq = dequant_w32(q, scales, biases, group, affine)
    y = matmul_f64(x, Wdq)
    g, u = y[:, :ffn], y[:, ffn:2 * ffn]
    return u * g / (1.0 + np.exp(-g))


def fused_ffn_f32(x, W, scales, biases, ffn: int, group: int = 64, bits: int = 4, affine: bool = True) -> np.ndarray:
    """The shader's own arithmetic: f32 dot products in word order, silu and product in f32, one f16 rounding
    (fused_ffn.wgsl:126-131: `silu_gate = gate * (1 / (1 + exp(-gate)))`, `output = f16(up * silu_gate)`)."""
    y = gemv_word_order_f32(x, W, scales, biases, group, bits, affine)
    y = np.atleast_2d(y).astype(F32)
    g, u = y[:, :ffn], y[:, ffn:2 * ffn]
    one = F32(1.0)
    silu = (g * (one / (one + np.exp(-g, dtype=F32)))).astype(F32)
    return (u * silu).astype(F32).astype(F16)
