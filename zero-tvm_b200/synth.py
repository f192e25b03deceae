"""Seeded synthetic tensors in the layouts the matmul kernels consume.

Packed weights `u32[N][K*bits/32]`, per-group `f16` scale and bias `[N][K/group]`,
activations `f16[M][K]`; expert stacks add a leading `[E(+1)]` axis with the shared
expert appended at index E (src/zero-tvm/mlx-weights.ts:362-373). Distributions:
codes uniform, scale = |N(0, sigma_s)|, bias ~ N(0, 0.05), x ~ N(0, 1); every f16
tensor is an f32 draw rounded to nearest-even. One `numpy.random.default_rng(seed)`
stream per tensor set, drawn in the fixed order x, codes, scale, bias, so the CPU
checker and the GPU see identical bytes. The reference's own benches are synthetic in
the same way (scripts/gemm-bench.mjs:447-463).
"""
from __future__ import annotations

import numpy as np


def pack_codes(q: np.ndarray, bits: int) -> np.ndarray:
    """codes u8 [..., K] -> u32 [..., K*bits/32].

    4-bit: code i of a word at bits [4i, 4i+4). 3-bit: code i of a row at bit 3i of the
    row's LSB-first bitstream (src/compiler/shaders/int4_matmul.gen.ts:115-131,157-167).
    """
    q = np.asarray(q, dtype=np.uint8)
    K = q.shape[-1]
    lead = q.shape[:-1]
    if bits == 4:
        out = np.zeros((*lead, K // 8), dtype=np.uint32)
        for i in range(8):
            out |= q[..., i::8].astype(np.uint32) << np.uint32(4 * i)
        return out
    if bits == 8:
        return np.ascontiguousarray(q).view("<u4").reshape(*lead, K // 4)
    if bits == 3:
        planes = np.empty((*lead, K, 3), dtype=np.uint8)
        for j in range(3):
            planes[..., j] = (q >> j) & 1
        by = np.packbits(planes.reshape(*lead, K * 3), axis=-1, bitorder="little")
        return np.ascontiguousarray(by).view("<u4").reshape(*lead, K * 3 // 32)
    raise ValueError("bits must be 3, 4 or 8")


def make_weights(rng: np.random.Generator, N: int, K: int, *, bits: int = 4, group: int = 64,
                 affine: bool = True, sigma_s: float = 0.01, lead: tuple = ()):
    """(codes u8, W u32, scales f16, biases f16|None) with optional leading stack axes."""
    q = rng.integers(0, 1 << bits, size=(*lead, N, K), dtype=np.uint8)
    s = np.abs(rng.standard_normal((*lead, N, K // group), dtype=np.float32) * np.float32(sigma_s))
    s = s.astype(np.float16)
    b = None
    if affine:
        b = (rng.standard_normal((*lead, N, K // group), dtype=np.float32) * np.float32(0.05)).astype(np.float16)
    return q, pack_codes(q, bits), s, b


def make_x(rng: np.random.Generator, M: int, K: int) -> np.ndarray:
    return rng.standard_normal((M, K), dtype=np.float32).astype(np.float16)


def projection(N: int, K: int, M: int = 1, *, seed: int = 0, bits: int = 4, group: int = 64,
               affine: bool = True, sigma_s: float | None = None):
    """One dense projection: dict(x, q, W, scales, biases, N, K, M, bits, group, affine)."""
    rng = np.random.default_rng(seed)
    if sigma_s is None:
        sigma_s = 0.02 if bits == 3 else 0.01
    x = make_x(rng, M, K)
    q, W, s, b = make_weights(rng, N, K, bits=bits, group=group, affine=affine, sigma_s=sigma_s)
    return dict(x=x, q=q, W=W, scales=s, biases=b, N=N, K=K, M=M, bits=bits, group=group, affine=affine)


# The dense 8B-class decode layer set: (name, N, K, f32 output).
DENSE_LAYER_SET = [
    ("q_proj", 4096, 4096, False), ("k_proj", 1024, 4096, False), ("v_proj", 1024, 4096, False),
    ("o_proj", 4096, 4096, False), ("gate_proj", 12288, 4096, False), ("up_proj", 12288, 4096, False),
    ("down_proj", 4096, 12288, False), ("lm_head", 151936, 4096, True),
]


# The same layer as the engine dispatches it for decode: q, k, v rows concatenated into one projection and gate, up into
# another (src/zero-tvm/engine-core.ts:1012-1018, :2290, :2517), so five launches instead of eight.
DENSE_LAYER_SET_FUSED = [
    ("qkv_proj", 6144, 4096, False), ("o_proj", 4096, 4096, False), ("gate_up_proj", 24576, 4096, False),
    ("down_proj", 4096, 12288, False), ("lm_head", 151936, 4096, True),
]


def moe_block(T: int, *, E: int = 256, hidden: int = 2048, ffn: int = 512, bits: int = 4, group: int = 64,
              seed: int = 0, has_shared: bool = True):
    """Expert stacks (shared expert at index E), activations and router logits for T tokens."""
    rng = np.random.default_rng(seed)
    x = make_x(rng, T, hidden)
    logits = rng.standard_normal((T, E + (1 if has_shared else 0)), dtype=np.float32)
    lead = (E + (1 if has_shared else 0),)
    stacks = {}
    for name, (n, k) in (("gate", (ffn, hidden)), ("up", (ffn, hidden)), ("down", (hidden, ffn))):
        _, W, s, b = make_weights(rng, n, k, bits=bits, group=group, affine=True, sigma_s=0.01, lead=lead)
        stacks[name] = (W, s, b)
    return dict(x=x, logits=logits, E=E, hidden=hidden, ffn=ffn, bits=bits, group=group,
                has_shared=has_shared, T=T, **stacks)
