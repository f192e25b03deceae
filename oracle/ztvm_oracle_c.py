"""ctypes binding of the C twin of the CPU oracle (oracle/ztvm_oracle.c).

TEST INFRASTRUCTURE ONLY, like the numpy oracle: same functions, fast enough for the
full benchmark sizes and used as the timed CPU baseline. Build with `make -C oracle`.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libztvm_oracle.so")
_lib = None


def build() -> str:
    """Compile the C oracle in place (gcc only, seconds)."""
    subprocess.check_call(["make", "-C", _HERE, "--no-print-directory"], stdout=subprocess.DEVNULL)
    return _SO


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        _lib = C.CDLL(_SO)
        _lib.zo_num_threads.restype = C.c_int
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _c(a, dt):
    return None if a is None else np.ascontiguousarray(a, dtype=dt)


def _f16bits(a):
    return None if a is None else np.ascontiguousarray(np.asarray(a, dtype=np.float16)).view(np.uint16)


def num_threads() -> int:
    return int(lib().zo_num_threads())


def unpack_codes(W, bits: int) -> np.ndarray:
    W = _c(W, np.uint32)
    N, KP = W.shape
    K = KP * 32 // bits
    q = np.empty((N, K), dtype=np.uint8)
    lib().zo_unpack_codes(_p(W), _p(q), C.c_long(N), C.c_long(K), C.c_int(bits))
    return q


def dequant(W, scales, biases, group: int, bits: int = 4, affine: bool = True, out_f16: bool = False):
    W = _c(W, np.uint32)
    N, KP = W.shape
    K = KP * 32 // bits
    s, b = _f16bits(scales), _f16bits(biases)
    out = np.empty((N, K), dtype=np.float16 if out_f16 else np.float32)
    lib().zo_dequant(_p(W), _p(s), _p(b), _p(out), C.c_long(N), C.c_long(K), C.c_int(bits), C.c_int(group),
                     C.c_int(int(affine)), C.c_int(int(out_f16)))
    return out


def matmul_f64(x, W, scales, biases, group: int, bits: int = 4, affine: bool = True, w16: bool = False):
    x = _f16bits(np.atleast_2d(x))
    W = _c(W, np.uint32)
    M, K = x.shape
    N = W.shape[0]
    s, b = _f16bits(scales), _f16bits(biases)
    y = np.empty((M, N), dtype=np.float64)
    lib().zo_matmul_f64(_p(x), _p(W), _p(s), _p(b), _p(y), C.c_long(M), C.c_long(N), C.c_long(K), C.c_int(bits),
                        C.c_int(group), C.c_int(int(affine)), C.c_int(int(w16)))
    return y


def gemv_ref(x, W, scales, biases, group: int, bits: int = 4, affine: bool = True, out_f32: bool = False,
             lanes: int = 32):
    x = _f16bits(np.atleast_2d(x))
    W = _c(W, np.uint32)
    M, K = x.shape
    N = W.shape[0]
    s, b = _f16bits(scales), _f16bits(biases)
    y = np.empty((M, N), dtype=np.float32 if out_f32 else np.float16)
    lib().zo_gemv_ref(_p(x), _p(W), _p(s), _p(b), _p(y), C.c_long(M), C.c_long(N), C.c_long(K), C.c_int(bits),
                      C.c_int(group), C.c_int(int(affine)), C.c_int(int(out_f32)), C.c_int(lanes))
    return y


def moe_gemv_ref(x, Wstack, sstack, bstack, ids, N: int, K: int, group: int, bits: int, in_slot_stride: int,
                 out_slot_stride: int, in_tok_stride: int, out_tok_stride: int, out: np.ndarray):
    """ids-indirect expert GEMV writing f16 into `out` (flat) with the given element strides."""
    ids = _c(ids, np.uint32)
    T, S = ids.shape
    xb = _f16bits(x)
    W = _c(Wstack, np.uint32)
    s, b = _f16bits(sstack), _f16bits(bstack)
    ob = out.view(np.uint16)
    lib().zo_moe_gemv_ref(_p(xb), _p(W), _p(s), _p(b), _p(ob), _p(ids), C.c_long(T), C.c_long(S), C.c_long(N),
                          C.c_long(K), C.c_int(bits), C.c_int(group), C.c_long(in_slot_stride),
                          C.c_long(out_slot_stride), C.c_long(in_tok_stride), C.c_long(out_tok_stride),
                          C.c_long(S))
    return out


def moe_matmul_f64(x, Wstack, sstack, bstack, ids, N: int, K: int, group: int, bits: int, in_per_slot: bool,
                   w16: bool = False):
    ids = _c(ids, np.uint32)
    T, S = ids.shape
    xb = _f16bits(x)
    W = _c(Wstack, np.uint32)
    s, b = _f16bits(sstack), _f16bits(bstack)
    y = np.empty((T, S, N), dtype=np.float64)
    in_slot = K if in_per_slot else 0
    in_tok = S * K if in_per_slot else K
    lib().zo_moe_matmul_f64(_p(xb), _p(W), _p(s), _p(b), _p(y), _p(ids), C.c_long(T), C.c_long(S), C.c_long(N),
                            C.c_long(K), C.c_int(bits), C.c_int(group), C.c_long(in_slot), C.c_long(in_tok),
                            C.c_long(S), C.c_int(int(w16)))
    return y


def router_topk(logits, E: int, K: int, norm_topk: bool, has_shared: bool):
    l = _c(np.atleast_2d(logits), np.float32)
    T = l.shape[0]
    S = K + int(has_shared)
    ids = np.empty((T, S), dtype=np.uint32)
    sc = np.empty((T, S), dtype=np.float32)
    lib().zo_router_topk(_p(l), _p(ids), _p(sc), C.c_long(T), C.c_int(E), C.c_int(K), C.c_int(int(norm_topk)),
                         C.c_int(int(has_shared)))
    return ids, sc


def silu_mul(gate_up, ffn: int):
    gu = _f16bits(gate_up)
    rows = gu.size // (2 * ffn)
    h = np.empty(gu.shape[:-1] + (ffn,), dtype=np.float16)
    lib().zo_silu_mul(_p(gu), _p(h.view(np.uint16)), C.c_long(rows), C.c_long(ffn))
    return h


def moe_combine(y_slots, scores):
    y = _f16bits(y_slots)
    T, S, d = y.shape
    sc = _c(scores, np.float32)
    out = np.empty((T, d), dtype=np.float16)
    lib().zo_moe_combine(_p(y), _p(sc), _p(out.view(np.uint16)), C.c_long(T), C.c_long(S), C.c_long(d))
    return out
