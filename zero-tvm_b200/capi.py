"""ctypes binding of libztvm_b200.so — the same C ABI a Node-API addon would bind.

There is no fallback: if the shared library is missing or a call fails, an exception carries the
library's own message. Buffers are raw device addresses (ints) or any object with `data_ptr()`.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# ZTVM_LIB: path of another build of the same library (A/B measurements of build-time variants)
LIB_PATH = os.environ.get("ZTVM_LIB") or os.path.join(_HERE, "lib", "libztvm_b200.so")

# every symbol include/ztvm_b200.h declares
SYMBOLS = [
    "ztvm_version", "ztvm_status_string", "ztvm_init", "ztvm_destroy", "ztvm_last_error", "ztvm_sync",
    "ztvm_int4_matmul", "ztvm_int4_matmul_multi", "ztvm_int4_matmul_host", "ztvm_int4_matmul_host_async", "ztvm_host_wait", "ztvm_int4_matmul_moe", "ztvm_int4_matmul_moe_noalloc",
    "ztvm_moe_router_logits", "ztvm_embedding_affine", "ztvm_moe_plan_reuse", "ztvm_moe_route_topk", "ztvm_moe_dispatch_plan", "ztvm_moe_ep_dispatch", "ztvm_int4_matmul_moe_ep", "ztvm_silu_mul_rows", "ztvm_peer_barrier", "ztvm_moe_ffn_ep", "ztvm_int4_matmul_nshard",
    "ztvm_fused_ffn",
    "ztvm_silu_mul",
    "ztvm_moe_combine", "ztvm_unpack_codes", "ztvm_unpack_codes_streamed", "ztvm_dequant", "ztvm_device_errors",
]

OK, ERR_NULL_POINTER, ERR_BAD_DIMS, ERR_UNSUPPORTED, ERR_ALIGNMENT, ERR_CUDA, ERR_BAD_CONTEXT, ERR_TOO_LARGE = range(8)


class ZtvmError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"ztvm status {status}: {message}")
        self.status = status


class MmDesc(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("K", "N", "M", "group", "bits", "affine", "out_f32")]


class MoeDesc(C.Structure):
    _fields_ = [("mm", MmDesc)] + [(n, C.c_uint32) for n in (
        "experts", "slots", "tokens", "in_slot_stride", "out_slot_stride", "in_tok_stride", "out_tok_stride",
        "ids_stride")]


class MoeEpLayout(C.Structure):
    """Receive buffers of every rank as mapped in this process (include/ztvm_b200.h: ztvm_moe_ep_layout)."""
    _fields_ = [(n, C.c_uint32) for n in ("world", "rank", "experts_per_rank", "seg_cap")] + [
        ("recv_x", C.c_void_p * 8), ("recv_ids", C.c_void_p * 8), ("recv_src", C.c_void_p * 8), ("recv_cnt", C.c_void_p * 8),
        ("cursors", C.c_void_p)]


class MoeFfnEpArgs(C.Structure):
    """One expert-parallel FFN step (include/ztvm_b200.h: ztvm_moe_ffn_ep_args)."""
    _fields_ = [("layout", MoeEpLayout)] + [(n, C.c_uint32) for n in (
        "tokens", "top_k", "has_shared", "ids_stride", "d", "ffn", "x_tok_stride")] + [(n, C.c_void_p) for n in (
        "ids", "x", "gate_w", "gate_scales", "gate_biases", "up_w", "up_scales", "up_biases", "down_w", "down_scales",
        "down_biases", "gate_up", "h")] + [("y_slots", C.c_void_p * 8), ("flags", C.c_void_p * 8)]


class MoeEpRows(C.Structure):
    """Layout of an expert-parallel id list (include/ztvm_b200.h: ztvm_moe_ep_rows)."""
    _fields_ = [("seg_counts", C.c_void_p), ("seg_cap", C.c_uint32), ("segments", C.c_uint32), ("dst_index", C.c_void_p),
                ("y_seg", C.c_void_p * 9), ("reuse_plan", C.c_uint32)]


_lib = None


def load() -> C.CDLL:
    """Loads the library; raises if it has not been built (no CPU path exists)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ZtvmError(-1, f"{LIB_PATH} is missing: build it with `python zero-tvm_b200/build.py` "
                            "(CUDA sm_100a only; this package has no CPU implementation)")
    lib = C.CDLL(LIB_PATH)
    vp, u32, i32 = C.c_void_p, C.c_uint32, C.c_int32
    lib.ztvm_version.restype = i32
    lib.ztvm_status_string.restype = C.c_char_p
    lib.ztvm_status_string.argtypes = [i32]
    lib.ztvm_last_error.restype = C.c_char_p
    lib.ztvm_last_error.argtypes = [vp]
    sig = {
        "ztvm_init": [i32, C.POINTER(vp)],
        "ztvm_destroy": [vp],
        "ztvm_sync": [vp],
        "ztvm_int4_matmul": [vp, C.POINTER(MmDesc), vp, vp, vp, vp, vp, vp],
        "ztvm_int4_matmul_multi": [vp, C.POINTER(MmDesc), C.POINTER(C.c_void_p), u32, u32, vp, vp, vp, vp, vp],
        "ztvm_int4_matmul_host": [vp, C.POINTER(MmDesc), vp, vp, vp, vp, vp],
        "ztvm_int4_matmul_host_async": [vp, C.POINTER(MmDesc), vp, vp, vp, vp, vp],
        "ztvm_host_wait": [vp],
        "ztvm_int4_matmul_moe": [vp, C.POINTER(MoeDesc), vp, vp, vp, vp, vp, vp, vp],
        "ztvm_int4_matmul_moe_noalloc": [vp, C.POINTER(MoeDesc), vp, vp, vp, vp, vp, vp, vp],
        "ztvm_moe_router_logits": [vp, u32, u32, u32, u32, vp, vp, vp, vp, vp, vp],
        "ztvm_embedding_affine": [vp, u32, u32, u32, u32, vp, vp, vp, vp, vp, vp],
        "ztvm_moe_plan_reuse": [vp, i32],
        "ztvm_moe_route_topk": [vp, u32, u32, u32, u32, u32, vp, vp, vp, vp],
        "ztvm_moe_dispatch_plan": [vp, vp, u32, u32, u32, u32, u32, u32, vp, vp, vp, vp],
        "ztvm_moe_ep_dispatch": [vp, C.POINTER(MoeEpLayout), vp, u32, u32, u32, u32, vp, u32, u32, vp],
        "ztvm_int4_matmul_moe_ep": [vp, C.POINTER(MoeDesc), C.POINTER(MoeEpRows), vp, vp, vp, vp, vp, vp, vp],
        "ztvm_silu_mul_rows": [vp, C.POINTER(MoeEpRows), u32, vp, vp, vp],
        "ztvm_peer_barrier": [vp, C.POINTER(C.c_void_p), u32, u32, vp],
        "ztvm_moe_ffn_ep": [vp, C.POINTER(MoeFfnEpArgs), vp],
        "ztvm_int4_matmul_nshard": [vp, C.POINTER(MmDesc), C.POINTER(C.c_void_p), u32, u32, u32, vp, vp, vp, vp, C.POINTER(C.c_void_p), vp],
        "ztvm_fused_ffn": [vp, C.POINTER(MmDesc), vp, vp, vp, vp, vp, vp],
        "ztvm_silu_mul": [vp, u32, u32, vp, vp, vp],
        "ztvm_moe_combine": [vp, u32, u32, u32, vp, vp, vp, vp],
        "ztvm_unpack_codes": [vp, C.POINTER(MmDesc), vp, vp, vp],
        "ztvm_unpack_codes_streamed": [vp, C.POINTER(MmDesc), vp, vp, vp],
        "ztvm_dequant": [vp, C.POINTER(MmDesc), vp, i32, vp, vp, vp, vp],
        "ztvm_device_errors": [vp, vp, C.POINTER(u32)],
    }
    for name, args in sig.items():
        fn = getattr(lib, name)
        fn.restype = i32
        fn.argtypes = args
    _lib = lib
    return lib


def ptr(buf):
    """Device (or host) address of `buf`: None, int, or an object with data_ptr() / ctypes data."""
    if buf is None:
        return None
    if isinstance(buf, int):
        return C.c_void_p(buf)
    if hasattr(buf, "data_ptr"):
        return C.c_void_p(buf.data_ptr())
    if hasattr(buf, "ctypes"):
        return C.c_void_p(buf.ctypes.data)
    raise TypeError(f"cannot take the address of {type(buf)!r}")


def stream_ptr(stream):
    if stream is None:
        return None
    if isinstance(stream, int):
        return C.c_void_p(stream)
    return C.c_void_p(stream.cuda_stream)  # torch.cuda.Stream


def check(status: int):
    if status != OK:
        raise ZtvmError(status, load().ztvm_last_error(None).decode())


class Context:
    """One per GPU; owns the library context (stream, staging, error counter)."""

    def __init__(self, device: int = 0):
        self._lib = load()
        h = C.c_void_p()
        check(self._lib.ztvm_init(device, C.byref(h)))
        self.handle = h
        self.device = device

    def close(self):
        if getattr(self, "handle", None):
            check(self._lib.ztvm_destroy(self.handle))
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def sync(self):
        check(self._lib.ztvm_sync(self.handle))

    # -- entry points, thin and literal --------------------------------------------------------
    def int4_matmul(self, desc: MmDesc, y, x, scales, packed_w, biases=None, stream=None):
        check(self._lib.ztvm_int4_matmul(self.handle, C.byref(desc), ptr(y), ptr(x), ptr(scales), ptr(packed_w),
                                         ptr(biases), stream_ptr(stream)))

    def int4_matmul_host_async(self, desc: MmDesc, y_host, x_host, scales, packed_w, biases=None):
        """Queued form of int4_matmul_host (page-locked buffers, three lanes round robin); host_wait() completes them."""
        check(self._lib.ztvm_int4_matmul_host_async(self.handle, C.byref(desc), ptr(y_host), ptr(x_host), ptr(scales),
                                                    ptr(packed_w), ptr(biases)))

    def host_wait(self):
        check(self._lib.ztvm_host_wait(self.handle))

    def int4_matmul_host(self, desc: MmDesc, y_host, x_host, scales, packed_w, biases=None):
        check(self._lib.ztvm_int4_matmul_host(self.handle, C.byref(desc), ptr(y_host), ptr(x_host), ptr(scales),
                                              ptr(packed_w), ptr(biases)))

    def int4_matmul_multi(self, desc: MmDesc, y_dsts, y_row_stride, x, scales, packed_w, biases=None, stream=None):
        """Decode matmul whose result goes to every address in `y_dsts` (ints or tensors; peers' buffers included)."""
        addrs = [d if isinstance(d, int) else d.data_ptr() for d in y_dsts]
        arr = (C.c_void_p * len(addrs))(*addrs)
        check(self._lib.ztvm_int4_matmul_multi(self.handle, C.byref(desc), arr, len(addrs), y_row_stride, ptr(x),
                                               ptr(scales), ptr(packed_w), ptr(biases), stream_ptr(stream)))

    def int4_matmul_moe(self, desc: MoeDesc, y, x, scales, packed_w, biases, ids, stream=None):
        check(self._lib.ztvm_int4_matmul_moe(self.handle, C.byref(desc), ptr(y), ptr(x), ptr(scales),
                                             ptr(packed_w), ptr(biases), ptr(ids), stream_ptr(stream)))

    def int4_matmul_moe_noalloc(self, desc: MoeDesc, y, x, scales, packed_w, biases, ids, stream=None):
        """The grouped MoE matmul with its plan in a fixed device array (no allocation; limits in the header)."""
        check(self._lib.ztvm_int4_matmul_moe_noalloc(self.handle, C.byref(desc), ptr(y), ptr(x), ptr(scales),
                                                     ptr(packed_w), ptr(biases), ptr(ids), stream_ptr(stream)))

    def moe_router_logits(self, D, rows, tokens, bits, logits, x, w, scales=None, biases=None, stream=None):
        check(self._lib.ztvm_moe_router_logits(self.handle, D, rows, tokens, bits, ptr(logits), ptr(x), ptr(w), ptr(scales),
                                               ptr(biases), stream_ptr(stream)))

    def embedding_affine(self, D, bits, vocab, seq_len, out, input_ids, scales, weights, biases, stream=None):
        check(self._lib.ztvm_embedding_affine(self.handle, D, bits, vocab, seq_len, ptr(out), ptr(input_ids), ptr(scales),
                                              ptr(weights), ptr(biases), stream_ptr(stream)))

    def moe_plan_reuse(self, enable: bool):
        """Consecutive int4_matmul_moe calls over one id list share its expert-sorted plan (see the header's contract)."""
        check(self._lib.ztvm_moe_plan_reuse(self.handle, int(enable)))

    def moe_route_topk(self, E, K, norm_topk, has_shared, tokens, ids, scores, logits, stream=None):
        check(self._lib.ztvm_moe_route_topk(self.handle, E, K, int(norm_topk), int(has_shared), tokens, ptr(ids),
                                            ptr(scores), ptr(logits), stream_ptr(stream)))

    def moe_dispatch_plan(self, ids, tokens, slots, ids_stride, experts, experts_per_rank, world, order, local_expert,
                          send_counts, stream=None):
        check(self._lib.ztvm_moe_dispatch_plan(self.handle, ptr(ids), tokens, slots, ids_stride, experts, experts_per_rank,
                                               world, ptr(order), ptr(local_expert), ptr(send_counts), stream_ptr(stream)))

    def moe_ep_dispatch(self, layout: MoeEpLayout, ids, tokens, top_k, has_shared, ids_stride, x, d, x_tok_stride, stream=None):
        check(self._lib.ztvm_moe_ep_dispatch(self.handle, C.byref(layout), ptr(ids), tokens, top_k, int(has_shared), ids_stride,
                                             ptr(x), d, x_tok_stride, stream_ptr(stream)))

    def int4_matmul_moe_ep(self, desc: MoeDesc, rows: MoeEpRows, y, x, scales, packed_w, biases, ids, stream=None):
        check(self._lib.ztvm_int4_matmul_moe_ep(self.handle, C.byref(desc), C.byref(rows), ptr(y), ptr(x), ptr(scales),
                                                ptr(packed_w), ptr(biases), ptr(ids), stream_ptr(stream)))

    def peer_barrier(self, flags, world, rank, stream=None):
        """flags: every rank's flag-array address as mapped in this process (ints)."""
        arr = (C.c_void_p * 8)(*[int(f) for f in flags])
        check(self._lib.ztvm_peer_barrier(self.handle, arr, world, rank, stream_ptr(stream)))

    def int4_matmul_nshard(self, desc: MmDesc, y_dsts, world, rank, y_row_stride, x, scales, packed_w, biases, flags, stream=None):
        """ztvm_int4_matmul_multi + ztvm_peer_barrier: y_dsts / flags are every rank's addresses as mapped here (ints)."""
        ya = (C.c_void_p * 8)(*[int(v) for v in y_dsts])
        fa = (C.c_void_p * 8)(*[int(v) for v in flags])
        check(self._lib.ztvm_int4_matmul_nshard(self.handle, C.byref(desc), ya, world, rank, y_row_stride, ptr(x), ptr(scales),
                                                ptr(packed_w), ptr(biases), fa, stream_ptr(stream)))

    def moe_ffn_ep(self, args: "MoeFfnEpArgs", stream=None):
        check(self._lib.ztvm_moe_ffn_ep(self.handle, C.byref(args), stream_ptr(stream)))

    def silu_mul_rows(self, rows: MoeEpRows, ffn, h, gate_up, stream=None):
        check(self._lib.ztvm_silu_mul_rows(self.handle, C.byref(rows), ffn, ptr(h), ptr(gate_up), stream_ptr(stream)))

    def fused_ffn(self, desc: MmDesc, h, x, scales, packed_w, biases=None, stream=None):
        """h = f16(up * silu(gate)) for the [2 * desc.N, K] stack of gate and up rows (desc.N = ffn)."""
        check(self._lib.ztvm_fused_ffn(self.handle, C.byref(desc), ptr(h), ptr(x), ptr(scales), ptr(packed_w), ptr(biases),
                                       stream_ptr(stream)))

    def silu_mul(self, rows, ffn, h, gate_up, stream=None):
        check(self._lib.ztvm_silu_mul(self.handle, rows, ffn, ptr(h), ptr(gate_up), stream_ptr(stream)))

    def moe_combine(self, tokens, slots, d, out, y_slots, scores, stream=None):
        check(self._lib.ztvm_moe_combine(self.handle, tokens, slots, d, ptr(out), ptr(y_slots), ptr(scores),
                                         stream_ptr(stream)))

    def unpack_codes(self, desc: MmDesc, codes, packed_w, stream=None):
        check(self._lib.ztvm_unpack_codes(self.handle, C.byref(desc), ptr(codes), ptr(packed_w), stream_ptr(stream)))

    def unpack_codes_streamed(self, desc: MmDesc, codes, packed_w, stream=None):
        """Codes as the streaming matrix-unit kernels consume them (in-place f16 subnormals scaled back to integers)."""
        check(self._lib.ztvm_unpack_codes_streamed(self.handle, C.byref(desc), ptr(codes), ptr(packed_w), stream_ptr(stream)))

    def dequant(self, desc: MmDesc, w_out, as_f16, scales, packed_w, biases=None, stream=None):
        check(self._lib.ztvm_dequant(self.handle, C.byref(desc), ptr(w_out), int(as_f16), ptr(scales),
                                     ptr(packed_w), ptr(biases), stream_ptr(stream)))

    def device_errors(self, stream=None) -> int:
        n = C.c_uint32(0)
        check(self._lib.ztvm_device_errors(self.handle, stream_ptr(stream), C.byref(n)))
        return n.value
