"""Weight ingest (host side): safetensors header, bf16 -> f16 with overflow count and subnormal rounding, and the
buffer plans that concatenate q/k/v, gate/up and the expert stacks with the shared expert at index E
(src/zero-tvm/mlx-weights.ts:45-127, :272-380)."""
import json
import struct

import numpy as np
import pytest

import zero_tvm_b200 as z
from zero_tvm_b200 import ingest


def _bf16(a):
    """f32 -> bf16 bits by truncation-free construction: values chosen to be bf16-representable."""
    u = np.asarray(a, dtype=np.float32).view(np.uint32)
    assert ((u & 0xFFFF) == 0).all()
    return (u >> 16).astype(np.uint16)


def test_bf16_to_f16_matches_the_float32_cast_and_counts_overflow():
    rng = np.random.default_rng(0)
    b = rng.integers(0, 1 << 16, size=200000, dtype=np.uint16)          # every class of bf16 pattern
    h, over = ingest.bf16_to_f16(b)
    f32 = ingest.bf16_to_f32(b)
    with np.errstate(over="ignore"):
        ref = f32.astype(np.float16).view(np.uint16)
    finite = np.isfinite(f32)
    too_big = finite & (np.abs(f32) > 65504.0 * (1 + 2.0**-12))
    same = ~too_big & ~np.isnan(f32)
    assert np.array_equal(h[same], ref[same])                            # incl. subnormals (round to nearest even) and zeros
    assert over == int(np.isinf(ref.view(np.float16)[finite]).sum()) and over > 0
    clamped = finite & np.isinf(ref.view(np.float16))
    assert ((h[clamped] & 0x7FFF) == 0x7BFF).all() and ((h[clamped] & 0x8000) == (b[clamped] & 0x8000)).all()
    assert np.isnan(h[np.isnan(f32)].view(np.float16)).all()
    # the band quantisation scales live in: f16 subnormals must survive, not flush
    s = _bf16(np.array([2.0**-16, 3 * 2.0**-18, 2.0**-24, 2.0**-25, 2.0**-26], dtype=np.float32))
    hs, ov = ingest.bf16_to_f16(s)
    assert ov == 0 and list(hs) == [0x0100, 0x00C0, 0x0001, 0x0000, 0x0000]      # 2^-25 ties to even (zero)


def _safetensors(records):
    meta, blobs, off = {}, [], 0
    for name, (dtype, arr) in records.items():
        raw = np.ascontiguousarray(arr).tobytes()
        meta[name] = {"dtype": dtype, "shape": list(arr.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    head = json.dumps({"__metadata__": {"format": "mlx"}, **meta}).encode()
    return struct.pack("<Q", len(head)) + head + b"".join(blobs)


def test_plans_concatenate_rows_and_append_the_shared_expert():
    rng = np.random.default_rng(1)
    E, ffn, d = 4, 128, 256
    pre = "language_model.model."
    rec = {}

    def quant(base, lead, N, K):
        q, W, s, b = z.synth.make_weights(rng, N, K, lead=lead)
        rec[f"{base}.weight"] = ("U32", W)
        rec[f"{base}.scales"] = ("BF16", _bf16(s.astype(np.float32)))    # f16 values are bf16-representable? only if low bits are zero:
        rec[f"{base}.biases"] = ("BF16", _bf16(b.astype(np.float32)))
        return W, s, b
    # scales / biases with at most 8 significant bits so they survive bf16 exactly
    orig_make = z.synth.make_weights

    def make8(rng_, N, K, **kw):
        q, W, s, b = orig_make(rng_, N, K, **kw)
        trunc = lambda a: (a.astype(np.float32).view(np.uint32) & np.uint32(0xFFFF0000)).view(np.float32).astype(np.float16)
        return q, W, trunc(s), trunc(b)
    z.synth.make_weights = make8
    try:
        p = f"{pre}layers.3"
        qkv = [quant(f"{p}.self_attn.{n}_proj", (), N, d) for n, N in (("q", 256), ("k", 64), ("v", 64))]
        quant(f"{p}.self_attn.o_proj", (), d, 256)
        moe = {}
        for proj, (N, K) in (("gate_proj", (ffn, d)), ("up_proj", (ffn, d)), ("down_proj", (d, ffn))):
            moe[proj] = (quant(f"{p}.mlp.switch_mlp.{proj}", (E,), N, K), quant(f"{p}.mlp.shared_expert.{proj}", (), N, K))
        router = (quant(f"{p}.mlp.gate", (), E, d), quant(f"{p}.mlp.shared_expert_gate", (), 1, d))
    finally:
        z.synth.make_weights = orig_make
    blob = _safetensors(rec)
    tensors, start = ingest.parse_safetensors_header(blob)
    plans = ingest.plan_attention(pre, 3) + ingest.plan_moe_ffn(pre, 3, shared_expert=True, router_bits=4)
    bufs, overflow = ingest.build_buffers(plans, tensors, blob, start)
    assert overflow == 0
    # q ++ k ++ v: one [384, d/8] matmul
    W = np.concatenate([t[0] for t in qkv])
    assert np.array_equal(bufs["c_attn_w"].reshape(W.shape), W)
    assert np.array_equal(bufs["c_attn_s"].view(np.float16).reshape(384, -1), np.concatenate([t[1] for t in qkv]))
    # expert stacks: shared expert at index E
    for proj, (stack, shared) in moe.items():
        got = bufs[f"moe_{proj}_w"].reshape(E + 1, *stack[0].shape[1:])
        assert np.array_equal(got[:E], stack[0]) and np.array_equal(got[E], shared[0])
        gb = bufs[f"moe_{proj}_b"].view(np.float16).reshape(E + 1, *stack[2].shape[1:])
        assert np.array_equal(gb[E], shared[2])
    assert bufs["router_w"].size == (E + 1) * d // 8 and np.array_equal(bufs["router_w"][-d // 8:], router[1][0].reshape(-1))
    # the ingested stacks are what the oracle (and the kernels) consume: codes unpack to the originals
    from oracle import ztvm_oracle as zo
    g = bufs["moe_gate_proj_w"].reshape(E + 1, ffn, d // 8)
    assert np.array_equal(zo.unpack_codes(g, 4)[E], zo.unpack_codes(moe["gate_proj"][1][0], 4))
    with pytest.raises(KeyError):
        ingest.build_buffers(ingest.plan_dense_ffn(pre, 3), tensors, blob, start)       # this layer has no dense FFN


def test_header_errors():
    with pytest.raises(ValueError):
        ingest.parse_safetensors_header(b"\x10\x00")
    with pytest.raises(ValueError):
        ingest.parse_safetensors_header(struct.pack("<Q", 100) + b"{}")
