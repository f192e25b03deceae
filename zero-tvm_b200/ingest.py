"""Weight ingest for MLX-format safetensors checkpoints: records -> the buffers the matmul kernels bind.

Host-side mirror of the loader steps that sit in front of this path in the reference
(src/zero-tvm/mlx-weights.ts): the safetensors header (:45-75), bf16 -> f16 for scales and biases with an
overflow count and round-to-nearest-even subnormals (:100-127), and the buffer plans that concatenate
records row-wise -- q ++ k ++ v and the expert stacks with the shared expert appended at index E, its gate
row appended to the router (:272-375). Packed codes are taken as they are ("raw"): the kernels read the
checkpoint's own layout. numpy only; nothing here touches a GPU.
"""
from __future__ import annotations

import json
import struct
from dataclasses import dataclass, field
from typing import Dict, List, Mapping, Optional, Sequence, Tuple

import numpy as np


@dataclass(frozen=True)
class TensorInfo:
    dtype: str
    shape: Tuple[int, ...]
    begin: int
    end: int


def parse_safetensors_header(head: bytes) -> Tuple[Dict[str, TensorInfo], int]:
    """(tensors, data_start) from the first bytes of a .safetensors file (mlx-weights.ts:45-75): a little-endian u64
    header length, then that many bytes of JSON; `data_offsets` are relative to the end of the header."""
    if len(head) < 8:
        raise ValueError("safetensors: shorter than its own length field")
    (n,) = struct.unpack("<Q", head[:8])
    if n >> 32:
        raise ValueError("safetensors: header longer than 4 GB")
    if len(head) < 8 + n:
        raise ValueError(f"safetensors: header is {n} bytes, only {len(head) - 8} supplied")
    meta = json.loads(head[8:8 + n].decode("utf-8"))
    tensors = {}
    for name, m in meta.items():
        if name == "__metadata__":
            continue
        tensors[name] = TensorInfo(m["dtype"], tuple(m["shape"]), int(m["data_offsets"][0]), int(m["data_offsets"][1]))
    return tensors, 8 + n


def bf16_to_f16(src: np.ndarray) -> Tuple[np.ndarray, int]:
    """bf16 bit patterns (u16) -> f16 bit patterns (u16) and the number of overflows (mlx-weights.ts:100-127).

    Normal values convert exactly (f16 has more mantissa bits). Values beyond f16's range are CLAMPED to the largest
    finite f16 and counted -- an infinite scale becomes NaN logits thousands of launches later -- and the caller
    should treat a non-zero count as an error. Values in f16's subnormal band are rounded to nearest even, as a
    float32 -> float16 cast does; anything smaller flushes to a signed zero. Inf / NaN keep their class."""
    b = np.ascontiguousarray(src, dtype=np.uint16)
    f32 = (b.astype(np.uint32) << np.uint32(16)).view(np.float32)
    with np.errstate(over="ignore"):
        h = f32.astype(np.float16).view(np.uint16).copy()      # RNE, subnormals kept: the cast the reference matches
    raw_exp = (b >> np.uint16(7)) & np.uint16(0xFF)
    finite = raw_exp != 0xFF
    over = finite & ((h & np.uint16(0x7FFF)) == np.uint16(0x7C00))
    h[over] = (b[over] & np.uint16(0x8000)) | np.uint16(0x7BFF)
    nan = ~finite & ((b & np.uint16(0x7F)) != 0)
    h[nan] = (b[nan] & np.uint16(0x8000)) | np.uint16(0x7E00)
    return h, int(over.sum())


def bf16_to_f32(src: np.ndarray) -> np.ndarray:
    """bf16 IS the top half of an f32: a shift (mlx-weights.ts:130-136)."""
    return (np.ascontiguousarray(src, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


# ---- buffer plans -------------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class Part:
    record: str
    convert: str          # 'raw' | 'bf16->f16' | 'bf16->f32'


@dataclass
class BufferPlan:
    name: str
    parts: List[Part] = field(default_factory=list)


def _trio(name: str, bases: Sequence[str]) -> List[BufferPlan]:
    """One quantised buffer trio per logical tensor -- weights, scales, biases -- each the concatenation of the same
    component of every part (mlx-weights.ts:281-295)."""
    return [BufferPlan(f"{name}_w", [Part(f"{b}.weight", "raw") for b in bases]),
            BufferPlan(f"{name}_s", [Part(f"{b}.scales", "bf16->f16") for b in bases]),
            BufferPlan(f"{name}_b", [Part(f"{b}.biases", "bf16->f16") for b in bases])]


def plan_attention(prefix: str, layer: int) -> List[BufferPlan]:
    """c_attn = q ++ k ++ v rows in one matmul, o_proj on its own (mlx-weights.ts:340-343)."""
    p = f"{prefix}layers.{layer}.self_attn"
    return _trio("c_attn", [f"{p}.q_proj", f"{p}.k_proj", f"{p}.v_proj"]) + _trio("o_proj", [f"{p}.o_proj"])


def plan_dense_ffn(prefix: str, layer: int) -> List[BufferPlan]:
    """gate ++ up rows in one matmul (the fused FFN front half the engine dispatches once), down on its own."""
    p = f"{prefix}layers.{layer}.mlp"
    return _trio("gate_up", [f"{p}.gate_proj", f"{p}.up_proj"]) + _trio("down_proj", [f"{p}.down_proj"])


def plan_moe_ffn(prefix: str, layer: int, *, shared_expert: bool = True, router_bits: int = 8) -> List[BufferPlan]:
    """Expert stacks [E(+1), N, ...] with the shared expert appended at index E and its gate row appended to the
    router, so nothing downstream treats it as a special case (mlx-weights.ts:358-380)."""
    p = f"{prefix}layers.{layer}.mlp"
    plans: List[BufferPlan] = []
    for proj in ("gate_proj", "up_proj", "down_proj"):
        bases = [f"{p}.switch_mlp.{proj}"] + ([f"{p}.shared_expert.{proj}"] if shared_expert else [])
        plans += _trio(f"moe_{proj}", bases)
    gates = [f"{p}.gate"] + ([f"{p}.shared_expert_gate"] if shared_expert else [])
    if router_bits == 16:
        plans.append(BufferPlan("router_w", [Part(f"{g}.weight", "bf16->f16") for g in gates]))
    else:
        plans += _trio("router", gates)
    return plans


_DTYPES = {"U32": np.uint32, "BF16": np.uint16, "F16": np.uint16, "F32": np.float32, "U8": np.uint8, "I32": np.int32}


def build_buffers(plans: Sequence[BufferPlan], tensors: Mapping[str, TensorInfo], data: bytes,
                  data_start: int = 0) -> Tuple[Dict[str, np.ndarray], int]:
    """The buffers of `plans` as flat arrays (u32 codes, f16 bit patterns as u16, f32) and the total overflow count.
    Parts are converted, then concatenated in order: row-major tensors stacked along their leading axis."""
    out: Dict[str, np.ndarray] = {}
    overflow = 0
    for plan in plans:
        pieces = []
        for part in plan.parts:
            if part.record not in tensors:
                raise KeyError(f"{plan.name}: record {part.record} is not in the checkpoint")
            t = tensors[part.record]
            raw = np.frombuffer(data, dtype=_DTYPES[t.dtype], count=(t.end - t.begin) // np.dtype(_DTYPES[t.dtype]).itemsize,
                                offset=data_start + t.begin)
            if part.convert == "raw":
                pieces.append(raw)
            elif part.convert == "bf16->f16":
                if t.dtype == "F16":                       # already what the kernels read
                    pieces.append(raw)
                elif t.dtype == "BF16":
                    h, ov = bf16_to_f16(raw)
                    overflow += ov
                    pieces.append(h)
                else:
                    raise ValueError(f"{part.record}: cannot make f16 from {t.dtype}")
            elif part.convert == "bf16->f32":
                pieces.append(bf16_to_f32(raw) if t.dtype == "BF16" else raw.astype(np.float32))
            else:
                raise ValueError(f"unknown conversion {part.convert}")
        out[plan.name] = np.concatenate(pieces) if len(pieces) > 1 else pieces[0].copy()
    return out, overflow
