"""Host-side mirror of the engine's matmul dispatch surface, on top of the C ABI.

The reference selects a WGSL pipeline by ENTRY NAME, binds buffers by slot
`[out, in, scales, weights, PODArgs, biases?, ids?]` (src/zero-tvm/engine-core.ts:76-92,
:1699-1703) and records `dispatch(enc, pipeline, bindGroup, wgX, wgY, wgZ, label)`
(src/zero-tvm/engine-core.ts:2151-2179). `CudaMatmulBackend.dispatch` takes the same things
and turns them into one call of libztvm_b200.so, so a call site keeps its shape:

    backend.dispatch("int4_matmul_tiled_vec4h_affine", [out, x, scales, weights, pod, biases], grid)

Everything the reference encodes in the entry name (bits, affine, f32 output, MoE) and in
PODArgs (K_PACKED, SCALES_PER_ROW, N, M_ROWS, MoE strides) is decoded here; the workgroup grid
only matters for the MoE kernels, where y is the token count and z the slot count.
"""
from __future__ import annotations

import re
from dataclasses import dataclass
from typing import Optional, Sequence

from . import capi
from .capi import MmDesc, MoeDesc


# ---- entry names (src/compiler/shaders/int4_matmul.gen.ts:32-152) ---------------------------
@dataclass(frozen=True)
class Int4MatmulOpts:
    out_f32: bool = False
    rows_per_wg: int = 1
    subgroups: bool = False
    m: int = 1
    vec4: bool = False
    vec4_half: bool = False
    m_dyn: bool = False
    affine: bool = False
    moe: bool = False
    q3: bool = False


def int4_matmul_entry(o: Int4MatmulOpts = Int4MatmulOpts()) -> str:
    """Entry-point name of a variant; same names and same rejections as the reference generator
    (int4_matmul.gen.ts:137-152 for names, :172-196 for the combinations it refuses)."""
    if o.moe and not o.affine:
        raise ValueError("moe requires affine")
    if o.q3 and not o.affine:
        raise ValueError("q3 requires affine")
    if o.affine and o.m != 1:
        raise ValueError("affine is implemented at m=1 (plus the mDyn path)")
    if o.q3 and (o.vec4 or o.vec4_half):
        raise ValueError("q3 has no wide-load path")
    if o.moe and o.vec4:
        raise ValueError("moe has no full-vec4 path")
    if o.rows_per_wg != 1 and not o.subgroups:
        raise ValueError("rowsPerWG > 1 requires subgroups")
    if o.m == 4 and (not o.subgroups or o.rows_per_wg != 4):
        raise ValueError("m=4 requires subgroups + rowsPerWG=4")
    if o.vec4 and (not o.subgroups or o.m != 1):
        raise ValueError("vec4 requires subgroups and m=1")
    if o.vec4_half and (o.vec4 or not o.subgroups or o.m != 1):
        raise ValueError("vec4Half requires subgroups + m=1 and excludes vec4")
    if o.m_dyn:
        if not o.subgroups or o.rows_per_wg != 4 or o.m != 1 or o.vec4 or o.vec4_half or o.out_f32:
            raise ValueError("mDyn requires subgroups + rowsPerWG=4 (no vec4/outF32/m=4)")
        return "int4_matmul_batched_dyn_affine" if o.affine else "int4_matmul_batched_dyn"
    if o.m == 4:
        return "int4_matmul_batched_m4"
    name = "int4_matmul"
    if o.out_f32:
        name += "_f32"
    if o.rows_per_wg == 4:
        name += "_tiled"
    elif o.rows_per_wg == 8:
        name += "_tiled8"
    elif o.subgroups:
        name += "_sg"
    if o.vec4:
        name += "_vec4"
    elif o.vec4_half:
        name += "_vec4h"
    if o.affine:
        name += "_affine"
    if o.q3:
        name += "_q3"
    if o.moe:
        name += "_moe"
    return name


# The prefill GEMM generators (int4_matmul.gen.ts:805-1456) and the runtime-M matvec (:580-695).
_GEMM_ENTRIES = {"int4_matmul_tiled_m", "int4_matmul_tiled_st", "int4_matmul_sgmat", "int4_matmul_sg_e1",
                 "int4_matmul_sg_e5", "int4_matmul_batched_dyn"}
_ENTRY_RE = re.compile(r"^int4_matmul(_f32)?(_tiled8|_tiled|_sg)?(_vec4h|_vec4)?(_affine)?(_q3)?(_moe)?$")


@dataclass(frozen=True)
class EntryInfo:
    affine: bool
    bits: int
    out_f32: bool
    moe: bool
    has_m_rows: bool      # PODArgs carries M_ROWS (runtime-M kernels)
    fixed_m: Optional[int]  # batched_m4


def parse_entry(entry: str) -> EntryInfo:
    """Decodes what an entry name fixes. Unknown names raise KeyError, as a missing pipeline does."""
    if entry == "int4_matmul_batched_m4":
        return EntryInfo(False, 4, False, False, False, 4)
    # the 8-bit family (src/compiler/shaders/int8_affine_matvec.wgsl, int8_affine_batched.wgsl): K_PACKED = K / 4
    if entry == "int8_affine_matvec":
        return EntryInfo(True, 8, False, False, False, None)
    if entry == "int8_affine_batched":
        return EntryInfo(True, 8, False, False, True, None)
    base = entry[:-len("_affine")] if entry.endswith("_affine") else entry
    if base in _GEMM_ENTRIES:
        return EntryInfo(entry.endswith("_affine"), 4, False, False, True, None)
    m = _ENTRY_RE.match(entry)
    if not m:
        raise KeyError(f"no such matmul pipeline: {entry}")
    f32, _rows, _wide, affine, q3, moe = m.groups()
    if (q3 or moe) and not affine:
        raise KeyError(f"no such matmul pipeline: {entry}")
    return EntryInfo(bool(affine), 3 if q3 else 4, bool(f32), bool(moe), False, None)


# ---- PODArgs builders (src/zero-tvm/engine-core.ts:787-794, :1021-1022, :1049-1056, :4033-4038) ----
def pod_args(K: int, N: int, *, bits: int = 4, group: int = 64, m_rows: Optional[int] = None):
    """[K_PACKED = K*bits/32, SCALES_PER_ROW = K/group, N(, M_ROWS)]."""
    p = [K * bits // 32, K // group, N]
    if m_rows is not None:
        p.append(m_rows)
    return p


def moe_gate_pod_args(d: int, ffn: int, slots: int, bits: int = 4):
    """gate / up: input shared across slots, output interleaved [slot][2*ffn] (engine-core.ts:1049-1052)."""
    return [d * bits // 32, d // 64, ffn, 0, 2 * ffn, d, slots * 2 * ffn, slots]


def moe_down_pod_args(d: int, ffn: int, slots: int, bits: int = 4):
    """down: per-slot input [slot][ffn], output [slot][d] (engine-core.ts:1053-1056)."""
    return [ffn * bits // 32, ffn // 64, d, ffn, d, slots * ffn, slots * d, slots]


def moe_slots(top_k: int, has_shared: bool) -> int:
    """moeSlots = topK + (shared ? 1 : 0) (src/compiler/model-spec.ts:659-660)."""
    return top_k + (1 if has_shared else 0)


# ---- variant resolution (src/zero-tvm/variants.ts:239-320, :370-388) -------------------------------
def resolve_matmul(*, affine: bool, K: int, out_f32: bool = False, subgroups: bool = True, q3: bool = False,
                   moe: bool = False) -> str:
    """The entry name the engine would pick for a decode projection: affine vs symmetric by checkpoint
    format, the wide-load rung by K divisibility (K%1024 -> vec4 for symmetric, K%512 -> vec4h), 4 rows per
    workgroup with subgroups. All of them land on the same CUDA GEMV; the name is kept so call sites and
    logs stay comparable with the reference."""
    if not subgroups:
        return int4_matmul_entry(Int4MatmulOpts(out_f32=out_f32, affine=affine, q3=q3))
    if q3 or (moe and K % 512):
        return int4_matmul_entry(Int4MatmulOpts(out_f32=out_f32, subgroups=True, rows_per_wg=4, affine=True,
                                                q3=q3, moe=moe))
    if affine:
        return int4_matmul_entry(Int4MatmulOpts(out_f32=out_f32, subgroups=True, rows_per_wg=4,
                                                vec4_half=(K % 512 == 0), affine=True, moe=moe))
    return int4_matmul_entry(Int4MatmulOpts(out_f32=out_f32, subgroups=True, rows_per_wg=4,
                                            vec4=(K % 1024 == 0), vec4_half=(K % 1024 != 0 and K % 512 == 0)))


def resolve_matmul_for_spec(*, weight_format: str, weight_bits: int = 4, K: int, out_f32: bool = False, q3: bool = False,
                            moe: bool = False) -> str:
    """One matmul instance for one spec (src/zero-tvm/variants.ts:370-388): the 8-bit branch first (an 8-bit checkpoint
    may never be served by the 4-bit kernels: silent wrong logits), everything else through resolve_matmul with the
    family decided by the checkpoint format."""
    if weight_bits == 8:
        if out_f32 or q3 or moe:
            raise ValueError("the 8-bit family has one matvec and one batched kernel: no f32-output, 3-bit or MoE twin")
        return "int8_affine_matvec"
    return resolve_matmul(affine=weight_format == "mlx-safetensors", K=K, out_f32=out_f32, q3=q3, moe=moe)


def resolve_chunk_cap(chunk_cap: Optional[int] = None, max_chunk_cap: Optional[int] = None, sgmat_avail: bool = True) -> int:
    """Rows per prefill chunk (src/zero-tvm/engine-core.ts:195-202): an explicit option wins; otherwise 1024 when the
    matrix-unit GEMM is there (it always is here), 64 without it, clamped by the spec's own maximum."""
    if chunk_cap is not None:
        return chunk_cap
    cap = 1024 if sgmat_avail else 64
    return cap if max_chunk_cap is None else min(cap, max_chunk_cap)


_GEMM_NAMES = {"e5": "int4_matmul_sg_e5", "e1": "int4_matmul_sg_e1", "sgmat": "int4_matmul_sgmat",
               "tiled": "int4_matmul_tiled_st", "matvec": "int4_matmul_batched_dyn"}


def pick_chunk_gemm_ladder(*, want: Optional[str] = None, chunk_tiled: bool = False, dims_ok: bool = True,
                           cap_tiles64: bool = True, e5_ready: bool = True, sgmat_ready: bool = True, cap: int = 1024):
    """The chunk-prefill GEMM ladder as the reference's pure function (src/zero-tvm/engine-core.ts:220-245):
    e5 > sgmat > tiled (only when asked for) > matvec. Returns (used, rejected): an EXPLICIT `want` that cannot run is a
    rejection carrying the throw text, never a silent substitution. All rungs land on the same tcgen05 GEMM here
    (matvec: the runtime-M GEMV path), so e5_ready / sgmat_ready default to True."""
    w = want if want is not None else ("e5" if e5_ready else "sgmat" if sgmat_ready else "matvec")
    ladder = [("e5", w == "e5" and dims_ok and cap_tiles64 and e5_ready),
              ("sgmat", w in ("sgmat", "e5") and dims_ok and sgmat_ready),
              ("tiled", (w == "tiled" or chunk_tiled) and dims_ok),
              ("matvec", True)]
    used = next(name for name, ok in ladder if ok)
    if want is not None and used != want:
        if not dims_ok:
            why = f"dims do not tile (cap {cap}, d/qDim/ffn must be %64 and cap %32)"
        elif want == "e5" and not cap_tiles64:
            why = f"E5 stages a 64-row tile, so cap must be %64 (got {cap})"
        elif want in ("e5", "sgmat"):
            why = "its pipeline was not built"
        else:
            why = "that pipeline was not built"
        return used, f"chunkGemm: asked for '{want}', can only run '{used}' — {why}"
    return used, None


def pick_chunk_gemm(requested: Optional[str], *, affine: bool, K: int, cap: int = 1024) -> str:
    """Entry name of the prefill GEMM for one projection: the ladder above with this projection's K as the tiling
    condition; a rejected explicit request raises (the reference throws at engine build, engine-core.ts:3969)."""
    suffix = "_affine" if affine else ""
    if requested is not None and requested not in _GEMM_NAMES:
        raise ValueError(f"unknown GEMM kernel '{requested}'")
    want = None if requested in (None, "e1") else requested
    used, rejected = pick_chunk_gemm_ladder(want=want, dims_ok=K % 64 == 0 and cap % 32 == 0, cap_tiles64=cap % 64 == 0, cap=cap)
    if rejected:
        raise ValueError(rejected)
    if requested == "e1":
        if K % 64:
            raise ValueError(f"GEMM kernel 'e1' needs K % 64 == 0 (K={K})")
        used = "e1"
    return _GEMM_NAMES[used] + suffix


# ---- the dispatch surface ---------------------------------------------------------------------------
class CudaMatmulBackend:
    """Drop-in for the matmul entries of compile() + dispatch(): one object per GPU."""

    def __init__(self, device: int = 0):
        self.ctx = capi.Context(device)

    def close(self):
        self.ctx.close()

    def dispatch(self, entry: str, bindings: Sequence, grid: Sequence[int] = (1, 1, 1), stream=None):
        """bindings = [out, in, scales, weights, PODArgs, biases?, ids?] in bind-group slot order;
        PODArgs is the list of u32 the engine writes into the uniform buffer.

        stream=None launches on the context's own stream, which is non-blocking: work queued on another stream (a
        tensor library's fills and copies, say) is NOT ordered against it. Pass that library's stream (a handle, a
        torch.cuda.Stream, or 1 for the legacy default stream), or synchronise both sides around the call."""
        info = parse_entry(entry)
        if len(bindings) < 5:
            raise ValueError("bind group needs [out, in, scales, weights, PODArgs, ...]")
        out, x, scales, weights, pod = bindings[:5]
        biases = bindings[5] if len(bindings) > 5 else None
        ids = bindings[6] if len(bindings) > 6 else None
        if info.affine and biases is None:
            raise ValueError(f"{entry}: affine variants bind biases at slot 5")
        k_packed, spr, n = int(pod[0]), int(pod[1]), int(pod[2])
        if k_packed <= 0 or spr <= 0 or (k_packed * 32) % info.bits:
            raise ValueError(f"{entry}: bad PODArgs {list(pod)}")
        K = k_packed * 32 // info.bits
        group = K // spr
        if info.moe:
            if len(pod) < 8 or ids is None:
                raise ValueError(f"{entry}: MoE variants need 8 PODArgs fields and ids at slot 6")
            gx, gy, gz = (list(grid) + [1, 1, 1])[:3]
            desc = MoeDesc(MmDesc(K, n, 1, group, info.bits, 1, 0), 0, gz, gy, int(pod[3]), int(pod[4]),
                           int(pod[5]), int(pod[6]), int(pod[7]))
            desc.experts = self._experts_of(weights, n, k_packed)
            self.ctx.int4_matmul_moe(desc, out, x, scales, weights, biases, ids, stream)
            return
        if info.fixed_m is not None:
            M = info.fixed_m
        elif info.has_m_rows:
            if len(pod) < 4:
                raise ValueError(f"{entry}: runtime-M kernels read M_ROWS from PODArgs[3]")
            M = int(pod[3])
            if M == 0:
                return
        else:
            M = 1
        desc = MmDesc(K, n, M, group, info.bits, int(info.affine), int(info.out_f32))
        self.ctx.int4_matmul(desc, out, x, scales, weights, biases if info.affine else None, stream)

    @staticmethod
    def _experts_of(weights, n: int, k_packed: int) -> int:
        """Rows of the expert stack, from the bound buffer's size (the reference relies on WebGPU's
        bounds checks; here an out-of-range id is counted and skipped, so the count must be known)."""
        if hasattr(weights, "numel"):
            return int(weights.numel() * weights.element_size() // (4 * n * k_packed))
        if hasattr(weights, "nbytes"):
            return int(weights.nbytes // (4 * n * k_packed))
        raise TypeError("MoE weights must be a sized buffer (tensor / array) so the expert count is known")

    # -- the router matvec and the embedding gather (their own bind-group orders in the reference) ---------------------
    def dispatch_router_logits(self, entry: str, bindings: Sequence, grid: Sequence[int] = (1, 1, 1), stream=None):
        """moe_router_logits / moe_router_logits_q4: [logits, x, w, scales, biases, {D, rows}]; moe_router_logits_f16:
        [logits, x, w, {D, rows}] (src/zero-tvm/engine-core.ts:2031-2033). grid = (rows, tokens, 1) (:2331, :4383)."""
        bits = {"moe_router_logits": 8, "moe_router_logits_q4": 4, "moe_router_logits_f16": 16}.get(entry)
        if bits is None:
            raise KeyError(f"no such router pipeline: {entry}")
        if bits == 16:
            logits, x, w, pod = bindings[:4]
            scales = biases = None
        else:
            logits, x, w, scales, biases, pod = bindings[:6]
        D, rows = int(pod[0]), int(pod[1])
        tokens = int((list(grid) + [1, 1])[1])
        self.ctx.moe_router_logits(D, rows, tokens, bits, logits, x, w, scales, biases, stream)

    def dispatch_embedding(self, entry: str, bindings: Sequence, D: int, stream=None):
        """embedding_affine / embedding_affine_int8: [out, input_ids, scales, weights, {seq_len, packGridDimX}, biases]
        (src/compiler/shaders/embedding_affine.wgsl:20-31); D is a pipeline constant in the reference."""
        bits = {"embedding_affine": 4, "embedding_affine_int8": 8}.get(entry)
        if bits is None:
            raise KeyError(f"no such embedding pipeline: {entry}")
        out, input_ids, scales, weights, pod, biases = bindings[:6]
        vocab = self._experts_of(weights, 1, D * bits // 32)
        self.ctx.embedding_affine(D, bits, vocab, int(pod[0]), out, input_ids, scales, weights, biases, stream)

    def dispatch_fused_ffn(self, entry: str, bindings: Sequence, D: int, ffn: int, m_rows: int = 1, stream=None):
        """fused_ffn: [output, input, scales, weights, {packGridDimX}] with the reference's symmetric group-32 weights
        (src/compiler/shaders/fused_ffn.wgsl:19-25; D and FFN_DIM are pipeline constants there); fused_ffn_affine:
        [output, input, scales, weights, {…}, biases], group 64 -- the sibling the engine lacks
        (src/zero-tvm/engine-core.ts:2513-2519). One workgroup per output in the reference: packGridDimX = ffn."""
        if entry not in ("fused_ffn", "fused_ffn_affine"):
            raise KeyError(f"no such fused FFN pipeline: {entry}")
        affine = entry.endswith("_affine")
        if len(bindings) < 5:
            raise ValueError("bind group needs [output, input, scales, weights, PODArgs, ...]")
        out, x, scales, weights = bindings[:4]
        biases = bindings[5] if affine and len(bindings) > 5 else None
        if affine and biases is None:
            raise ValueError(f"{entry}: affine variants bind biases at slot 5")
        desc = MmDesc(D, ffn, m_rows, 64 if affine else 32, 4, int(affine), 0)
        self.ctx.fused_ffn(desc, out, x, scales, weights, biases, stream)

    # MoE glue, same argument order as the reference bind groups
    def moe_router_topk(self, ids, scores, logits, E: int, K: int, norm_topk: bool, has_shared: bool, tokens: int,
                        stream=None):
        self.ctx.moe_route_topk(E, K, norm_topk, has_shared, tokens, ids, scores, logits, stream)

    def silu_mul(self, out, gate_up, rows: int, ffn: int, stream=None):
        self.ctx.silu_mul(rows, ffn, out, gate_up, stream)

    def moe_combine(self, out, y_slots, scores, tokens: int, slots: int, d: int, stream=None):
        self.ctx.moe_combine(tokens, slots, d, out, y_slots, scores, stream)
