"""CPU tests of the host side: entry names, PODArgs, variant resolution, and that the C-ABI library
loads and exports every symbol the header declares (no compute without a GPU)."""
import ctypes
import os
import re

import pytest

import zero_tvm_b200 as z
from zero_tvm_b200.backend import (Int4MatmulOpts, int4_matmul_entry, moe_down_pod_args, moe_gate_pod_args,
                                   moe_slots, parse_entry, pick_chunk_gemm, pod_args, resolve_matmul)

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# The 34 shipped variants, in the order of INT4_MATMUL_VARIANTS (int4_matmul.gen.ts:701-766).
SHIPPED = [
    (dict(), "int4_matmul"),
    (dict(subgroups=True), "int4_matmul_sg"),
    (dict(subgroups=True, rows_per_wg=4), "int4_matmul_tiled"),
    (dict(subgroups=True, rows_per_wg=8), "int4_matmul_tiled8"),
    (dict(out_f32=True), "int4_matmul_f32"),
    (dict(out_f32=True, subgroups=True), "int4_matmul_f32_sg"),
    (dict(out_f32=True, subgroups=True, rows_per_wg=4), "int4_matmul_f32_tiled"),
    (dict(out_f32=True, subgroups=True, rows_per_wg=8), "int4_matmul_f32_tiled8"),
    (dict(subgroups=True, rows_per_wg=4, m=4), "int4_matmul_batched_m4"),
    (dict(subgroups=True, rows_per_wg=4, m_dyn=True), "int4_matmul_batched_dyn"),
    (dict(subgroups=True, rows_per_wg=4, m_dyn=True, affine=True), "int4_matmul_batched_dyn_affine"),
    (dict(subgroups=True, vec4=True), "int4_matmul_sg_vec4"),
    (dict(subgroups=True, rows_per_wg=4, vec4=True), "int4_matmul_tiled_vec4"),
    (dict(out_f32=True, subgroups=True, vec4=True), "int4_matmul_f32_sg_vec4"),
    (dict(out_f32=True, subgroups=True, rows_per_wg=4, vec4=True), "int4_matmul_f32_tiled_vec4"),
    (dict(subgroups=True, vec4_half=True), "int4_matmul_sg_vec4h"),
    (dict(subgroups=True, rows_per_wg=4, vec4_half=True), "int4_matmul_tiled_vec4h"),
    (dict(out_f32=True, subgroups=True, vec4_half=True), "int4_matmul_f32_sg_vec4h"),
    (dict(out_f32=True, subgroups=True, rows_per_wg=4, vec4_half=True), "int4_matmul_f32_tiled_vec4h"),
    (dict(affine=True), "int4_matmul_affine"),
    (dict(out_f32=True, affine=True), "int4_matmul_f32_affine"),
    (dict(subgroups=True, affine=True), "int4_matmul_sg_affine"),
    (dict(subgroups=True, rows_per_wg=4, affine=True), "int4_matmul_tiled_affine"),
    (dict(out_f32=True, subgroups=True, affine=True), "int4_matmul_f32_sg_affine"),
    (dict(out_f32=True, subgroups=True, rows_per_wg=4, affine=True), "int4_matmul_f32_tiled_affine"),
    (dict(subgroups=True, vec4_half=True, affine=True), "int4_matmul_sg_vec4h_affine"),
    (dict(subgroups=True, rows_per_wg=4, vec4_half=True, affine=True), "int4_matmul_tiled_vec4h_affine"),
    (dict(out_f32=True, subgroups=True, vec4_half=True, affine=True), "int4_matmul_f32_sg_vec4h_affine"),
    (dict(out_f32=True, subgroups=True, rows_per_wg=4, vec4_half=True, affine=True),
     "int4_matmul_f32_tiled_vec4h_affine"),
    (dict(affine=True, moe=True, subgroups=True, rows_per_wg=4), "int4_matmul_tiled_affine_moe"),
    (dict(affine=True, moe=True, subgroups=True, rows_per_wg=4, vec4_half=True),
     "int4_matmul_tiled_vec4h_affine_moe"),
    (dict(affine=True, q3=True), "int4_matmul_affine_q3"),
    (dict(affine=True, q3=True, subgroups=True, rows_per_wg=4), "int4_matmul_tiled_affine_q3"),
    (dict(affine=True, q3=True, moe=True, subgroups=True, rows_per_wg=4), "int4_matmul_tiled_affine_q3_moe"),
]


def test_shipped_variant_names_and_decoding():
    assert len(SHIPPED) == 34
    for kw, name in SHIPPED:
        o = Int4MatmulOpts(**kw)
        assert int4_matmul_entry(o) == name
        info = parse_entry(name)
        assert info.affine == o.affine and info.bits == (3 if o.q3 else 4)
        assert info.out_f32 == o.out_f32 and info.moe == o.moe
        assert info.has_m_rows == o.m_dyn and info.fixed_m == (4 if o.m == 4 else None)


@pytest.mark.parametrize("kw", [
    dict(moe=True), dict(q3=True), dict(affine=True, m=4, subgroups=True, rows_per_wg=4),
    dict(affine=True, q3=True, subgroups=True, vec4_half=True), dict(affine=True, moe=True, subgroups=True, vec4=True),
    dict(rows_per_wg=4), dict(m=4), dict(vec4=True), dict(subgroups=True, vec4=True, vec4_half=True),
    dict(subgroups=True, rows_per_wg=4, m_dyn=True, out_f32=True),
])
def test_generator_rejections(kw):
    """The combinations int4MatmulWGSL throws on (int4_matmul.gen.ts:172-196)."""
    with pytest.raises(ValueError):
        int4_matmul_entry(Int4MatmulOpts(**kw))


def test_prefill_gemm_entries_and_unknown():
    for base in ("int4_matmul_tiled_m", "int4_matmul_tiled_st", "int4_matmul_sgmat", "int4_matmul_sg_e1",
                 "int4_matmul_sg_e5"):
        for aff in (False, True):
            info = parse_entry(base + ("_affine" if aff else ""))
            assert info.has_m_rows and info.affine == aff and info.bits == 4
    for bad in ("int4_matmul_q3", "int4_matmul_moe", "rms_norm", "int4_matmul_tiled_vec4_vec4h"):
        with pytest.raises(KeyError):
            parse_entry(bad)


def test_pod_args():
    assert pod_args(2048, 8192) == [256, 32, 8192]
    assert pod_args(4096, 12288, bits=3) == [384, 64, 12288]
    assert pod_args(2048, 8192, group=32, m_rows=512) == [256, 64, 8192, 512]
    # Qwen3.6-35B-A3B-class: d=2048, ffn=512, 8+1 slots (engine-core.ts:1049-1056)
    assert moe_slots(8, True) == 9 and moe_slots(8, False) == 8
    assert moe_gate_pod_args(2048, 512, 9) == [256, 32, 512, 0, 1024, 2048, 9 * 1024, 9]
    assert moe_down_pod_args(2048, 512, 9) == [64, 8, 2048, 512, 2048, 9 * 512, 9 * 2048, 9]
    assert moe_gate_pod_args(2048, 512, 9, bits=3)[0] == 192


def test_resolve_matmul():
    """tests/unit/resolve-matmul-affine.test.ts:76-117: affine picks the affine family, wide rung by K."""
    assert resolve_matmul(affine=True, K=4096) == "int4_matmul_tiled_vec4h_affine"
    assert resolve_matmul(affine=True, K=4096, out_f32=True) == "int4_matmul_f32_tiled_vec4h_affine"
    assert resolve_matmul(affine=True, K=768) == "int4_matmul_tiled_affine"
    assert resolve_matmul(affine=False, K=3072) == "int4_matmul_tiled_vec4"
    assert resolve_matmul(affine=False, K=2560) == "int4_matmul_tiled_vec4h"
    assert resolve_matmul(affine=False, K=1408) == "int4_matmul_tiled"
    assert resolve_matmul(affine=True, K=4096, subgroups=False) == "int4_matmul_affine"
    assert resolve_matmul(affine=True, K=4096, q3=True) == "int4_matmul_tiled_affine_q3"
    assert resolve_matmul(affine=True, K=2048, moe=True) == "int4_matmul_tiled_vec4h_affine_moe"
    assert resolve_matmul(affine=True, K=768, moe=True) == "int4_matmul_tiled_affine_moe"
    assert resolve_matmul(affine=True, K=2048, moe=True, q3=True) == "int4_matmul_tiled_affine_q3_moe"


def test_pick_chunk_gemm():
    """tests/unit/chunk-gemm-pick.test.ts: default ladder, and an explicit request that cannot run throws."""
    assert pick_chunk_gemm(None, affine=True, K=2048) == "int4_matmul_sg_e5_affine"
    assert pick_chunk_gemm(None, affine=False, K=2080) == "int4_matmul_batched_dyn"
    assert pick_chunk_gemm("e1", affine=True, K=4096) == "int4_matmul_sg_e1_affine"
    assert pick_chunk_gemm("matvec", affine=True, K=2080) == "int4_matmul_batched_dyn_affine"
    with pytest.raises(ValueError):
        pick_chunk_gemm("e5", affine=True, K=2080)
    with pytest.raises(ValueError):
        pick_chunk_gemm("nope", affine=True, K=2048)


def _declared_symbols():
    hdr = open(os.path.join(ROOT, "include", "ztvm_b200.h")).read()
    return re.findall(r"ZTVM_API\s+[\w\s\*]+?\b(ztvm_\w+)\s*\(", hdr)


def test_library_exports_every_declared_symbol():
    z.build.build()
    lib = ctypes.CDLL(z.capi.LIB_PATH)
    declared = _declared_symbols()
    assert len(declared) >= 15
    assert sorted(declared) == sorted(z.capi.SYMBOLS)
    for name in declared:
        assert hasattr(lib, name), name
    assert z.capi.load().ztvm_version() == 100
    assert z.capi.load().ztvm_status_string(3) == b"unsupported combination"


def test_no_cpu_path():
    """Without a GPU the product fails loudly instead of computing somewhere else."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(z.ZtvmError) as e:
        z.Context(0)
    assert e.value.status in (z.capi.ERR_CUDA, z.capi.ERR_BAD_CONTEXT)
    # validation that needs no device: a NULL context is refused by every entry point
    lib = z.capi.load()
    d = z.MmDesc(2048, 8192, 1, 64, 4, 1, 0)
    assert lib.ztvm_int4_matmul(None, ctypes.byref(d), None, None, None, None, None, None) == z.capi.ERR_BAD_CONTEXT
    assert lib.ztvm_destroy(None) == z.capi.ERR_BAD_CONTEXT
    assert b"NULL" in lib.ztvm_last_error(None)


def test_backend_dispatch_argument_errors_need_no_gpu():
    be = object.__new__(z.backend.CudaMatmulBackend)  # no context: only the decoding is exercised
    with pytest.raises(KeyError):
        be.dispatch("int4_matmul_nope", [1, 2, 3, 4, [256, 32, 8]])
    with pytest.raises(ValueError):
        be.dispatch("int4_matmul_affine", [1, 2, 3, 4, [256, 32, 8]])            # no biases at slot 5
    with pytest.raises(ValueError):
        be.dispatch("int4_matmul_tiled_affine_moe", [1, 2, 3, 4, [256, 32, 8], 5])  # no ids / short PODArgs
    with pytest.raises(ValueError):
        be.dispatch("int4_matmul_batched_dyn_affine", [1, 2, 3, 4, [256, 32, 8], 5])  # no M_ROWS


def test_bench_workload_parsing_and_algorithmic_bytes():
    """bench.py's shape: syntax and its algorithmic-byte count (weights + scales + biases + activations + outputs)."""
    import importlib.util
    import os
    spec = importlib.util.spec_from_file_location("ztvm_bench", os.path.join(os.path.dirname(os.path.dirname(__file__)), "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    assert bench.workload_shapes("shape:12288x4096x4") == [("W[12288,4096] M=4", 12288, 4096, 4, False)]
    assert bench.workload_shapes("shape:151936x4096x1xf32")[0][-1] is True
    assert bench.workload_shapes("prefill_gemm_m512")[0][1:4] == (8192, 2048, 512)
    assert len(bench.workload_shapes("decode_layer_set")) == 8
    # config 0: 8192 x 2048 int4 g64 affine, M = 1, f16 out
    assert bench.algorithmic_bytes(8192, 2048, 1) == 8192 * 1024 + 2 * 8192 * 32 * 2 + 2048 * 2 + 8192 * 2
    with pytest.raises(SystemExit):
        bench.workload_shapes("no_such_workload")


def test_plan_dispatch_uses_a_kernels_hook_when_there_is_one():
    """sharded.plan_dispatch: the tensor-op plan and a kernels object's dispatch_plan give interchangeable plans."""
    import numpy as np
    import torch
    from zero_tvm_b200 import sharded
    rng = np.random.default_rng(5)
    ids = torch.from_numpy(rng.integers(0, 32, size=(20, 4)).astype(np.int32))
    ref = sharded.plan_dispatch(ids, 32, 1)
    assert ref.send_counts == [80] and ref.recv_counts == [80]
    assert sorted(ref.order.tolist()) == list(range(80))
    assert torch.equal(ref.local_expert, (ids.reshape(-1).to(torch.int64)[ref.order] % 32).to(torch.int32))

    class Hook:
        calls = 0

        def dispatch_plan(self, ids_routed, epr, world):
            Hook.calls += 1
            flat = ids_routed.reshape(-1).to(torch.int64)
            order = torch.argsort(flat, stable=True)            # by expert: also by owner rank
            return order, (flat[order] % epr).to(torch.int32), torch.bincount(flat // epr, minlength=world)[:world]

    got = sharded.plan_dispatch(ids, 32, 1, kernels=Hook())
    assert Hook.calls == 1 and got.send_counts == ref.send_counts
    assert sorted(got.order.tolist()) == list(range(80))
    assert torch.equal(got.local_expert, (ids.reshape(-1).to(torch.int64)[got.order] % 32).to(torch.int32))


def test_chunk_cap_and_gemm_ladder():
    """resolveChunkCap and pickChunkGemm as the reference's pure functions (src/zero-tvm/engine-core.ts:195-245)."""
    from zero_tvm_b200.backend import pick_chunk_gemm_ladder, resolve_chunk_cap
    assert resolve_chunk_cap() == 1024 and resolve_chunk_cap(sgmat_avail=False) == 64
    assert resolve_chunk_cap(chunk_cap=96) == 96 and resolve_chunk_cap(max_chunk_cap=256) == 256
    assert resolve_chunk_cap(max_chunk_cap=256, sgmat_avail=False) == 64
    assert pick_chunk_gemm_ladder() == ("e5", None)
    assert pick_chunk_gemm_ladder(e5_ready=False) == ("sgmat", None)
    assert pick_chunk_gemm_ladder(e5_ready=False, sgmat_ready=False) == ("matvec", None)
    assert pick_chunk_gemm_ladder(cap_tiles64=False) == ("sgmat", None)            # nothing asked for: the ladder applies
    assert pick_chunk_gemm_ladder(chunk_tiled=True, e5_ready=False, sgmat_ready=False) == ("tiled", None)
    used, why = pick_chunk_gemm_ladder(want="e5", cap_tiles64=False, cap=96)
    assert used == "sgmat" and "cap must be %64 (got 96)" in why
    used, why = pick_chunk_gemm_ladder(want="sgmat", dims_ok=False, cap=1000)
    assert used == "matvec" and "dims do not tile" in why
    used, why = pick_chunk_gemm_ladder(want="e5", e5_ready=False)
    assert used == "sgmat" and "not built" in why
    assert pick_chunk_gemm_ladder(want="tiled") == ("tiled", None) and pick_chunk_gemm_ladder(want="matvec") == ("matvec", None)


def test_resolve_matmul_for_spec_and_int8_entries():
    from zero_tvm_b200.backend import parse_entry, resolve_matmul_for_spec
    assert resolve_matmul_for_spec(weight_format="mlx-safetensors", weight_bits=8, K=4096) == "int8_affine_matvec"
    assert resolve_matmul_for_spec(weight_format="mlx-safetensors", K=4096) == "int4_matmul_sg_tiled_vec4h_affine" or \
        resolve_matmul_for_spec(weight_format="mlx-safetensors", K=4096).endswith("_affine")
    assert not resolve_matmul_for_spec(weight_format="mlc", K=4096).endswith("_affine")
    with pytest.raises(ValueError):
        resolve_matmul_for_spec(weight_format="mlx-safetensors", weight_bits=8, K=4096, moe=True)
    for name, m_rows in (("int8_affine_matvec", False), ("int8_affine_batched", True)):
        info = parse_entry(name)
        assert info.bits == 8 and info.affine and info.has_m_rows == m_rows and not info.moe


def test_public_header_is_plain_c():
    """include/ztvm_b200.h is the binding surface for cgo / N-API / ctypes style callers: it must compile as C99 by itself."""
    import os
    import shutil
    import subprocess
    import tempfile
    if not shutil.which("gcc"):
        pytest.skip("no C compiler")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    with tempfile.TemporaryDirectory() as d:
        src = os.path.join(d, "hdr.c")
        with open(src, "w") as fh:
            fh.write('#include "ztvm_b200.h"\nint main(void) { ztvm_mm_desc d = {0}; (void)d; return 0; }\n')
        r = subprocess.run(["gcc", "-std=c99", "-Wall", "-Wextra", "-pedantic", "-Werror", "-fsyntax-only",
                            "-I", os.path.join(root, "include"), src], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
