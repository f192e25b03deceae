"""ztvm_int4_matmul_moe_noalloc: the grouped MoE matmul with its plan in a fixed device array.

Checked through the C ABI against ztvm_int4_matmul_moe on the same inputs (from 128 pairs on both entry points pick
the same grouped kernel; the cases below cover the streaming kernel and the tensor-core tiles): bit-identical outputs,
on two calls in a row, and again after the shapes changed in between. Every output is also graded against the
oracle's fp64 anchor (2e-3), including a call below 128 pairs, where the allocating entry point runs the per-pair
GEMV and the two results are close but not bit-identical.
The file name keeps it last in collection order, so it also runs after every other GPU test has used the library.
"""
import numpy as np
import pytest

import zero_tvm_b200 as z
from oracle import ztvm_oracle as zo
from conftest import record_parity

pytestmark = pytest.mark.gpu
TOL = 2e-3


def check_against_oracle(oracle_c, y_bits, mb, ids, tiles):
    """fp64 anchor over the weights the kernel multiplies: W16 for the tensor-core tiles, fl32(s*q+b) otherwise."""
    d, ffn = mb["hidden"], mb["ffn"]
    ref = oracle_c.moe_matmul_f64(mb["x"], *mb["gate"], ids, ffn, d, 64, 4, in_per_slot=False, w16=tiles)
    y = y_bits.view(np.float16).astype(np.float64)
    err = zo.rel_err_scaled(y, ref, 1e-2 if tiles else 1e-3)
    record_parity(err, zo.rel_err(y, ref))
    assert err <= TOL, f"rel err {err:.3e}"


def moe_desc(K, N, experts, slots, tokens, in_slot, out_slot, in_tok, out_tok, bits=4):
    return z.MoeDesc(z.MmDesc(K, N, 1, 64, bits, 1, 0), experts, slots, tokens, in_slot, out_slot, in_tok, out_tok, slots)


def both_entries(backend, dev, mb, ids, slots, seed_fill):
    """gate projection of `mb` over `ids` through the allocating and the non-allocating entry point."""
    T, d, ffn, E1 = mb["T"], mb["hidden"], mb["ffn"], mb["E"] + int(mb["has_shared"])
    gw, gs, gb = (dev.put(a) for a in mb["gate"])
    x, idt = dev.put(mb["x"]), dev.put(ids)
    desc = moe_desc(d, ffn, E1, slots, T, 0, ffn, d, slots * ffn)
    y_ref = dev.empty((T, slots, ffn), np.float16, fill=seed_fill)
    y_new = dev.empty((T, slots, ffn), np.float16, fill=seed_fill)
    backend.ctx.int4_matmul_moe(desc, y_ref, x, gs, gw, gb, idt)
    backend.ctx.int4_matmul_moe_noalloc(desc, y_new, x, gs, gw, gb, idt)
    backend.ctx.sync()
    assert backend.ctx.device_errors() == 0
    return dev.get(y_ref).view(np.uint16), dev.get(y_new).view(np.uint16)


def test_noalloc_matches_the_allocating_entry_twice_in_a_row(backend, dev, oracle_c):
    mb = z.synth.moe_block(48, E=16, hidden=512, ffn=256, seed=11)
    slots = 5
    rng = np.random.default_rng(3)
    ids = rng.integers(0, 17, size=(48, slots), dtype=np.uint32)          # 240 pairs: the grouped path on both sides
    for call in range(2):
        ref, new = both_entries(backend, dev, mb, ids, slots, seed_fill=3.0 + call)
        assert np.array_equal(ref, new), f"call {call}"
        assert (ref != np.float16(3.0 + call).view(np.uint16)).any()     # something was written
        check_against_oracle(oracle_c, new, mb, ids, tiles=True)         # 240 pairs over 17 experts (14 each): tensor-core tiles
    # a different problem (more experts, fewer rows per expert), then the first one again: nothing may survive in
    # the array from one call to the next
    mb2 = z.synth.moe_block(32, E=64, hidden=256, ffn=128, seed=12)
    ids2 = np.random.default_rng(4).integers(0, 65, size=(32, 9), dtype=np.uint32)
    ref2, new2 = both_entries(backend, dev, mb2, ids2, 9, seed_fill=5.0)
    assert np.array_equal(ref2, new2)
    check_against_oracle(oracle_c, new2, mb2, ids2, tiles=False)     # 288 pairs over 65 experts: streaming kernel
    ref, new = both_entries(backend, dev, mb, ids, slots, seed_fill=9.0)
    assert np.array_equal(ref, new)
    # many pairs per expert: both entry points run the tensor-core tiles
    mb3 = z.synth.moe_block(192, E=2, hidden=256, ffn=128, seed=13)
    ids3 = np.random.default_rng(5).integers(0, 3, size=(192, 3), dtype=np.uint32)
    ref3, new3 = both_entries(backend, dev, mb3, ids3, 3, seed_fill=2.0)
    assert np.array_equal(ref3, new3)
    check_against_oracle(oracle_c, new3, mb3, ids3, tiles=True)
    # below 128 pairs the allocating entry point runs the per-pair GEMV while this one still runs a grouped kernel:
    # both must meet the oracle, bit-identity between them is not promised there
    mb4 = z.synth.moe_block(6, E=8, hidden=512, ffn=128, seed=14)
    ids4 = np.random.default_rng(6).integers(0, 9, size=(6, 4), dtype=np.uint32)
    ref4, new4 = both_entries(backend, dev, mb4, ids4, 4, seed_fill=4.0)
    check_against_oracle(oracle_c, ref4, mb4, ids4, tiles=False)
    check_against_oracle(oracle_c, new4, mb4, ids4, tiles=False)


def test_noalloc_counts_bad_ids_and_leaves_their_rows_alone(backend, dev):
    mb = z.synth.moe_block(32, E=8, hidden=256, ffn=128, seed=6)
    slots = 5
    ids = np.random.default_rng(0).integers(0, 9, size=(32, slots), dtype=np.uint32)
    ids[7, 1] = 1000
    gw, gs, gb = (dev.put(a) for a in mb["gate"])
    y = dev.empty((32, slots, 128), np.float16, fill=7.0)
    backend.ctx.int4_matmul_moe_noalloc(moe_desc(256, 128, 9, slots, 32, 0, 128, 256, slots * 128), y, dev.put(mb["x"]),
                                        gs, gw, gb, dev.put(ids))
    assert backend.ctx.device_errors() == 1
    got = dev.get(y)
    assert (got[7, 1] == 7.0).all() and (got[7, 0] != 7.0).any()


def test_noalloc_refuses_what_does_not_fit_or_is_not_a_tile_shape(backend, dev):
    mb = z.synth.moe_block(2, E=8, hidden=256, ffn=128, seed=1)
    gw, gs, gb = (dev.put(a) for a in mb["gate"])
    x = dev.put(mb["x"])
    y = dev.empty((2, 3, 128), np.float16)
    ids = dev.put(np.zeros((2, 3), dtype=np.uint32))

    def call(**kw):
        a = dict(K=256, N=128, experts=9, slots=3, tokens=2, in_slot=0, out_slot=128, in_tok=256, out_tok=384)
        a.update(kw)
        backend.ctx.int4_matmul_moe_noalloc(moe_desc(**a), y, x, gs, gw, gb, ids)

    call()
    call(tokens=0)                                     # empty list: a no-op
    # refusals happen before any launch, so the (too small) buffers above are never touched
    for kw, code, word in ((dict(tokens=65536 // 3 + 1), z.capi.ERR_TOO_LARGE, "65536"),
                           (dict(experts=1025), z.capi.ERR_TOO_LARGE, "1024"),
                           (dict(bits=3), z.capi.ERR_UNSUPPORTED, "bits"),
                           (dict(in_tok=252), z.capi.ERR_ALIGNMENT, "strides")):
        with pytest.raises(z.ZtvmError) as e:
            call(**kw)
        assert e.value.status == code and word in str(e.value), (kw, e.value)
    backend.ctx.sync()
