"""A whole step of this path recorded once and replayed from a CUDA graph through the C ABI: a dense decode layer's
projections and an MoE block (router logits -> top-k -> gate, up -> SiLU -> down -> combine), as the engine records
its per-token dispatch sequence (src/zero-tvm/engine-core.ts:2194-2202, :2290-2349). Replays must reproduce the eager
sequence bit for bit, including after the inputs changed in place."""
import numpy as np
import pytest

import zero_tvm_b200 as z
from zero_tvm_b200.backend import moe_down_pod_args, moe_gate_pod_args, pod_args, resolve_matmul

pytestmark = pytest.mark.gpu


def test_decode_step_graph_matches_eager(backend, dev):
    import torch
    rng = np.random.default_rng(5)
    d, ffn_dense, E, K_top, ffn = 512, 1024, 16, 4, 256
    slots, T = K_top + 1, 1
    rec = z.recorder.DecodeRecorder(backend)
    # dense part: fused qkv, o, fused gate_up, down
    x = dev.put(z.synth.make_x(rng, T, d))
    outs = {}
    for name, N, Kd in (("qkv", 768, d), ("o", d, d), ("gate_up", 2 * ffn_dense, d), ("down", d, ffn_dense)):
        _, W, s, b = z.synth.make_weights(rng, N, Kd)
        xin = x if Kd == d else dev.put(z.synth.make_x(rng, T, Kd))
        y = dev.empty((T, N), np.float16, fill=float("nan"))
        rec.dispatch(resolve_matmul(affine=True, K=Kd), [y, xin, dev.put(s), dev.put(W), pod_args(Kd, N), dev.put(b)], ((N + 3) // 4, 1, 1))
        outs[name] = y
    # MoE block
    mb = z.synth.moe_block(T, E=E, hidden=d, ffn=ffn, seed=9)
    _, RW, rs, rb = z.synth.make_weights(rng, E + 1, d, bits=8)
    logits = dev.empty((T, E + 1), np.float32, fill=float("nan"))
    ids = dev.empty((T, slots), np.uint32, fill=0)
    scores = dev.empty((T, slots), np.float32, fill=0.0)
    gu = dev.empty((T, slots, 2 * ffn), np.float16, fill=float("nan"))
    h = dev.empty((T, slots, ffn), np.float16, fill=float("nan"))
    ys = dev.empty((T, slots, d), np.float16, fill=float("nan"))
    y_moe = dev.empty((T, d), np.float16, fill=float("nan"))
    st = {n: tuple(dev.put(a) for a in mb[n]) for n in ("gate", "up", "down")}
    eg, ed = resolve_matmul(affine=True, K=d, moe=True), resolve_matmul(affine=True, K=ffn, moe=True)
    rec.router_logits("moe_router_logits", [logits, x, dev.put(RW), dev.put(rs), dev.put(rb), [d, E + 1]], (E + 1, T, 1))
    rec.router_topk(ids, scores, logits, E, K_top, True, True, T)
    rec.dispatch(eg, [gu, x, st["gate"][1], st["gate"][0], moe_gate_pod_args(d, ffn, slots), st["gate"][2], ids], (ffn // 4, T, slots))
    rec.dispatch(eg, [gu.view(-1)[ffn:], x, st["up"][1], st["up"][0], moe_gate_pod_args(d, ffn, slots), st["up"][2], ids], (ffn // 4, T, slots))
    rec.silu_mul(h, gu, T * slots, ffn)
    rec.dispatch(ed, [ys, h, st["down"][1], st["down"][0], moe_down_pod_args(d, ffn, slots), st["down"][2], ids], (d // 4, T, slots))
    rec.moe_combine(y_moe, ys, scores, T, slots, d)
    assert len(rec) == 11

    def snapshot():
        torch.cuda.synchronize()
        return {k: v.cpu().numpy().copy().view(np.uint16) for k, v in {**outs, "moe": y_moe}.items()}

    torch.cuda.synchronize()
    rec.run_eager()
    want = snapshot()
    assert all(np.isfinite(v.view(np.float16).astype(np.float32)).all() for v in want.values())
    step = rec.capture()
    for v in list(outs.values()) + [y_moe]:
        v.fill_(float("nan"))
    torch.cuda.synchronize()
    step.replay(); step.synchronize()
    got = snapshot()
    for k in want:
        assert np.array_equal(got[k], want[k]), k
    # a new token: the same buffers, new contents (as the engine rewrites its activation buffers in place)
    x.copy_(torch.from_numpy(z.synth.make_x(rng, T, d)).cuda())
    torch.cuda.synchronize()
    rec.run_eager()
    want2 = snapshot()
    assert not np.array_equal(want2["moe"], want["moe"])
    step.replay(); step.synchronize()
    got2 = snapshot()
    for k in want2:
        assert np.array_equal(got2[k], want2[k]), k
    assert backend.ctx.device_errors() == 0
