"""Generates tests/golden/*.npz by running the reference's OWN numpy code on seeded inputs.

Run once in a checkout that has the reference project mounted:

    python tests/golden/make_golden.py /path/to/reference

Two pieces of the reference can be executed without its GPU stack:

dequant_from_*.npz

`scripts/make-dsv2-layer-ref.py` cannot be imported (it parses argv at module scope), so
the single function `dequant_from` (lines 102-116) is located with `ast`, compiled on
its own against numpy and executed on seeded inputs. Nothing of its source is stored:
only the inputs and the outputs it produced. The reference documents that function as
bit-identical to `mx.dequantize`, which makes these the only executed-reference vectors
available for this path (the reference's WGSL and JS need WebGPU / node).

kernel_ref_q{4,3}_*.npz
`scripts/make-kernel-ref.py` builds its expected output inside `qwen36moe()`, a function that first imports mlx and
opens a checkpoint (both absent here). The statements that follow (lines 55-66: the 4-bit nibble unpack / the 3-bit
LSB-first bit-stream unpack, then `xg`, `dot`, `y` = sum_g s_g*dot_g + b_g*xsum_g) are pure numpy. They are
located with `ast` inside that function (the `if bits == 4` statement and the assignments to xg, dot, y), compiled on
their own and executed on seeded Wq / scales / biases / x. Stored: the inputs, the codes `nib` and `y` they produced.

silu_mul_ref.npz
`scripts/make-dsv2-layer-ref.py:283-284` `silu_mul(gate, up)` is a two-line numpy function; it is located with `ast`
and run on seeded f32 inputs that hold f16 values (what the engine's silu_mul kernel reads), large magnitudes included.

router_ref_*.npz
The same script routes one token in plain numpy at module level (lines 327-345: softmax over all experts, stable
arg-sort for a DESCENDING order with ties to the lower index, the K weights scaled and optionally renormalised). Those
statements (the assignments to probs, ids, topk_w, the `probs /= ...` and the `if args.norm_topk_prob`) are located
with `ast`, compiled on their own and executed once per token on seeded logits, some with exact ties.
"""
import ast
import os
import sys
import types

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def load_dequant_from(ref_root: str):
    path = os.path.join(ref_root, "scripts", "make-dsv2-layer-ref.py")
    tree = ast.parse(open(path).read())
    fn = next(n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name == "dequant_from")
    mod = ast.Module(body=[fn], type_ignores=[])
    ns = {"np": np}
    exec(compile(mod, path, "exec"), ns)
    return ns["dequant_from"]


def load_kernel_ref_statements(ref_root: str):
    """The unpack + factored-GEMV statements of qwen36moe() as a callable(ns) that executes them in `ns`."""
    path = os.path.join(ref_root, "scripts", "make-kernel-ref.py")
    tree = ast.parse(open(path).read())
    fn = next(n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name == "qwen36moe")
    picked = []
    for node in fn.body:
        if isinstance(node, ast.If) and isinstance(node.test, ast.Compare) and getattr(node.test.left, "id", "") == "bits":
            picked.append(node)                                   # if bits == 4: nibbles  else: bit stream
        elif isinstance(node, ast.Assign) and len(node.targets) == 1 and getattr(node.targets[0], "id", "") in ("xg", "dot", "y"):
            picked.append(node)
    names = [getattr(n.targets[0], "id", None) if isinstance(n, ast.Assign) else "if" for n in picked]
    assert names == ["if", "xg", "dot", "y"], names
    code = compile(ast.Module(body=picked, type_ignores=[]), path, "exec")

    def run(ns):
        exec(code, ns)
        return ns
    return run


def make_kernel_ref(ref_root: str):
    run = load_kernel_ref_statements(ref_root)
    cases = {
        # name: (bits, N, K, seed, scale sigma)
        "q4_small": (4, 24, 512, 21, 0.01), "q4_wide": (4, 48, 2048, 22, 0.01),
        "q3_small": (3, 24, 512, 23, 0.02), "q3_wide": (3, 48, 4096, 24, 0.02), "q3_ragged": (3, 13, 1408, 25, 0.02),
    }
    G = 64
    for name, (bits, N, K, seed, sig) in cases.items():
        rng = np.random.default_rng(seed)
        Wq = rng.integers(0, 1 << 32, size=(N, K * bits // 32), dtype=np.uint64).astype(np.uint32)
        S = np.abs(rng.standard_normal((N, K // G), dtype=np.float32) * np.float32(sig))
        B = rng.standard_normal((N, K // G), dtype=np.float32) * np.float32(0.05)
        x = (rng.standard_normal(K) * 0.05).astype(np.float16)     # the reference's activation scale (line 53)
        ns = {"np": np, "bits": bits, "Wq": Wq, "N": N, "K": K, "NG": K // G, "G": G, "x_f16": x,
              "scales_f16": S.astype(np.float16), "bias_f16": B.astype(np.float16)}
        run(ns)
        nib, y = ns["nib"], ns["y"]
        assert nib.shape == (N, K) and nib.max() < (1 << bits) and y.shape == (N,)
        np.savez_compressed(os.path.join(HERE, f"kernel_ref_{name}.npz"), W=Wq, scales=ns["scales_f16"],
                            biases=ns["bias_f16"], x=x, codes=nib.astype(np.uint8), y=y.astype(np.float32),
                            bits=np.int32(bits))
        print(name, Wq.shape, "-> codes", nib.shape, "y", y.shape)


def make_silu_mul(ref_root: str):
    path = os.path.join(ref_root, "scripts", "make-dsv2-layer-ref.py")
    tree = ast.parse(open(path).read())
    fn = next(n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name == "silu_mul")
    ns = {"np": np}
    exec(compile(ast.Module(body=[fn], type_ignores=[]), path, "exec"), ns)
    rng = np.random.default_rng(31)
    gate = (rng.standard_normal((64, 96)) * 3.0).astype(np.float16)
    up = (rng.standard_normal((64, 96)) * 2.0).astype(np.float16)
    gate[0, :8] = np.array([0.0, -0.0, 12.0, -12.0, 30.0, -30.0, 6.1e-5, -6.1e-5], dtype=np.float16)
    h = ns["silu_mul"](gate.astype(np.float32), up.astype(np.float32))
    assert h.dtype == np.float32 and h.shape == gate.shape
    np.savez_compressed(os.path.join(HERE, "silu_mul_ref.npz"), gate=gate, up=up, h=h)
    print("silu_mul", gate.shape, "->", h.shape)


def make_router(ref_root: str):
    path = os.path.join(ref_root, "scripts", "make-dsv2-layer-ref.py")
    tree = ast.parse(open(path).read())
    picked = []
    for node in ast.walk(tree):
        if isinstance(node, ast.If) and isinstance(node.test, ast.UnaryOp) and getattr(node.test.operand, "id", "") == "MOE":
            for st in node.orelse:                       # the MoE branch, in source order
                if isinstance(st, ast.Assign) and getattr(st.targets[0], "id", "") in ("probs", "ids", "topk_w"):
                    picked.append(st)
                elif isinstance(st, ast.AugAssign) and getattr(st.target, "id", "") == "probs":
                    picked.append(st)
                elif isinstance(st, ast.If) and "norm_topk_prob" in ast.dump(st.test):
                    picked.append(st)
    kinds = [type(n).__name__ + ":" + (getattr(getattr(n, "targets", [None])[0], "id", "") if isinstance(n, ast.Assign) else "") for n in picked]
    assert kinds == ["Assign:probs", "AugAssign:", "Assign:ids", "Assign:topk_w", "If:"], kinds
    code = compile(ast.Module(body=picked, type_ignores=[]), path, "exec")
    for name, (T, E, K, seed, norm) in {"e64_k6_raw": (24, 64, 6, 41, False), "e256_k8_norm": (24, 256, 8, 42, True),
                                        "e16_k4_norm": (12, 16, 4, 43, True)}.items():
        rng = np.random.default_rng(seed)
        logits = rng.standard_normal((T, E)).astype(np.float32)
        logits[1, 5] = logits[1, 3]                      # exact ties: the lower index must come first
        logits[2, E - 1] = logits[2, 0] = logits[2].max() + np.float32(0.5)
        logits[3, :] = np.float32(0.25)                  # all equal: experts 0..K-1 in order
        ids = np.zeros((T, K), dtype=np.uint32)
        w = np.zeros((T, K), dtype=np.float32)
        for t in range(T):
            ns = {"np": np, "router_logits": logits[t].copy(), "K": K,
                  "args": types.SimpleNamespace(routed_scaling=1.0, norm_topk_prob=norm)}
            exec(code, ns)
            ids[t], w[t] = ns["ids"], ns["topk_w"].astype(np.float32)
        np.savez_compressed(os.path.join(HERE, f"router_ref_{name}.npz"), logits=logits, ids=ids, weights=w,
                            norm=np.int32(norm))
        print("router", name, logits.shape, "->", ids.shape)


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py <path to a checkout of the reference project>")
    ref_root = sys.argv[1]
    make_silu_mul(ref_root)
    make_router(ref_root)
    make_kernel_ref(ref_root)
    dequant_from = load_dequant_from(ref_root)
    cases = {
        # name: (N, K, seed, scale sigma, extreme)
        "small": (16, 256, 11, 0.01, False),
        "ragged": (13, 1408, 12, 0.02, False),
        "wide": (40, 2048, 13, 0.01, False),
        # scales/biases spanning subnormal..large f16, so the f32 add and the f16 rounding both bite
        "extreme": (24, 512, 14, 1.0, True),
    }
    for name, (N, K, seed, sig, extreme) in cases.items():
        rng = np.random.default_rng(seed)
        W = rng.integers(0, 1 << 32, size=(N, K // 8), dtype=np.uint64).astype(np.uint32)
        s = np.abs(rng.standard_normal((N, K // 64), dtype=np.float32) * np.float32(sig))
        b = rng.standard_normal((N, K // 64), dtype=np.float32) * np.float32(0.05)
        if extreme:
            e = rng.integers(-22, 8, size=s.shape)
            s = s * np.exp2(e).astype(np.float32)
            b = b * np.exp2(rng.integers(-20, 10, size=b.shape)).astype(np.float32)
        s16, b16 = s.astype(np.float16), b.astype(np.float16)
        w = dequant_from(W, s16, b16, group=64, bits=4)          # f32 holding f16-representable values
        assert w.dtype == np.float32 and (w.astype(np.float16).astype(np.float32) == w).all()
        np.savez_compressed(os.path.join(HERE, f"dequant_from_{name}.npz"), W=W, scales=s16, biases=b16,
                            w16=w.astype(np.float16))
        print(name, W.shape, "->", w.shape)


if __name__ == "__main__":
    main()
