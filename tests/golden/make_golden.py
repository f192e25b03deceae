"""Generates tests/golden/dequant_from_*.npz from the reference's OWN numpy dequantiser.

Run once in a checkout that has the reference project mounted:

    python tests/golden/make_golden.py /path/to/reference

`scripts/make-dsv2-layer-ref.py` cannot be imported (it parses argv at module scope), so
the single function `dequant_from` (lines 102-116) is located with `ast`, compiled on
its own against numpy and executed on seeded inputs. Nothing of its source is stored:
only the inputs and the outputs it produced. The reference documents that function as
bit-identical to `mx.dequantize`, which makes these the only executed-reference vectors
available for this path (the reference's WGSL and JS need WebGPU / node).
"""
import ast
import os
import sys

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


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py <path to a checkout of the reference project>")
    ref_root = sys.argv[1]
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
