"""Builds oracle/_ref/: the one piece of the reference's own CPU code for this path that runs without its GPU stack.

TEST / BASELINE INFRASTRUCTURE ONLY (the product never touches it).

    python oracle/make_ref.py /path/to/reference

`scripts/make-dsv2-layer-ref.py` of the reference project holds `dequant_from(q, scales, biases, group, bits)`, a
numpy function its authors document as bit-identical to the vendor dequantiser. The file parses argv at module scope,
so it cannot be imported; the function definition is located with `ast`, compiled on its own and the resulting code
object is written with `marshal` to oracle/_ref/dequant_from.bin -- a compiled artefact of the reference's source,
built where that source lies, like a shared library would be. No source text is stored, and oracle/_ref/ is kept out
of the history. `load_dequant_from()` gives the function back (same interpreter version needed, as for any .pyc).
"""
from __future__ import annotations

import ast
import marshal
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
OUT = os.path.join(OUT_DIR, "dequant_from.bin")
SOURCE = os.path.join("scripts", "make-dsv2-layer-ref.py")


def build(ref_root: str) -> str:
    path = os.path.join(ref_root, SOURCE)
    tree = ast.parse(open(path).read())
    fn = next(n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name == "dequant_from")
    code = compile(ast.Module(body=[fn], type_ignores=[]), SOURCE, "exec")
    os.makedirs(OUT_DIR, exist_ok=True)
    with open(OUT, "wb") as fh:
        marshal.dump((sys.version_info[:2], f"{SOURCE}:{fn.lineno}-{fn.end_lineno}", code), fh)
    return OUT


def load_dequant_from():
    """The reference's dequant_from, or None when oracle/_ref/ has not been built (or another Python built it)."""
    if not os.path.exists(OUT):
        return None
    import numpy as np
    with open(OUT, "rb") as fh:
        try:
            ver, where, code = marshal.load(fh)
        except (ValueError, EOFError, TypeError):
            return None
    if tuple(ver) != tuple(sys.version_info[:2]):
        return None
    ns = {"np": np}
    exec(code, ns)
    fn = ns["dequant_from"]
    fn.reference_location = where
    return fn


if __name__ == "__main__":
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_ref.py <path to a checkout of the reference project>")
    print(build(sys.argv[1]))
