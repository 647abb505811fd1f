"""Golden JANGTQ codebooks, made with the reference's own compute_codebook.

    python tests/golden/make_golden_tq.py --ref /path/to/jangq

jang_tools/turboquant/codebook.py imports mlx at module level but compute_codebook itself is plain numpy, so
the file is loaded with an empty stand-in for `mlx.core`.  Writes tests/golden/tq_codebooks.json:
{"<dim>x<bits>": [centroids]} for the dimensions and widths the JANGTQ bundles use.
"""
import argparse
import importlib.util
import json
import os
import sys
import types

HERE = os.path.dirname(os.path.abspath(__file__))
CASES = [(d, b) for d in (128, 768, 1024, 2048, 3072, 4096, 6144) for b in (2, 3, 4)]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("JANGQ_REF", ""))
    a = ap.parse_args()
    mx, core = types.ModuleType("mlx"), types.ModuleType("mlx.core")
    core.array = object
    mx.core = core
    sys.modules.setdefault("mlx", mx)
    sys.modules.setdefault("mlx.core", core)
    path = os.path.join(a.ref, "jang-tools", "jang_tools", "turboquant", "codebook.py")
    spec = importlib.util.spec_from_file_location("ref_tq_codebook", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    out = {f"{d}x{b}": list(mod.compute_codebook(d, b)) for d, b in CASES}
    with open(os.path.join(HERE, "tq_codebooks.json"), "w") as f:
        json.dump(out, f)


if __name__ == "__main__":
    main()
