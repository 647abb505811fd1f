#!/usr/bin/env python3
"""Generate imatrix_ref.npz from the reference's activation-weighted affine fit.

Run where the reference tree is mounted:

    python tests/golden/make_golden_imatrix.py --ref /path/to/reference

Calls jang_tools.affine.quantize_imatrix_affine_numpy on seeded matrices (every width, group sizes 32/64/128,
with hand-made corner groups and importance vectors that include zeros and a wide dynamic range) and stores
inputs and outputs.  The tests read only the .npz file.
"""
from __future__ import annotations

import argparse
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def case(rng, rows, K, gs):
    w = (rng.standard_normal((rows, K)) * 0.02).astype(np.float32)
    g = w.reshape(rows, K // gs, gs)
    g[0, 0] = 0.0                                   # all-zero group: the fit degenerates, min/max grid is kept
    g[1, 0] = 0.0371                                # constant group
    g[2, 0, 5] = 2.5                                # one outlier
    g[3, 0] = np.linspace(-1.0, 1.0, gs)            # exact grid
    g[4 % rows, -1] = 1e-9 * rng.standard_normal(gs)   # below the scale floor
    imp = (rng.standard_normal(K) ** 2).astype(np.float32) * np.exp(rng.standard_normal(K) * 2).astype(np.float32)
    imp[::17] = 0.0                                 # ignored columns get the floor
    return w, imp


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("JANGQ_REF"), required="JANGQ_REF" not in os.environ,
                    help="root of the reference source tree (or set JANGQ_REF)")
    args = ap.parse_args()
    sys.path.insert(0, os.path.join(args.ref, "jang-tools"))
    from jang_tools.affine import quantize_imatrix_affine_numpy

    rng = np.random.default_rng(777)
    out = {}
    for gs in (32, 64, 128):
        for bits in (2, 3, 4, 5, 6, 8):
            w, imp = case(rng, 24, 512, gs)
            packed, s, b, err = quantize_imatrix_affine_numpy(w, imp, bits=bits, group_size=gs)
            key = f"b{bits}_g{gs}"
            out[key + "_w"], out[key + "_imp"] = w, imp
            out[key + "_packed"], out[key + "_scales"], out[key + "_biases"] = packed, s, b
            out[key + "_err"] = np.float64(err)
    w, imp = case(rng, 16, 256, 64)                 # a different iteration count
    packed, s, b, err = quantize_imatrix_affine_numpy(w, imp, bits=3, group_size=64, iterations=2)
    out["it2_w"], out["it2_imp"], out["it2_packed"], out["it2_scales"], out["it2_biases"] = w, imp, packed, s, b
    np.savez_compressed(os.path.join(HERE, "imatrix_ref.npz"), **out)
    print("wrote imatrix_ref.npz", len(out), "arrays")


if __name__ == "__main__":
    main()
