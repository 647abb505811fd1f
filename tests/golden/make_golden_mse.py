"""Golden vectors for the clip-ratio-search quantizer, made by the reference itself.

Runs jang_tools.quantize.quantize_tensor(method="mse") (jang_tools/quantize.py:153-191,
:211-289) on a seeded tensor with a constant block, a zero block and an outlier, at
2/3/4 bits (the widths the search covers) and 6 bits (which falls through to RTN),
for 32-, 64- and 128-weight blocks.  The fixture records the numpy version: the reference
multiplies float32 minima by float64 clip ratios, so its arithmetic follows that
version's promotion rules (float64 under NumPy >= 2).

    python tests/golden/make_golden_mse.py --ref <checkout of the reference>
"""
import argparse
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", required=True, help="root of the reference checkout")
    args = ap.parse_args()
    sys.path.insert(0, os.path.join(args.ref, "jang-tools"))
    from jang_tools.quantize import quantize_tensor

    rng = np.random.default_rng(11)
    w = (rng.standard_normal((24, 512)) * 0.02).astype(np.float16).astype(np.float32)
    w[0, :128] = 0.25                                # constant block
    w[1, 128:256] = 0.0                              # zero block
    w[2, 7] = 0.9                                    # outlier the search clips
    w[3, 300] = -1.1
    out = {"w": w, "numpy_version": np.array(np.__version__)}
    for gs in (32, 64, 128):
        for bits in (2, 3, 4, 6):
            qt = quantize_tensor(w, np.full(w.size // gs, bits, np.uint8), block_size=gs, method="mse")
            key = f"g{gs}_b{bits}"
            out[key + "_packed"] = qt.qweight.view(np.uint32).reshape(24, 512 * bits // 32)
            out[key + "_scales"] = qt.scales.reshape(24, 512 // gs)
            out[key + "_biases"] = qt.biases.reshape(24, 512 // gs)
    np.savez_compressed(os.path.join(HERE, "mse_ref.npz"), **out)


if __name__ == "__main__":
    main()
