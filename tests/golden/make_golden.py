#!/usr/bin/env python3
"""Generate the golden vectors in this folder from the reference itself.

Run where the reference tree is mounted:

    python tests/golden/make_golden.py --ref /path/to/reference

It imports the reference's own numpy code (jang-tools/jang_tools/affine.py,
pack.py, quantize.py) and reads the reference's MLX-generated fixture
(jang-runtime/Tests/JANGCoreMetalTests/fixtures/matmul_4bit_64x128.safetensors),
then writes small .npz files next to this script.  The tests only read the
.npz files, so they run where the reference is not mounted.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def adversarial_matrix(rng, rows, K, gs):
    """N(0,0.02) weights with hand-made groups that hit the quantizer's corners."""
    w = (rng.standard_normal((rows, K)) * 0.02).astype(np.float32)
    G = K // gs
    g = w.reshape(rows, G, gs)
    g[0, 0] = 0.0                                   # all-zero group
    g[1, 0] = 0.0371                                # constant positive
    g[2, 0] = -0.0371                               # constant negative
    g[3, 0] = np.abs(g[3, 0])                       # all positive
    g[4, 0] = -np.abs(g[4, 0])                      # all negative (max seeded with 0)
    g[5, 0, 7] = 3.5                                # single large outlier
    g[6, 0, 3] = -3.5
    g[7 % rows, G - 1] = np.linspace(-1.0, 1.0, gs) # exact grid -> .5 ties after scaling
    g[0, G - 1] = np.where(np.arange(gs) % 2 == 0, 0.0, -0.0)   # signed zeros
    g[1, G - 1] = 6e-8 * np.sign(rng.standard_normal(gs))       # f16 subnormals
    g[2, G - 1] = np.arange(gs) * 0.5                           # half-integer ladder
    g[3, G - 1] = np.concatenate([[0.0, 0.5, 1.5, 3.0], np.zeros(gs - 4)])
    return g.reshape(rows, K)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("JANGQ_REF"), required="JANGQ_REF" not in os.environ,
                    help="root of the reference source tree (or set JANGQ_REF)")
    args = ap.parse_args()
    sys.path.insert(0, os.path.join(args.ref, "jang-tools"))
    from jang_tools.affine import dequantize_affine_numpy, quantize_native_affine_numpy
    from jang_tools.pack import pack_bits, unpack_bits
    from jang_tools.quantize import quantize_tensor

    # ---- affine quantizer + dequantizer, every width x group size -------------
    out = {}
    meta = []
    rows, K = 8, 384
    for bits in (2, 3, 4, 5, 6, 8):
        for gs in (32, 64, 128):
            rng = np.random.default_rng(1000 * bits + gs)
            w16 = adversarial_matrix(rng, rows, K, gs).astype(np.float16)
            packed, s, b, _ = quantize_native_affine_numpy(w16, bits=bits, group_size=gs)
            deq = dequantize_affine_numpy(packed, s, b, bits=bits, group_size=gs)
            key = f"b{bits}_g{gs}"
            out[key + "_w"] = w16
            out[key + "_packed"] = packed
            out[key + "_scales"] = s
            out[key + "_biases"] = b
            out[key + "_deq"] = deq.astype(np.float32)
            meta.append({"key": key, "bits": bits, "group_size": gs, "rows": rows, "K": K})
    np.savez_compressed(os.path.join(HERE, "affine_ref.npz"), **out)

    # ---- a mid-size plain-gaussian case (config-1 distribution, reduced) -------
    rng = np.random.default_rng(0)
    w = (rng.standard_normal((64, 1024)) * 0.02).astype(np.float16)
    mid = {"w": w}
    for bits in (2, 3, 4, 6, 8):
        packed, s, b, _ = quantize_native_affine_numpy(w, bits=bits, group_size=64)
        mid[f"b{bits}_packed"], mid[f"b{bits}_scales"], mid[f"b{bits}_biases"] = packed, s, b
    np.savez_compressed(os.path.join(HERE, "affine_ref_gauss.npz"), **mid)

    # ---- RTN fallback (quantize.py:211-289), as convert.py:1571-1592 re-views it
    rtn = {}
    rng = np.random.default_rng(7)
    w = (rng.standard_normal((16, 256)) * 0.02).astype(np.float32)
    w[0, :64] = 0.25                                 # constant block
    rtn["w"] = w
    for bits in (2, 3, 4, 6, 8):
        n_blocks = w.size // 64
        qt = quantize_tensor(w, np.full(n_blocks, bits, np.uint8), block_size=64, method="rtn")
        rtn[f"b{bits}_packed"] = qt.qweight.view(np.uint32).reshape(16, 256 * bits // 32)
        rtn[f"b{bits}_scales"] = qt.scales.reshape(16, 4)
        rtn[f"b{bits}_biases"] = qt.biases.reshape(16, 4)
    np.savez_compressed(os.path.join(HERE, "rtn_ref.npz"), **rtn)

    # ---- pack/unpack streams -----------------------------------------------------
    pk = {}
    for bits in (1, 2, 3, 4, 5, 6, 8):
        rng = np.random.default_rng(42 + bits)
        v = rng.integers(0, 1 << bits, size=256, dtype=np.uint8)
        pk[f"b{bits}_values"] = v
        pk[f"b{bits}_bytes"] = pack_bits(v, bits)
        assert np.array_equal(unpack_bits(pk[f"b{bits}_bytes"], bits, 256), v)
    np.savez_compressed(os.path.join(HERE, "pack_ref.npz"), **pk)

    # ---- the reference's MLX-generated golden vector ----------------------------
    from safetensors.numpy import load_file
    fx_dir = os.path.join(args.ref, "jang-runtime", "Tests", "JANGCoreMetalTests", "fixtures")
    fx = load_file(os.path.join(fx_dir, "matmul_4bit_64x128.safetensors"))
    info = json.load(open(os.path.join(fx_dir, "fixture_info.json")))
    np.savez_compressed(
        os.path.join(HERE, "mlx_matmul_4bit_64x128.npz"),
        packed=fx["W.weight"], scales=fx["W.scales"], biases=fx["W.biases"], x=fx["x"],
        y_ref=fx["y_ref"], seed=np.uint64(info["seed"]), bits=np.int32(info["bits"]),
        group_size=np.int32(info["group_size"]))

    json.dump({"affine_ref": meta}, open(os.path.join(HERE, "golden_index.json"), "w"), indent=1)
    print("golden vectors written to", HERE)


if __name__ == "__main__":
    main()
