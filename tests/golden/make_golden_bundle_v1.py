#!/usr/bin/env python3
"""Generate tests/golden/bundle_v1/ (legacy layout) with the reference's own quantizer and v1 writer.

Run where the reference tree is mounted:

    python tests/golden/make_golden_bundle_v1.py --ref /path/to/reference

Quantizes three seeded tensors with jang_tools.quantize.quantize_tensor(method="rtn") (a 4-bit 2-D matrix, a
3-bit matrix, a 2-bit stacked expert tensor [E, out, in] named ...experts.gate_up_proj), writes them with
jang_tools.format.writer.write_jang_model (two shards) next to one float tensor, and stores the reference's
own dequantize_tensor outputs in bundle_v1_expected.npz.  The tests read only these files.
"""
from __future__ import annotations

import argparse
import os
import shutil
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("JANGQ_REF"), required="JANGQ_REF" not in os.environ,
                    help="root of the reference source tree (or set JANGQ_REF)")
    args = ap.parse_args()
    sys.path.insert(0, os.path.join(args.ref, "jang-tools"))
    from jang_tools.format.writer import write_jang_model
    from jang_tools.quantize import dequantize_tensor, quantize_tensor

    rng = np.random.default_rng(4242)
    specs = {
        "model.layers.0.self_attn.q_proj": ((24, 128), 4),
        "model.layers.0.mlp.down_proj": ((16, 192), 3),
        "model.layers.0.mlp.experts.gate_up_proj": ((3, 8, 64), 2),
    }
    qts, expected = {}, {}
    for name, (shape, bits) in specs.items():
        w = (rng.standard_normal(shape) * 0.02).astype(np.float32)
        n_blocks = w.size // 64
        qt = quantize_tensor(w, np.full(n_blocks, bits, dtype=np.uint8), 64, method="rtn")
        qts[name] = qt
        expected[name] = dequantize_tensor(qt, 64).astype(np.float32)
    out = os.path.join(HERE, "bundle_v1")
    shutil.rmtree(out, ignore_errors=True)
    write_jang_model(out, qts, {"model_type": "llama", "hidden_size": 128}, {"quantization": {"block_size": 64}},
                     passthrough_tensors={"model.norm.weight": rng.standard_normal(128).astype(np.float16)},
                     max_shard_bytes=2500)
    np.savez_compressed(os.path.join(HERE, "bundle_v1_expected.npz"), **expected)
    print("wrote", out, sorted(os.listdir(out)))


if __name__ == "__main__":
    main()
