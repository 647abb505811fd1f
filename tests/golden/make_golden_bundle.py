#!/usr/bin/env python3
"""Generate tests/golden/bundle_v2/ with the reference's own writer and quantizer.

Run where the reference tree is mounted:

    python tests/golden/make_golden_bundle.py --ref /path/to/reference

It quantizes four small seeded matrices with jang_tools.affine.quantize_native_affine_numpy (8-bit q_proj,
2-bit gate_proj, 3-bit stacked experts, 6-bit lm_head with group size 128), adds one float tensor, and writes
them with jang_tools.format.writer.write_jang_v2_model (two shards).  The tests read only the written
directory, so they run where the reference is not mounted.
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
    from jang_tools.affine import quantize_native_affine_numpy
    from jang_tools.format.writer import write_jang_v2_model

    rng = np.random.default_rng(20240607)
    specs = {
        "model.layers.0.self_attn.q_proj": ((32, 256), 8, 64),
        "model.layers.0.mlp.gate_proj": ((48, 128), 2, 64),
        "model.layers.0.mlp.switch_mlp.up_proj": ((4, 16, 128), 3, 64),
        "lm_head": ((40, 256), 6, 128),
    }
    tensors, manifest = {}, {}
    for name, (shape, bits, gs) in specs.items():
        w = (rng.standard_normal(shape) * 0.02).astype(np.float16)
        flat = w.reshape(-1, shape[-1])
        q, s, b, _ = quantize_native_affine_numpy(flat, bits=bits, group_size=gs)
        q = q.reshape(shape[:-1] + (q.shape[-1],))
        s = s.reshape(shape[:-1] + (s.shape[-1],))
        b = b.reshape(shape[:-1] + (b.shape[-1],))
        tensors[name + ".weight"], tensors[name + ".scales"], tensors[name + ".biases"] = q, s, b
        manifest[name] = {"source_tensor": name + ".weight", "bits": bits, "group_size": gs,
                          "weight_key": name + ".weight", "scales_key": name + ".scales", "biases_key": name + ".biases",
                          "weight_shape": list(q.shape), "scales_shape": list(s.shape), "biases_shape": list(b.shape)}
    tensors["model.norm.weight"] = rng.standard_normal(256).astype(np.float16)
    out = os.path.join(HERE, "bundle_v2")
    shutil.rmtree(out, ignore_errors=True)
    model_config = {"model_type": "llama", "hidden_size": 256, "num_hidden_layers": 1, "vocab_size": 40}
    jang_config = {"quantization": {"bit_widths_used": [2, 3, 6, 8], "block_size": 64,
                                    "quantization_backend": "quantize_native_affine_numpy",
                                    "tensor_quantization_manifest_schema": 1,
                                    "tensor_quantization_manifest_count": len(manifest),
                                    "tensor_quantization_manifest": manifest}}
    write_jang_v2_model(out, tensors, model_config, jang_config, max_shard_bytes=12000)
    print("wrote", out, sorted(os.listdir(out)))


if __name__ == "__main__":
    main()
