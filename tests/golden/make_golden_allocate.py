"""Golden vectors of the bit-width allocators, made with the reference's own functions.

    python tests/golden/make_golden_allocate.py --ref /path/to/jangq

writes tests/golden/allocate_ref.json: for several synthetic tensor lists (dense decoder, routed MoE with
and without a shared expert) the maps that jang_tools.allocate.allocate_bits_profile_compact and
allocate_bits_budget_compact return.  tests/test_allocate.py replays them without the reference.
"""
import argparse
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))


def tensor_list(L, E, shared):
    out = []
    for l in range(L):
        for p in "qkvo":
            out.append((f"model.layers.{l}.self_attn.{p}_proj.weight", 4096 * 4096 // 64))
        if E:
            out.append((f"model.layers.{l}.mlp.gate.weight", E * 4096 // 64))
            for part in ("gate_proj", "up_proj", "down_proj"):
                out.append((f"model.layers.{l}.mlp.switch_mlp.{part}.weight", E * 1024 * 4096 // 64))
                out.append((f"model.layers.{l}.mlp.experts.3.{part}.weight", 1024 * 4096 // 64))
            if shared:
                for part in ("gate_proj", "up_proj", "down_proj"):
                    out.append((f"model.layers.{l}.mlp.shared_expert.{part}.weight", 1024 * 4096 // 64))
        else:
            for part in ("gate_proj", "up_proj", "down_proj"):
                out.append((f"model.layers.{l}.mlp.{part}.weight", 11008 * 4096 // 64))
    out += [("model.embed_tokens.weight", 32000 * 4096 // 64), ("lm_head.weight", 32000 * 4096 // 64)]
    return out


CASES = ((6, 0, False), (8, 128, False), (8, 512, True), (3, 256, True), (1, 0, False))
TARGETS = (2.0, 2.5, 3.0, 3.7, 4.0, 4.5, 6.0, 8.0)
PROFILES = ("JANG_2S", "JANG_2M", "JANG_2L", "JANG_1L", "JANG_3M", "JANG_4M", "JANG_6M")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("JANGQ_REF", ""))
    a = ap.parse_args()
    sys.path.insert(0, os.path.join(a.ref, "jang-tools"))
    from jang_tools import allocate as ra
    out = []
    for L, E, sh in CASES:
        info = tensor_list(L, E, sh)
        rec = {"layers": L, "experts": E, "shared": sh, "budget": {}, "profile": {}}
        for tb in TARGETS:
            m = ra.allocate_bits_budget_compact(info, tb, E, sh)
            rec["budget"][str(tb)] = [m[n] for n, _ in info]
        for prof in PROFILES:
            m = ra.allocate_bits_profile_compact(info, prof, E, sh)
            rec["profile"][prof] = [m[n] for n, _ in info]
        out.append(rec)
    with open(os.path.join(HERE, "allocate_ref.json"), "w") as f:
        json.dump(out, f, separators=(",", ":"))


if __name__ == "__main__":
    main()
