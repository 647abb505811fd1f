"""Host-side bit-width map rules (jangq_b200/allocate.py) on the BASELINE configurations."""
import pytest

from jangq_b200 import allocate as al


def test_profile_on_dense_llama_names():
    names = [f"model.layers.0.self_attn.{p}_proj.weight" for p in "qkvo"] + \
            [f"model.layers.0.mlp.{p}_proj.weight" for p in ("gate", "up", "down")] + \
            ["model.embed_tokens.weight", "lm_head.weight"]
    m = al.allocate_bits_profile(names, "JANG_2L")
    # the reference's JANG_2L: attention and the output head critical (8), embeddings important (6), MLP 2;
    # the dense decoder benchmark uses this map with the head taken down to 6 bits
    assert [m[n] for n in names] == [8, 8, 8, 8, 2, 2, 2, 6, 8]


def test_moe_rules_router_shared_and_asymmetry():
    names = ["model.layers.3.mlp.gate.weight", "model.layers.3.mlp.experts.7.gate_proj.weight",
             "model.layers.3.mlp.experts.7.up_proj.weight", "model.layers.3.mlp.experts.7.down_proj.weight",
             "model.layers.3.mlp.shared_expert.up_proj.weight", "model.layers.0.mlp.up_proj.weight"]
    m = al.allocate_bits_profile(names, "JANG_2M", num_experts=128)
    assert m[names[0]] == 8 and m[names[1]] == m[names[2]] == m[names[3]] == 2
    assert m[names[4]] == 8 and m[names[5]] == 8                       # always-active MLPs are critical
    m512 = al.allocate_bits_profile(names, "JANG_2M", num_experts=512)
    assert (m512[names[1]], m512[names[2]], m512[names[3]]) == (4, 2, 3)
    assert al.is_router(names[0]) and not al.is_router(names[1])
    with pytest.raises(ValueError):
        al.allocate_bits_profile(names, "JANG_9X")


def test_group_size_policy():
    assert al.model_group_size(128) == 64 and al.model_group_size(512) == 128
    assert al.tensor_group_size("layers.0.mlp.experts.0.up_proj", 4096, 128) == 128
    assert al.tensor_group_size("layers.0.mlp.gate", 4096, 128) == 64
    assert al.tensor_group_size("x.proj", 96, 128) == 32 and al.tensor_group_size("x.proj", 48, 64) is None


@pytest.mark.parametrize("bits,gs,K", [(2, 64, 4096), (3, 64, 4096), (4, 128, 4096), (6, 64, 2048), (8, 64, 4096), (8, 32, 64)])
def test_shape_inference_round_trip(bits, gs, K):
    assert al.infer_bits_and_group_size(K * bits // 32, K // gs, group_size=gs) == (bits, gs)


def test_shape_inference_tiebreak():
    # packed/sidecar width ratio 8 fits (8,32), (4,64) and (2,128)
    assert al.infer_bits_and_group_size(512, 64) == (8, 32)
    assert al.infer_bits_and_group_size(512, 64, prefer_high_bits=False) == (2, 128)
    assert al.infer_bits_and_group_size(512, 64, group_size=64) == (4, 64)
    with pytest.raises(ValueError):
        al.infer_bits_and_group_size(7, 3)


def test_allocators_replay_reference_maps():
    """Profile and budget allocators against maps the reference's own functions produced
    (tests/golden/allocate_ref.json, written by tests/golden/make_golden_allocate.py)."""
    import importlib.util
    import json
    import os
    gold = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
    spec = importlib.util.spec_from_file_location("make_golden_allocate", os.path.join(gold, "make_golden_allocate.py"))
    mk = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mk)
    cases = json.load(open(os.path.join(gold, "allocate_ref.json")))
    assert len(cases) == len(mk.CASES)
    for rec in cases:
        info = mk.tensor_list(rec["layers"], rec["experts"], rec["shared"])
        names = [n for n, _ in info]
        for tb, want in rec["budget"].items():
            m = al.allocate_bits_budget(info, float(tb), rec["experts"], rec["shared"])
            assert [m[n] for n in names] == want, (rec["layers"], rec["experts"], tb)
        for prof, want in rec["profile"].items():
            m = al.allocate_bits_profile(names, prof, rec["experts"], rec["shared"])
            assert [m[n] for n in names] == want, (rec["layers"], rec["experts"], prof)
