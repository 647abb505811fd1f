"""JANG v2 bundle I/O against a bundle written by the reference's own writer (tests/golden/bundle_v2, made by
tests/golden/make_golden_bundle.py with jang_tools.format.writer.write_jang_v2_model)."""
import json
import os
import shutil

import numpy as np
import pytest

from jangq_b200 import bundle as B
from oracle import jang_oracle as jo

HERE = os.path.dirname(os.path.abspath(__file__))
GOLD = os.path.join(HERE, "golden", "bundle_v2")
SPECS = {
    "model.layers.0.self_attn.q_proj": ((32, 256), 8, 64),
    "model.layers.0.mlp.gate_proj": ((48, 128), 2, 64),
    "model.layers.0.mlp.switch_mlp.up_proj": ((4, 16, 128), 3, 64),
    "lm_head": ((40, 256), 6, 128),
}


def test_detection():
    assert B.is_jang_model(GOLD) and B.is_v2_model(GOLD)
    assert not B.is_jang_model(HERE)
    with pytest.raises(B.BundleError):
        B.open_bundle(HERE)


def test_read_matches_manifest_and_oracle_quantizer():
    """Every module's width and group size follow from the shapes and equal the writer's manifest; the stored
    codes and sidecars are what the oracle's quantizer makes of the same seeded weights (f16 source)."""
    b = B.open_bundle(GOLD)
    assert b.quantized_modules() == sorted(SPECS)
    assert b.jang_config["format"] == "jang" and b.jang_config["format_version"] == "2.0"
    rng = np.random.default_rng(20240607)
    for name, (shape, bits, gs) in SPECS.items():           # same order as the generating script
        spec = b.quant_spec(name)
        assert (spec.bits, spec.group_size) == (bits, gs), name
        w = (rng.standard_normal(shape) * 0.02).astype(np.float16)
        q, s, bi = b.tensor(name + ".weight"), b.tensor(name + ".scales"), b.tensor(name + ".biases")
        assert q.dtype == np.uint32 and s.dtype == np.float16 and bi.dtype == np.float16
        assert q.shape == shape[:-1] + (shape[-1] * bits // 32,) and s.shape == shape[:-1] + (shape[-1] // gs,)
        pk, so, bo = jo.quantize_affine(w.reshape(-1, shape[-1]).astype(np.float32), bits, gs, src_dtype="f16")
        assert np.array_equal(pk, q.reshape(pk.shape))
        assert np.array_equal(so.astype(np.float16), s.reshape(so.shape))
        assert np.array_equal(bo.astype(np.float16), bi.reshape(bo.shape))
    assert b.tensor("model.norm.weight").shape == (256,)
    with pytest.raises(KeyError):
        b.tensor("nope")
    b.close()


def test_writer_reproduces_the_reference_bundle(tmp_path):
    """Writing the golden bundle's tensors back gives the same files: configs and index equal as JSON, shard
    files byte for byte."""
    b = B.open_bundle(GOLD)
    order = list(json.load(open(os.path.join(GOLD, B.INDEX_FILENAME)))["weight_map"])
    tensors = {n: b.tensor(n) for n in order}
    model_config = {k: v for k, v in b.config.items() if k != "quantization"}
    jang_config = {k: v for k, v in b.jang_config.items() if k not in ("format", "format_version")}
    out = tmp_path / "copy"
    B.write_bundle(out, tensors, model_config, jang_config, max_shard_bytes=12000)
    for f in ("config.json", "jang_config.json", B.INDEX_FILENAME):
        assert json.load(open(out / f)) == json.load(open(os.path.join(GOLD, f))), f
    shards = sorted(p for p in os.listdir(GOLD) if p.endswith(".safetensors"))
    assert shards == sorted(p.name for p in out.glob("*.safetensors"))
    for s in shards:
        assert (out / s).read_bytes() == open(os.path.join(GOLD, s), "rb").read(), s
    b.close()


def test_open_without_index_and_missing_shard(tmp_path):
    d = tmp_path / "b"
    shutil.copytree(GOLD, d)
    os.remove(d / B.INDEX_FILENAME)
    b = B.open_bundle(d)
    assert b.quantized_modules() == sorted(SPECS)
    b.close()
    d2 = tmp_path / "c"
    shutil.copytree(GOLD, d2)
    os.remove(d2 / "model-00002-of-00003.safetensors")
    with pytest.raises(B.BundleError):
        B.open_bundle(d2)


def test_v1_and_corrupt_configs(tmp_path):
    d = tmp_path / "v1"
    d.mkdir()
    (d / "jang_config.json").write_text(json.dumps({"format": "jang", "format_version": "1.1"}))
    (d / "model.jang.safetensors").write_bytes(b"")
    assert B.is_jang_model(d) and not B.is_v2_model(d)
    with pytest.raises(B.BundleError):
        B.open_bundle(d)
    e = tmp_path / "bad"
    e.mkdir()
    (e / "jang_config.json").write_text("{not json")
    assert B.is_jang_model(e) and not B.is_v2_model(e)


def test_shape_inference_order():
    # 4-bit/gs64 over K=256 and 2-bit/gs128 over K=512 give the same shapes: the hint decides, routers prefer 64
    assert B.infer_bits_group_size(32, 4, 64) == (4, 64)
    assert B.infer_bits_group_size(32, 4, 128) == (2, 128)
    assert B.infer_bits_group_size(32, 4, 128, is_router=True) == (4, 64)
    assert B.infer_bits_group_size(32, 4, 64, in_features=512) == (2, 128)     # the logical width settles it
    assert B.infer_bits_group_size(16, 4, 128) == (2, 64)                      # the hint does not fit: next candidate
    assert B.infer_bits_group_size(48, 4, 64) == (6, 64)
    assert B.infer_bits_group_size(40, 4, 64) == (5, 64)
    with pytest.raises(B.BundleError):
        B.infer_bits_group_size(7, 4, 64)


def test_stale_config_entry_loses_to_shapes(tmp_path):
    d = tmp_path / "stale"
    shutil.copytree(GOLD, d)
    cfg = json.load(open(d / "config.json"))
    cfg["quantization"]["lm_head"]["bits"] = 2
    (d / "config.json").write_text(json.dumps(cfg))
    b = B.open_bundle(d)
    assert (b.quant_spec("lm_head").bits, b.quant_spec("lm_head").group_size) == (6, 128)
    b.close()


def test_expand_1bit_known_answer():
    x = np.array([[0x00000001, 0x80000000, 0xFFFFFFFF, 0x00010002]], dtype=np.uint32)
    y = B.expand_1bit_to_2bit(x)
    assert y.shape == (1, 8)
    assert y.tolist() == [[1, 0, 0, 0x40000000, 0x55555555, 0x55555555, 4, 1]]
    # values survive: the 2-bit codes of y are the bits of x
    ref = ((x[..., None] >> np.arange(32, dtype=np.uint32)) & 1).reshape(1, -1)
    assert np.array_equal(jo.unpack_rows(y, 2, 128).reshape(1, -1), ref)


GOLD_V1 = os.path.join(HERE, "golden", "bundle_v1")


def test_v1_repack_dequantizes_to_the_reference_values(tmp_path):
    """A v1 bundle written by the reference's legacy writer (tests/golden/bundle_v1), repacked to v2 and
    dequantized by the oracle, gives the reference's own dequantize_tensor values bit for bit; the stacked
    gate_up_proj experts are split into switch_mlp.gate_proj / up_proj."""
    assert B.is_jang_model(GOLD_V1) and not B.is_v2_model(GOLD_V1)
    exp = np.load(os.path.join(HERE, "golden", "bundle_v1_expected.npz"))
    t = B.read_v1_tensors(GOLD_V1)
    assert t["model.norm.weight"].dtype == np.float16 and t["model.norm.weight"].shape == (128,)
    for name, bits in (("model.layers.0.self_attn.q_proj", 4), ("model.layers.0.mlp.down_proj", 3)):
        wq, s, b = t[name + ".weight"], t[name + ".scales"], t[name + ".biases"]
        assert wq.dtype == np.uint32 and s.dtype == np.float16
        assert B.infer_bits_group_size(wq.shape[-1], s.shape[-1], 64) == (bits, 64)
        deq = jo.dequantize_affine(wq, s.astype(np.float32), b.astype(np.float32), bits, 64)
        assert np.array_equal(deq, exp[name])
    full = exp["model.layers.0.mlp.experts.gate_up_proj"]                # [3, 8, 64]
    for nm, sl in (("gate_proj", slice(0, 4)), ("up_proj", slice(4, 8))):
        base = "model.layers.0.mlp.switch_mlp." + nm
        wq, s, b = t[base + ".weight"], t[base + ".scales"], t[base + ".biases"]
        assert wq.shape == (3, 4, 4)
        deq = jo.dequantize_affine(wq.reshape(12, 4), s.astype(np.float32).reshape(12, 1), b.astype(np.float32).reshape(12, 1), 2, 64)
        assert np.array_equal(deq.reshape(3, 4, 64), full[:, sl, :])
    out = tmp_path / "v2"
    B.repack_v1_to_v2(GOLD_V1, out)
    b2 = B.open_bundle(out)
    assert B.is_v2_model(out) and b2.jang_config["format_version"] == "2.0"
    assert b2.quant_spec("model.layers.0.mlp.down_proj").bits == 3
    assert b2.config["quantization"]["model.layers.0.mlp.switch_mlp.up_proj"] == {"group_size": 64, "bits": 2, "mode": "affine"}
    assert np.array_equal(b2.tensor("model.layers.0.self_attn.q_proj.weight"), t["model.layers.0.self_attn.q_proj.weight"])
    b2.close()


def test_load_jang_model_builds_the_module_tree():
    """load_jang_model (jang_tools/loader.py:1078 call shape) on the bundles the reference's writers made: a
    module tree under the bundle's names, widths from the shapes, v1 repacked on the fly; built on the CPU
    here (no kernel runs), the GPU tests call the modules."""
    import torch
    from jangq_b200 import JANGLinear, JANGSwitchLinear, load_jang_model
    here = os.path.dirname(os.path.abspath(__file__))
    model, tok = load_jang_model(os.path.join(here, "golden", "bundle_v2"), device="cpu")
    assert tok is None and model.jang_config.get("format")
    q = model.get_submodule("model.layers.0.self_attn.q_proj")
    assert isinstance(q, JANGLinear) and q.weight.dtype == torch.int32
    sw = model.get_submodule("model.layers.0.mlp.switch_mlp.up_proj")
    assert isinstance(sw, JANGSwitchLinear) and (sw.n_experts, sw.out_features, sw.in_features, sw.bits) == (4, 16, 128, 3)
    b = B.open_bundle(os.path.join(here, "golden", "bundle_v2"))
    assert sorted(model.state_dict().keys()) == sorted(b.names())
    b.close()
    m1, _ = load_jang_model(os.path.join(here, "golden", "bundle_v1"), device="cpu")
    assert isinstance(m1.get_submodule("model.layers.0.mlp.switch_mlp.gate_proj"), JANGSwitchLinear)
    with pytest.raises(FileNotFoundError):
        load_jang_model(here)
