"""JANG bundle directories: read and write v2, repack v1 to v2, and turn a bundle into the torch modules of this
package.

A v2 bundle (jang_tools/format/writer.py:30-193) is a directory with
  config.json                    the model config plus a "quantization" block: default group_size/bits/mode
                                 and one {"group_size", "bits", "mode"[, "storage_bits"]} entry per module whose
                                 width differs (what mlx-lm's quantization predicate reads);
  jang_config.json               {"format": "jang", "format_version": "2.0", "quantization": {"bit_widths_used",
                                 "block_size", "tensor_quantization_manifest": {module: {bits, group_size, ...}}}};
  model-XXXXX-of-YYYYY.safetensors   shards with metadata {"format": "mlx"}; a quantized module `m` is stored as
                                 m.weight uint32 [.., N, K*bits/32], m.scales / m.biases float16 [.., N, K/gs];
                                 a module's tensors never straddle shards;
  model.safetensors.index.json   {"metadata": {"format", "format_version", "total_size"}, "weight_map"}.
The bit width of a module is not stored with the tensor: it follows from the shapes,
bits = w_cols * 32 / (s_cols * group_size) (jang_tools/loader.py:1922-1975), with the config's entry as the hint
for the group size.  One-bit storage (jang_tools/affine.py:402-416) expands to two-bit codes on load.

Host-side only: numpy + safetensors, no GPU needed until `load_modules` moves tensors to a device.
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from pathlib import Path

import numpy as np

FORMAT_NAME = "jang"
FORMAT_VERSION = "2.0"
CONFIG_FILENAMES = ("jang_config.json", "jjqf_config.json", "jang_cfg.json", "mxq_config.json")   # loader.py:34
INDEX_FILENAME = "model.safetensors.index.json"
ALLOWED_BITS = (2, 3, 4, 5, 6, 8)
ALLOWED_STORAGE_BITS = (1,) + ALLOWED_BITS


class BundleError(ValueError):
    pass


def find_config_path(path) -> Path | None:
    """The bundle's JANG config file, or None (jang_tools/loader.py:116-121)."""
    p = Path(path)
    for name in CONFIG_FILENAMES:
        if (p / name).exists():
            return p / name
    return None


def is_jang_model(path) -> bool:
    """jang_tools/loader.py:149-151."""
    return find_config_path(path) is not None


def is_v2_model(path) -> bool:
    """v2 = MLX-native safetensors (jang_tools/loader.py:154-181): an index file, or standard shards without
    *.jang.safetensors ones, or format_version >= 2 in the JANG config.  A corrupt config reads as "not v2"."""
    p = Path(path)
    if (p / INDEX_FILENAME).exists():
        return True
    if any(p.glob("model-*.safetensors")) and not any(p.glob("*.jang.safetensors")):
        return True
    cfg = find_config_path(p)
    if cfg is not None:
        try:
            version = str(json.loads(cfg.read_text()).get("format_version", "1.0"))
            return int(version.split(".")[0]) >= 2
        except (OSError, ValueError, AttributeError):
            return False
    return False


def infer_bits_group_size(w_cols: int, s_cols: int, group_size_hint: int = 64, in_features: int | None = None,
                          is_router: bool = False) -> tuple[int, int]:
    """(bits, group_size) of a quantized tensor from its last dimensions: w_cols*32/bits == s_cols*gs.

    Several pairs can satisfy the equation; the candidates are tried in the reference's order
    (jang_tools/loader.py:1922-1975): with a known logical input width the group sizes that reproduce it come
    first; router/gate tensors prefer 64; everything else prefers the hint (the module's configured group
    size), then 64, 128.  Raises BundleError when no allowed width fits."""
    hint = int(group_size_hint)
    if in_features:
        cands = [g for g in (hint, 64, 128, 32) if in_features % g == 0 and s_cols * g == in_features]
        cands = list(dict.fromkeys(cands))
        cands += [g for g in (hint, 64, 128, 32) if g not in cands]
    elif is_router:
        cands = list(dict.fromkeys([64, hint, 128]))
    else:
        cands = list(dict.fromkeys([hint, 64, 128]))
    for gs in cands:
        in_dim = s_cols * gs
        if in_dim <= 0 or (w_cols * 32) % in_dim != 0:
            continue
        bits = (w_cols * 32) // in_dim
        if bits in ALLOWED_BITS and (not in_features or in_dim == in_features):
            return bits, gs
    in_dim = s_cols * hint
    if in_dim > 0 and (w_cols * 32) // in_dim in ALLOWED_BITS and (w_cols * 32) % in_dim == 0:
        return (w_cols * 32) // in_dim, hint
    raise BundleError(f"no (bits, group_size) fits weight columns {w_cols} and scale columns {s_cols}")


def expand_1bit_to_2bit(packed: np.ndarray) -> np.ndarray:
    """uint32-packed 1-bit codes -> uint32-packed 2-bit codes with the same values
    (jang_tools/affine.py:402-416): bit i of a word becomes the 2-bit field i of the pair of output words."""
    src = np.ascontiguousarray(packed, dtype=np.uint32)
    bits = ((src[..., None] >> np.arange(32, dtype=np.uint32)) & np.uint32(1)).astype(np.uint32)   # [.., W, 32]
    shifts = (2 * np.arange(16, dtype=np.uint32))
    low = (bits[..., :16] << shifts).sum(axis=-1, dtype=np.uint64).astype(np.uint32)
    high = (bits[..., 16:] << shifts).sum(axis=-1, dtype=np.uint64).astype(np.uint32)
    out = np.empty(src.shape[:-1] + (src.shape[-1] * 2,), dtype=np.uint32)
    out[..., 0::2] = low
    out[..., 1::2] = high
    return out


@dataclass
class QuantSpec:
    bits: int
    group_size: int
    storage_bits: int | None = None


@dataclass
class Bundle:
    """An opened bundle: configs, the tensor -> shard map, and lazy tensor reads."""
    path: Path
    config: dict
    jang_config: dict
    weight_map: dict[str, str]
    _handles: dict = field(default_factory=dict, repr=False)

    def names(self) -> list[str]:
        return list(self.weight_map)

    def tensor(self, name: str) -> np.ndarray:
        from safetensors import safe_open
        shard = self.weight_map.get(name)
        if shard is None:
            raise KeyError(name)
        h = self._handles.get(shard)
        if h is None:
            h = self._handles[shard] = safe_open(str(self.path / shard), framework="np")
        return h.get_tensor(name)

    def quantized_modules(self) -> list[str]:
        """Module paths that have .weight (uint32), .scales and .biases."""
        names = set(self.weight_map)
        return sorted(n[:-len(".scales")] for n in names
                      if n.endswith(".scales") and n[:-len(".scales")] + ".weight" in names
                      and n[:-len(".scales")] + ".biases" in names)

    def default_group_size(self) -> int:
        q = self.config.get("quantization") or {}
        return int(q.get("group_size", (self.jang_config.get("quantization") or {}).get("block_size", 64)))

    def quant_spec(self, module: str, w_shape=None, s_shape=None) -> QuantSpec:
        """The module's (bits, group_size): shapes are authoritative (a config entry can be stale after a
        loader-side repack), the config's per-module entry or default only supplies the group-size hint."""
        q = self.config.get("quantization") or {}
        entry = q.get(module) if isinstance(q.get(module), dict) else {}
        manifest = (self.jang_config.get("quantization") or {}).get("tensor_quantization_manifest") or {}
        m = manifest.get(module) if isinstance(manifest.get(module), dict) else {}
        hint = int(entry.get("group_size", m.get("group_size", self.default_group_size())))
        storage = entry.get("storage_bits", m.get("storage_bits"))
        if w_shape is None:
            w_shape = self.tensor(module + ".weight").shape
        if s_shape is None:
            s_shape = self.tensor(module + ".scales").shape
        w_cols = int(w_shape[-1]) * (2 if storage == 1 else 1)
        name_lower = module.lower()
        is_router = ".gate." in name_lower or name_lower.endswith(".gate") or "shared_expert_gate" in name_lower
        bits, gs = infer_bits_group_size(w_cols, int(s_shape[-1]), hint, is_router=is_router)
        return QuantSpec(bits, gs, int(storage) if isinstance(storage, int) else None)

    def close(self):
        self._handles.clear()


def _read_json(path: Path, what: str) -> dict:
    try:
        data = json.loads(path.read_text())
    except (OSError, ValueError) as e:
        raise BundleError(f"cannot read {what} {path}: {e}") from e
    if not isinstance(data, dict):
        raise BundleError(f"{what} {path} is not a JSON object")
    return data


def open_bundle(path) -> Bundle:
    """Open a v2 bundle directory.  Without an index file the shards are listed and scanned."""
    from safetensors import safe_open
    p = Path(path)
    cfg_path = find_config_path(p)
    if cfg_path is None:
        raise BundleError(f"{p} is not a JANG bundle (none of {', '.join(CONFIG_FILENAMES)})")
    if not is_v2_model(p):
        raise BundleError(f"{p} is a v1 bundle (*.jang.safetensors); repack it with repack_v1_to_v2 first")
    jang_config = _read_json(cfg_path, "JANG config")
    config = _read_json(p / "config.json", "model config") if (p / "config.json").exists() else {}
    if (p / INDEX_FILENAME).exists():
        weight_map = _read_json(p / INDEX_FILENAME, "index").get("weight_map")
        if not isinstance(weight_map, dict):
            raise BundleError(f"{p / INDEX_FILENAME} has no weight_map")
        missing = sorted({s for s in weight_map.values() if not (p / s).exists()})
        if missing:
            raise BundleError(f"shards named by the index are missing: {missing[:3]}")
    else:
        weight_map = {}
        for shard in sorted(p.glob("model*.safetensors")):
            with safe_open(str(shard), framework="np") as f:
                for k in f.keys():
                    weight_map[k] = shard.name
    return Bundle(p, config, jang_config, dict(weight_map))


def _shard(tensors: dict[str, np.ndarray], max_bytes: int) -> list[list[str]]:
    """Greedy shards in insertion order; the tensors of one module (same name up to the last dot) stay
    together (jang_tools/format/writer.py:271-303)."""
    groups: dict[str, list[str]] = {}
    for name in tensors:
        groups.setdefault(name.rsplit(".", 1)[0], []).append(name)
    shards, cur, size = [], [], 0
    for names in groups.values():
        g = sum(tensors[n].nbytes for n in names)
        if cur and size + g > max_bytes:
            shards.append(cur)
            cur, size = [], 0
        cur.extend(names)
        size += g
    if cur:
        shards.append(cur)
    return shards


def _write_json(path: Path, obj: dict) -> None:
    path.write_text(json.dumps(obj, indent=2) + "\n")


def write_bundle(path, tensors: dict[str, np.ndarray], model_config: dict, jang_config: dict,
                 max_shard_bytes: int = 5 * 1024 ** 3) -> None:
    """Write a v2 bundle the reference's loader reads (jang_tools/format/writer.py:30-193): config.json with the
    quantization block (default = the narrowest width used, one entry per manifest module), jang_config.json
    stamped format/format_version, shards with metadata {"format": "mlx"}, the index with total_size = bytes
    of the shard files.  `tensors` holds MLX-layout arrays: m.weight uint32, m.scales / m.biases float16."""
    from safetensors.numpy import save_file
    p = Path(path)
    p.mkdir(parents=True, exist_ok=True)
    jq = jang_config.get("quantization") or {}
    widths = jq.get("bit_widths_used") or [4]
    block = int(jq.get("block_size", 64))
    quantization = {"group_size": block, "bits": int(min(widths)), "mode": "affine"}
    manifest = jq.get("tensor_quantization_manifest")
    if isinstance(manifest, dict):
        for module, spec in manifest.items():
            if not isinstance(module, str) or not isinstance(spec, dict):
                continue
            bits, gs = spec.get("bits"), spec.get("group_size")
            if isinstance(bits, int) and isinstance(gs, int):
                entry = {"group_size": gs, "bits": bits, "mode": "affine"}
                storage = spec.get("storage_bits")
                if isinstance(storage, int):
                    if isinstance(storage, bool) or storage not in ALLOWED_STORAGE_BITS:
                        raise BundleError(f"invalid storage bit width {storage} for {module}")
                    entry["storage_bits"] = storage
                quantization[module] = entry
    cfg_out = dict(model_config)
    cfg_out["quantization"] = quantization
    _write_json(p / "config.json", cfg_out)
    jc = dict(jang_config)
    jc.setdefault("format", FORMAT_NAME)
    jc["format_version"] = FORMAT_VERSION
    _write_json(p / CONFIG_FILENAMES[0], jc)
    for name, arr in tensors.items():
        if name.endswith(".weight") and name[:-len(".weight")] + ".scales" in tensors and arr.dtype != np.uint32:
            raise BundleError(f"{name}: packed codes must be uint32, got {arr.dtype}")
    shards = _shard(tensors, max_shard_bytes)
    weight_map = {}
    for i, names in enumerate(shards):
        shard_name = f"model-{i + 1:05d}-of-{len(shards):05d}.safetensors"
        save_file({n: np.ascontiguousarray(tensors[n]) for n in names}, str(p / shard_name), metadata={"format": "mlx"})
        for n in names:
            weight_map[n] = shard_name
    total = sum((p / s).stat().st_size for s in set(weight_map.values()))
    _write_json(p / INDEX_FILENAME, {"metadata": {"format": FORMAT_NAME, "format_version": FORMAT_VERSION,
                                                  "total_size": total}, "weight_map": weight_map})


def load_modules(path, device="cuda", sidecar_dtype=None, only=None) -> dict:
    """The bundle's quantized modules as this package's torch modules: {module path: JANGLinear} for 2-D
    tensors, {module path: ExpertBank} for stacked experts [E, N, Kp].  Sidecars keep the stored float16
    unless `sidecar_dtype` asks for a cast (the reference's runtime modules use bfloat16,
    jangrt/linear.py:35-38).  One-bit storage is expanded to two-bit codes.  `only` filters module paths."""
    import torch

    from . import moe
    from .linear import JANGLinear
    b = open_bundle(path)
    out = {}
    for m in b.quantized_modules():
        if only is not None and not only(m):
            continue
        w = b.tensor(m + ".weight")
        s = b.tensor(m + ".scales")
        bi = b.tensor(m + ".biases")
        if w.dtype != np.uint32:
            continue                                      # a float module that happens to have scales
        spec = b.quant_spec(m, w.shape, s.shape)
        if spec.storage_bits == 1:
            w = expand_1bit_to_2bit(w)
        dt = sidecar_dtype or torch.float16
        wt = torch.from_numpy(w.view(np.int32)).to(device)
        st = torch.from_numpy(np.ascontiguousarray(s)).to(device).to(dt)
        bt = torch.from_numpy(np.ascontiguousarray(bi)).to(device).to(dt)
        if w.ndim == 2:
            n, k = w.shape[0], s.shape[-1] * spec.group_size
            lin = JANGLinear(k, n, spec.bits, spec.group_size, bias=(m + ".bias") in b.weight_map, device=device, dtype=dt)
            lin.weight, lin.scales, lin.biases = wt, st, bt
            if lin.bias is not None:
                lin.bias = torch.from_numpy(np.ascontiguousarray(b.tensor(m + ".bias"))).to(device).to(dt)
            out[m] = lin
        elif w.ndim == 3:
            out[m] = moe.ExpertBank(wt, st, bt, spec.bits, spec.group_size)
        else:
            raise BundleError(f"{m}.weight has {w.ndim} dimensions")
    b.close()
    return out


V1_INDEX_NAMES = ("model.jang.index.json", "model.jjqf.index.json", "model.mxq.index.json")
V1_SHARD_GLOBS = ("*.jang.safetensors", "*.jjqf.safetensors", "*.mxq.safetensors")
V1_SUFFIXES = (".qweight", ".scales", ".zeros", ".biases", ".bit_map", ".block_offsets", ".shape", ".bits")


def read_v1_tensors(path) -> dict[str, np.ndarray]:
    """The tensors of a v1 bundle repacked into the v2 (MLX) layout, as jang_tools/loader.py:1326-1655 does on
    load: for every quantized base `b` (b.qweight uint8 stream, b.scales, b.biases or b.zeros, b.bits or
    b.bit_map, b.shape)
      codes   = the byte stream padded to whole words, viewed uint32, cut to out*ceil(in*bits/32) words and
                shaped [out, words] (stacked experts: [E, out, words]);
      biases  = stored biases, or -scales*zeros for the oldest files, zeros if neither exists;
      scales/biases are padded with 1.0 / 0.0 to out*ceil(in/block) groups and shaped like the codes;
      a missing width means 4 bits; a missing shape means [n_blocks, block_size];
      names   = b.weight / b.scales / b.biases; a stacked `...experts.gate_up_proj` is split along `out` into
                `...switch_mlp.gate_proj` and `...switch_mlp.up_proj` (loader.py:1591-1606).
    Sidecars come back as float16 when they were stored so (the repack is then lossless), float32 when biases
    had to be computed from zero points.  Other tensors pass through unchanged."""
    from safetensors import safe_open
    p = Path(path)
    cfg_path = find_config_path(p)
    if cfg_path is None:
        raise BundleError(f"{p} is not a JANG bundle")
    block = int((_read_json(cfg_path, "JANG config").get("quantization") or {}).get("block_size", 64))
    shards = []
    for name in V1_INDEX_NAMES:
        if (p / name).exists():
            wm = _read_json(p / name, "index").get("weight_map") or {}
            shards = [p / s for s in sorted(set(wm.values()))]
            break
    if not shards:
        for pat in V1_SHARD_GLOBS:
            shards.extend(sorted(p.glob(pat)))
    if not shards:
        raise BundleError(f"no v1 weight files in {p}")
    raw = {}
    for s in shards:
        with safe_open(str(s), framework="np") as f:
            for k in f.keys():
                raw[k] = f.get_tensor(k)
    bases = sorted({k[:-len(suf)] for k in raw for suf in V1_SUFFIXES if k.endswith(suf)})
    quant_keys = {b + suf for b in bases for suf in V1_SUFFIXES}
    out: dict[str, np.ndarray] = {}
    for b in bases:
        if b + ".qweight" not in raw or b + ".scales" not in raw:
            raise BundleError(f"{b}: qweight or scales missing")
        scales = raw[b + ".scales"]
        keep_f16 = scales.dtype == np.float16
        sc = scales.astype(np.float32).reshape(-1)
        if b + ".biases" in raw:
            keep_f16 = keep_f16 and raw[b + ".biases"].dtype == np.float16
            bi = raw[b + ".biases"].astype(np.float32).reshape(-1)
        elif b + ".zeros" in raw:
            bi = -sc * raw[b + ".zeros"].astype(np.float32).reshape(-1)
            keep_f16 = False
        else:
            bi = np.zeros_like(sc)
        if b + ".bits" in raw:
            bits = int(raw[b + ".bits"].reshape(-1)[0])
        elif b + ".bit_map" in raw:
            bits = int(raw[b + ".bit_map"].reshape(-1)[0])
        else:
            bits = 4
        if bits not in ALLOWED_STORAGE_BITS:
            raise BundleError(f"{b}: invalid bit width {bits}")
        n_blocks = sc.shape[0]
        shape = tuple(int(x) for x in raw[b + ".shape"].reshape(-1)) if b + ".shape" in raw else (n_blocks, block)
        if len(shape) >= 3:
            experts, e_out, in_dim = shape[0], int(np.prod(shape[1:-1])), shape[-1]
            out_dim = experts * e_out
        elif len(shape) == 2:
            experts, e_out = 0, 0
            out_dim, in_dim = shape
        else:
            raise BundleError(f"{b}: shape {shape} is not a matrix")
        data = raw[b + ".qweight"].astype(np.uint8, copy=False).tobytes()
        data += b"\x00" * ((4 - len(data) % 4) % 4)
        words = np.frombuffer(data, dtype=np.uint32)
        per_row = (in_dim * bits + 31) // 32
        need = out_dim * per_row
        if words.shape[0] < need:
            words = np.pad(words, (0, need - words.shape[0]))
        words = words[:need]
        groups_row = (in_dim + block - 1) // block
        need_g = out_dim * groups_row
        if n_blocks < need_g:
            sc = np.pad(sc, (0, need_g - n_blocks), constant_values=1.0)
            bi = np.pad(bi, (0, need_g - n_blocks), constant_values=0.0)
        lead = (experts, e_out) if experts else (out_dim,)
        wq = words.reshape(lead + (per_row,))
        dt = np.float16 if keep_f16 else np.float32
        s2 = sc[:need_g].reshape(lead + (groups_row,)).astype(dt)
        b2 = bi[:need_g].reshape(lead + (groups_row,)).astype(dt)
        if experts and "gate_up_proj" in b:
            mid = e_out // 2
            prefix = b.replace("experts.gate_up_proj", "switch_mlp")
            for nm, sl in (("gate_proj", slice(0, mid)), ("up_proj", slice(mid, e_out))):
                out[f"{prefix}.{nm}.weight"] = np.ascontiguousarray(wq[:, sl, :])
                out[f"{prefix}.{nm}.scales"] = np.ascontiguousarray(s2[:, sl, :])
                out[f"{prefix}.{nm}.biases"] = np.ascontiguousarray(b2[:, sl, :])
        else:
            out[b + ".weight"], out[b + ".scales"], out[b + ".biases"] = wq, s2, b2
    for k, v in raw.items():
        if k not in quant_keys:
            out[k] = v
    return out


def repack_v1_to_v2(src, dst, max_shard_bytes: int = 5 * 1024 ** 3) -> None:
    """Rewrite a v1 bundle directory as a v2 bundle: tensors through `read_v1_tensors`, a manifest with the
    width of every module (from the shapes), configs carried over."""
    src = Path(src)
    tensors = read_v1_tensors(src)
    cfg_path = find_config_path(src)
    jang_config = _read_json(cfg_path, "JANG config")
    model_config = _read_json(src / "config.json", "model config") if (src / "config.json").exists() else {}
    model_config.pop("quantization", None)
    block = int((jang_config.get("quantization") or {}).get("block_size", 64))
    manifest, widths = {}, set()
    for name in tensors:
        if name.endswith(".scales") and name[:-7] + ".weight" in tensors and tensors[name[:-7] + ".weight"].dtype == np.uint32:
            m = name[:-7]
            bits, gs = infer_bits_group_size(tensors[m + ".weight"].shape[-1], tensors[name].shape[-1], block)
            widths.add(bits)
            manifest[m] = {"bits": bits, "group_size": gs, "weight_key": m + ".weight", "scales_key": m + ".scales",
                           "biases_key": m + ".biases", "weight_shape": list(tensors[m + ".weight"].shape),
                           "scales_shape": list(tensors[name].shape), "biases_shape": list(tensors[m + ".biases"].shape)}
    jc = {k: v for k, v in jang_config.items() if k != "format_version"}
    q = dict(jc.get("quantization") or {})
    q.update({"bit_widths_used": sorted(widths) or [4], "block_size": block, "tensor_quantization_manifest": manifest})
    jc["quantization"] = q
    write_bundle(dst, tensors, model_config, jc, max_shard_bytes)


# ---- load_jang_model -------------------------------------------------------------------------------
def _tree_set(root, dotted: str, leaf) -> None:
    """Hang `leaf` into nested torch containers under its dotted path (numeric parts included)."""
    import torch
    parts = dotted.split(".")
    node = root
    for p in parts[:-1]:
        if p not in node._modules:
            node.add_module(p, torch.nn.Module())
        node = node._modules[p]
    if isinstance(leaf, torch.nn.Module):
        node.add_module(parts[-1], leaf)
    else:
        node.register_buffer(parts[-1], leaf)


def load_jang_model(model_path, device="cuda", sidecar_dtype=None, float_dtype=None):
    """(model, tokenizer) of a JANG bundle, the call shape of jang_tools/loader.py:1078.

    The reference returns an mlx-lm network; here `model` is a torch module tree that follows the bundle's
    tensor names: every quantized module is a JANGLinear (2-D weight), a JANGSwitchLinear (stacked experts
    [E, out, packed]) or a JANGEmbedding (names ending in embed_tokens / wte / word_embeddings), every other
    tensor a buffer at its dotted path, so `model.get_submodule("model.layers.0.self_attn.q_proj")(x)` runs the
    quantized product and `model.state_dict()` carries the bundle's names.  `model.config` and
    `model.jang_config` hold the two JSON files.  The network's own forward (attention, norms, sampling) is
    outside the quantized path and is not built.  v1 bundles are repacked in memory first, as the reference
    does on load.  `tokenizer` comes from transformers.AutoTokenizer when the directory has tokenizer files,
    else None."""
    import torch

    from .linear import JANGEmbedding, JANGLinear, JANGSwitchLinear
    p = Path(model_path)
    cfg_path = find_config_path(p)
    if cfg_path is None:
        raise FileNotFoundError(f"No JANG config found in {p}")
    jang_cfg = _read_json(cfg_path, "JANG config")
    if not jang_cfg.get("format"):
        raise ValueError(f"JANG config {cfg_path.name} is missing 'format' field")
    dt = sidecar_dtype or torch.float16
    model = torch.nn.Module()
    model.jang_config = jang_cfg
    model.config = _read_json(p / "config.json", "model config") if (p / "config.json").exists() else {}

    if is_v2_model(p):
        b = open_bundle(p)
        names = b.names()
        get = b.tensor
        spec_of = lambda m, ws, ss: b.quant_spec(m, ws, ss)          # noqa: E731
        closer = b.close
    else:
        tensors = read_v1_tensors(p)
        names = sorted(tensors)
        get = tensors.__getitem__
        block = int((jang_cfg.get("quantization") or {}).get("block_size", 64))

        def spec_of(m, ws, ss):
            bits, gs = infer_bits_group_size(ws[-1], ss[-1], block)
            return QuantSpec(bits, gs, bits)
        closer = lambda: None                                          # noqa: E731

    quantized = {n[:-len(".scales")] for n in names if n.endswith(".scales") and n[:-len(".scales")] + ".weight" in names}
    done = set()
    for m in sorted(quantized):
        w, s = get(m + ".weight"), get(m + ".scales")
        if w.dtype != np.uint32:
            continue
        bi = get(m + ".biases")
        spec = spec_of(m, w.shape, s.shape)
        if spec.storage_bits == 1:
            w = expand_1bit_to_2bit(w)
        wt = torch.from_numpy(np.ascontiguousarray(w).view(np.int32)).to(device)
        st = torch.from_numpy(np.ascontiguousarray(s)).to(device).to(dt)
        bt = torch.from_numpy(np.ascontiguousarray(bi)).to(device).to(dt)
        k = s.shape[-1] * spec.group_size
        if w.ndim == 3:
            leaf = JANGSwitchLinear(w.shape[0], k, w.shape[1], spec.bits, spec.group_size, device=device, dtype=dt)
        elif m.rsplit(".", 1)[-1] in ("embed_tokens", "wte", "word_embeddings"):
            leaf = JANGEmbedding(w.shape[0], k, spec.bits, spec.group_size, device=device, dtype=dt)
        elif w.ndim == 2:
            has_bias = (m + ".bias") in names
            leaf = JANGLinear(k, w.shape[0], spec.bits, spec.group_size, bias=has_bias, device=device, dtype=dt)
            if has_bias:
                leaf.bias = torch.from_numpy(np.ascontiguousarray(get(m + ".bias"))).to(device).to(dt)
                done.add(m + ".bias")
        else:
            raise BundleError(f"{m}.weight has {w.ndim} dimensions")
        leaf.weight, leaf.scales, leaf.biases = wt, st, bt
        _tree_set(model, m, leaf)
        done.update((m + ".weight", m + ".scales", m + ".biases"))
    for n in names:
        if n in done:
            continue
        t = torch.from_numpy(np.ascontiguousarray(get(n)))
        if float_dtype is not None and t.is_floating_point():
            t = t.to(float_dtype)
        _tree_set(model, n, t.to(device))
    closer()

    tokenizer = None
    if any((p / f).exists() for f in ("tokenizer.json", "tokenizer.model", "tokenizer_config.json")):
        try:
            from transformers import AutoTokenizer
            tokenizer = AutoTokenizer.from_pretrained(str(p))
        except Exception:            # a bundle without usable tokenizer files still loads its weights
            tokenizer = None
    return model, tokenizer
