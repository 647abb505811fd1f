"""Host-side bit-width map: which tensor gets how many bits, which group size, and how the
loader recovers (bits, group_size) from tensor shapes.  Pure metadata, no kernels.

Mirrors the rules of the reference for the tensor families the BASELINE configurations use
(dense Llama-shaped decoders and routed-MoE stacks):

    Tier / classify_tensor        jang_tools/allocate.py:259-318 (first matching name pattern wins)
    JANG_PROFILES                 jang_tools/allocate.py:489-514 (critical, important, compress bits)
    allocate_bits_profile_compact jang_tools/allocate.py:1086-1124
    MLP asymmetry floors          jang_tools/allocate.py:345-357 (>= 256 experts: gate 4, down 3)
    group-size policy             jang_tools/convert.py:558-599, 770-783
    infer_bits_and_group_size     jang_tools/loader.py:1958-1973, quant_shape_inference.py:24-75

The reference's pattern table also names dozens of model-zoo specific tensors (Mamba, MLA,
vision towers, ...); those families are outside this package's scope and fall to the same
default the reference uses for unknown projections (COMPRESS).
"""
from __future__ import annotations

import enum
from typing import Iterable

ALLOWED_BITS = (2, 3, 4, 5, 6, 8)
GROUP_SIZES = (128, 64, 32)


class Tier(enum.Enum):
    CRITICAL = "critical"      # full attention, output head, routers, shared experts: breaks first at low bits
    IMPORTANT = "important"    # embeddings, linear-attention projections
    COMPRESS = "compress"      # MLP / routed-expert projections: the bulk of the bytes


# (substring, tier); order matters — the first match wins, exactly as in the reference
_RULES = (
    ("lm_head", Tier.CRITICAL), ("shared_expert_gate", Tier.CRITICAL), ("shared_expert", Tier.CRITICAL),
    ("q_proj", Tier.CRITICAL), ("k_proj", Tier.CRITICAL), ("v_proj", Tier.CRITICAL), ("o_proj", Tier.CRITICAL),
    ("qkv_proj", Tier.CRITICAL),
    ("embed_tokens", Tier.IMPORTANT), ("wte", Tier.IMPORTANT), ("word_embeddings", Tier.IMPORTANT),
    ("router.proj", Tier.CRITICAL), ("router", Tier.CRITICAL),
    ("gate_up_proj", Tier.COMPRESS), ("gate_proj", Tier.COMPRESS), ("up_proj", Tier.COMPRESS),
    ("down_proj", Tier.COMPRESS), ("w1", Tier.COMPRESS), ("w2", Tier.COMPRESS), ("w3", Tier.COMPRESS),
    ("out_proj", Tier.COMPRESS), ("proj", Tier.COMPRESS), ("fc", Tier.COMPRESS),
)

JANG_PROFILES = {
    "JANG_2S": (6, 4, 2), "JANG_2M": (8, 4, 2), "JANG_2L": (8, 6, 2), "JANG_1L": (8, 8, 2),
    "JANG_3S": (6, 3, 3), "JANG_3M": (8, 3, 3), "JANG_3L": (8, 4, 3),
    "JANG_4S": (6, 4, 4), "JANG_4M": (8, 4, 4), "JANG_4L": (8, 6, 4),
    "JANG_6M": (8, 6, 6),
}

_MLP_FLOORS = {"gate_proj": 4, "gate_up_proj": 4, "w1": 4, "down_proj": 3, "w2": 3}
_MLP_FLOOR_MIN_EXPERTS = 256


def classify_tensor(name: str, num_experts: int = 0, has_shared_mlp: bool = False) -> Tier:
    """Sensitivity tier of a tensor from its name."""
    low = name.lower()
    if (num_experts > 0 or has_shared_mlp) and "experts" not in low:
        # dense MLPs inside a MoE model run for every token: keep them high precision
        if any(p in low for p in ("mlp.gate_proj", "mlp.up_proj", "mlp.down_proj", "mlp.fc1", "mlp.fc2")):
            return Tier.CRITICAL
    for pat, tier in _RULES:
        if pat in low:
            return tier
    if ".gate." in low or low.endswith(".gate"):
        return Tier.CRITICAL                                 # MoE router named "gate"
    return Tier.COMPRESS


def is_router(name: str) -> bool:
    """Routers are never quantized (f16 passthrough, jang_tools/convert.py:1336-1345)."""
    low = name.lower()
    return (".gate." in low or low.endswith(".gate") or ".router." in low or low.endswith(".router")) \
        and "gate_proj" not in low


def allocate_bits_profile(tensor_names: Iterable[str], profile: str = "JANG_3M", num_experts: int = 0,
                          has_shared_mlp: bool = False, apply_mlp_asymmetry: bool = True) -> dict[str, int]:
    """tensor name -> bits for a named profile (the per-tensor bit-width map)."""
    profile = profile.upper()
    if profile not in JANG_PROFILES:
        raise ValueError(f"Unknown profile '{profile}'. Available: {list(JANG_PROFILES)}")
    crit, imp, comp = JANG_PROFILES[profile]
    by_tier = {Tier.CRITICAL: crit, Tier.IMPORTANT: imp, Tier.COMPRESS: comp}
    out = {}
    for name in tensor_names:
        bits = by_tier[classify_tensor(name, num_experts, has_shared_mlp)]
        low = name.lower()
        if apply_mlp_asymmetry and num_experts >= _MLP_FLOOR_MIN_EXPERTS and "expert" in low \
                and "shared_expert" not in low:
            for part, floor in _MLP_FLOORS.items():
                if part in low:
                    bits = max(bits, floor)
                    break
        out[name] = bits
    return out


def model_group_size(num_experts: int) -> int:
    """Bundle-wide default: 128 for models with 150 or more experts, else 64."""
    return 128 if num_experts >= 150 else 64


def tensor_group_size(name: str, in_dim: int, default_gs: int = 64) -> int | None:
    """Group size of one tensor: routers stay at 64; otherwise the largest of 128/64/32 not above
    the bundle's default that divides in_dim; None = leave the tensor unquantized."""
    want = 64 if is_router(name) or "shared_expert_gate" in name.lower() else default_gs
    for gs in GROUP_SIZES:
        if gs <= want and in_dim > 0 and in_dim % gs == 0:
            return gs
    return None


def infer_bits_and_group_size(weight_cols: int, scales_cols: int, group_size: int | None = None,
                              prefer_high_bits: bool = True) -> tuple[int, int]:
    """(bits, group_size) from the packed width and the sidecar width of a module:
    bits * group_size = 32 * weight_cols / scales_cols.  With the bundle's group size known the
    bit width is unique; otherwise the candidates are ranked high-bit first (attention, embeddings)
    or low-bit first (routed experts), as the reference's tiebreaker does."""
    if scales_cols <= 0 or (32 * weight_cols) % scales_cols:
        raise ValueError(f"shapes do not describe a quantized tensor: {weight_cols} packed / {scales_cols} groups")
    product = 32 * weight_cols // scales_cols
    cands = [(b, product // b) for b in ALLOWED_BITS if product % b == 0 and product // b in GROUP_SIZES]
    if group_size is not None:
        cands = [c for c in cands if c[1] == group_size]
    if not cands:
        raise ValueError(f"no (bits, group_size) pair gives bits*group_size = {product}")
    cands.sort(key=lambda c: c[0], reverse=prefer_high_bits)
    return cands[0]


def _step(bits: int, up: bool) -> int | None:
    """Neighbouring allowed width (2 -> 3 -> 4 -> 5 -> 6 -> 8), None at either end."""
    i = ALLOWED_BITS.index(bits) + (1 if up else -1)
    return ALLOWED_BITS[i] if 0 <= i < len(ALLOWED_BITS) else None


def _routed_expert_part(low: str) -> str | None:
    """The MLP projection a routed-expert tensor name carries (None for anything else)."""
    if "shared_expert" in low or "expert" not in low:
        return None
    for part in ("gate_up_proj", "gate_proj", "up_proj", "down_proj", "w1", "w2", "w3"):
        if part in low:
            return part
    return None


def _asymmetry_floor(name: str, bits: int, num_experts: int, base_bits: int = 0) -> int:
    """Lowest width a routed-expert projection may get in a model with >= 256 experts: the namesake
    width for 4-bit-and-up budgets, else gate 4 / down 3 (jang_tools/allocate.py:427-474)."""
    low = name.lower()
    if num_experts < _MLP_FLOOR_MIN_EXPERTS or "shared_expert" in low:
        return bits
    if base_bits >= 4 and any(p in low for p in ("gate_proj", "gate_up_proj", "w1", "up_proj", "w3", "down_proj", "w2")):
        return max(bits, base_bits)
    for part, floor in _MLP_FLOORS.items():
        if part in low:
            return max(bits, floor)
    return bits


def _layer_index(name: str) -> int | None:
    parts = name.split(".")
    for i, p in enumerate(parts[:-1]):
        if p == "layers":
            try:
                return int(parts[i + 1])
            except ValueError:
                return None
    return None


def allocate_bits_budget(tensor_info: Iterable[tuple[str, int]], target_bits: float = 4.0, num_experts: int = 0,
                         has_shared_mlp: bool = False) -> dict[str, int]:
    """Budget-neutral per-tensor map (jang_tools/allocate.py:1127-1221, allocate_bits_budget_compact):
    tensor_info = [(name, number of 64-weight blocks)]; the result averages about `target_bits` per weight.

    Every tensor starts at the largest allowed width not above the target.  CRITICAL tensors climb up to
    four steps (two when they make up 5 % or more of the model), tensors of the first and last two layers one
    more step (routed experts of a 2-bit budget excepted), and the overspend is paid back by moving
    COMPRESS tensors, smallest first, one step down wherever the expert floors allow it."""
    info = list(tensor_info)
    total = sum(n for _, n in info)
    base = max((b for b in ALLOWED_BITS if b <= target_bits), default=2)
    tier = {name: classify_tensor(name, num_experts, has_shared_mlp) for name, _ in info}
    bits = {name: base for name, _ in info}

    critical = sum(n for name, n in info if tier[name] is Tier.CRITICAL)
    steps = 4 if (critical / total if total else 0.0) < 0.05 else 2
    for name, _ in info:
        if tier[name] is Tier.CRITICAL:
            for _ in range(steps):
                nxt = _step(bits[name], True)
                if nxt is None:
                    break
                bits[name] = nxt

    layer = {name: _layer_index(name) for name, _ in info}
    known = [l for l in layer.values() if l is not None]
    n_layers = max(known) + 1 if known else 1
    for name, _ in info:
        l = layer[name]
        if l is None or (base == 2 and _routed_expert_part(name.lower()) is not None):
            continue
        if l < 2 or l >= n_layers - 2:
            nxt = _step(bits[name], True)
            if nxt is not None:
                bits[name] = nxt

    over = sum(bits[name] * n for name, n in info) - target_bits * total
    lower = _step(base, False)
    if over > 0 and lower is not None:
        for name, n in sorted(((name, n) for name, n in info if tier[name] is Tier.COMPRESS), key=lambda t: t[1]):
            if over <= 0:
                break
            if _asymmetry_floor(name, lower, num_experts, base) > lower:
                continue
            bits[name] = lower
            over -= (base - lower) * n
    return bits
