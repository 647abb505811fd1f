"""Pin the CPU oracle against vectors produced by the reference's own code
(tests/golden/make_golden.py) and against the reference's MLX golden vector."""
import os

import numpy as np
import pytest

from oracle import jang_oracle as jo

BITS = (2, 3, 4, 5, 6, 8)
GSS = (32, 64, 128)


def _load(golden_dir, name):
    return np.load(os.path.join(golden_dir, name))


def test_pack_known_answers():
    # reference known-answer bytes: jang-tools/tests/test_pack.py:33-61
    assert jo.pack_rows(np.array([[0, 1, 2, 3] * 4], np.uint8), 2).view(np.uint8)[0, 0] == 0xE4
    v4 = np.array([[5, 10, 3, 15, 0, 0, 0, 0]], np.uint8)
    by = jo.pack_rows(v4, 4).view(np.uint8)[0]
    assert by[0] == 0xA5 and by[1] == 0xF3
    # 3-bit example from the reference docstring (pack.py:22-25); only bytes 0
    # and 2 of the docstring are self-consistent with LSB-first packing, so pin
    # against the reference's computed stream in pack_ref.npz instead.


@pytest.mark.parametrize("bits", (2, 3, 4, 5, 6, 8))
def test_pack_stream_matches_reference(golden_dir, bits):
    z = _load(golden_dir, "pack_ref.npz")
    v = z[f"b{bits}_values"]
    ref = z[f"b{bits}_bytes"]
    got = jo.pack_rows(v[None, :], bits).view(np.uint8).reshape(-1)
    assert np.array_equal(got, ref)
    assert np.array_equal(jo.unpack_rows(ref.view("<u4")[None, :], bits, v.size)[0], v)


@pytest.mark.parametrize("gs", GSS)
@pytest.mark.parametrize("bits", BITS)
def test_affine_quantizer_matches_reference(golden_dir, bits, gs):
    z = _load(golden_dir, "affine_ref.npz")
    key = f"b{bits}_g{gs}"
    w = z[key + "_w"]
    packed, s, b = jo.quantize_affine(w, bits, gs, src_dtype="f16", f16_tiny_guard=True)
    assert np.array_equal(packed, z[key + "_packed"])
    assert np.array_equal(s, z[key + "_scales"].astype(np.float32))
    assert np.array_equal(b, z[key + "_biases"].astype(np.float32))
    deq = jo.dequantize_affine(packed, s, b, bits, gs)
    assert np.array_equal(deq, z[key + "_deq"])


@pytest.mark.parametrize("bits", (2, 3, 4, 6, 8))
def test_affine_quantizer_gaussian(golden_dir, bits):
    z = _load(golden_dir, "affine_ref_gauss.npz")
    packed, s, b = jo.quantize_affine(z["w"], bits, 64, src_dtype="f16", f16_tiny_guard=True)
    assert np.array_equal(packed, z[f"b{bits}_packed"])
    assert np.array_equal(s, z[f"b{bits}_scales"].astype(np.float32))
    assert np.array_equal(b, z[f"b{bits}_biases"].astype(np.float32))


@pytest.mark.parametrize("bits", (2, 3, 4, 6, 8))
def test_rtn_matches_reference(golden_dir, bits):
    z = _load(golden_dir, "rtn_ref.npz")
    packed, s, b = jo.quantize_rtn(z["w"], bits, 64)
    assert np.array_equal(packed, z[f"b{bits}_packed"])
    assert np.array_equal(s, z[f"b{bits}_scales"].astype(np.float32))
    assert np.array_equal(b, z[f"b{bits}_biases"].astype(np.float32))


@pytest.mark.parametrize("gs", (32, 64, 128))
@pytest.mark.parametrize("bits", (2, 3, 4, 6))
def test_mse_matches_reference(golden_dir, bits, gs):
    """quantize_tensor(method="mse") (quantize.py:153-191): the oracle reproduces the reference's
    codes and float16 sidecars, including the constant, zero and outlier blocks of the fixture."""
    z = _load(golden_dir, "mse_ref.npz")
    packed, s, b = jo.quantize_mse(z["w"], bits, gs)
    key = f"g{gs}_b{bits}"
    assert np.array_equal(packed, z[key + "_packed"])
    assert np.array_equal(s, z[key + "_scales"].astype(np.float32))
    assert np.array_equal(b, z[key + "_biases"].astype(np.float32))


def test_mse_search_clips_outliers(golden_dir):
    """The search is not a no-op: on the fixture at 2 bits it picks a narrower range than min/max
    for most blocks, and its reconstruction error is lower than plain RTN's."""
    z = _load(golden_dir, "mse_ref.npz")
    w = z["w"]
    pm, sm, bm = jo.quantize_mse(w, 2, 64)
    pr, sr, br = jo.quantize_rtn(w, 2, 64)
    assert (sm < sr).mean() > 0.5
    em = ((jo.dequantize_affine(pm, sm, bm, 2, 64) - w) ** 2).mean()
    er = ((jo.dequantize_affine(pr, sr, br, 2, 64) - w) ** 2).mean()
    assert em < er


def test_mlx_golden_vector(golden_dir):
    """The reference's only MLX-made vector: regenerate W and x from the seed
    (jang-tools/scripts/gen_matmul_fixture.py:34-36), quantize with f32 source
    and f16 sidecars -> identical codes/scales/biases; y within 1e-2
    (QuantizedMatmul4Tests.swift:83-84)."""
    z = _load(golden_dir, "mlx_matmul_4bit_64x128.npz")
    rng = np.random.default_rng(int(z["seed"]))
    W = rng.standard_normal((128, 64)).astype(np.float32)
    x = rng.standard_normal((64,)).astype(np.float16)
    assert np.array_equal(x, z["x"])
    packed, s, b = jo.quantize_affine(W, 4, 64, src_dtype="f32", sidecar_dtype="f16")
    assert np.array_equal(packed, z["packed"])
    assert np.array_equal(s, z["scales"].astype(np.float32))
    assert np.array_equal(b, z["biases"].astype(np.float32))
    y = jo.qmatmul(x.astype(np.float32), packed, s, b, 4, 64)[0]
    y_ref = z["y_ref"]
    assert np.all(np.abs(y - y_ref) < 1e-2)
    assert np.all(np.abs(y - y_ref) / np.maximum(np.abs(y_ref), 1e-6) < 1e-2)
    y2 = jo.qmatmul_group_order(x.astype(np.float32), packed, s, b, 4, 64)[0]
    # y_ref came from mx.dequantize's f16 weights, hence the fixture's own 1e-2 bound
    assert np.all(np.abs(y2 - y_ref) < 1e-2) and np.allclose(y2, y, atol=1e-4)


def test_bf16_rounding_helpers():
    torch = pytest.importorskip("torch")
    x = np.random.default_rng(3).standard_normal(4096).astype(np.float32) * 1e-3
    ref = torch.from_numpy(x).to(torch.bfloat16).float().numpy()
    assert np.array_equal(jo.round_to(x, "bf16"), ref)


def test_moe_sort_and_naive_layer():
    rng = np.random.default_rng(0)
    T, k, E, H, I = 9, 2, 4, 64, 64
    idx = rng.integers(0, E, (T, k)).astype(np.int32)
    order, inv, off = jo.moe_sort(idx, E)
    flat = idx.reshape(-1)
    assert np.all(np.diff(flat[order]) >= 0) and np.array_equal(order[inv], np.arange(T * k))
    assert off[-1] == T * k
    x = rng.standard_normal((T, H)).astype(np.float32)
    w = rng.random((T, k)).astype(np.float32)
    mats = [(rng.standard_normal(s) * 0.1).astype(np.float32) for s in ((E, I, H), (E, I, H), (E, H, I))]
    q = []
    for m in mats:
        trip = [jo.quantize_affine(m[e], 8, 32, src_dtype="f32") for e in range(E)]
        q.append((np.stack([t[0] for t in trip]), np.stack([t[1] for t in trip]),
                  np.stack([t[2] for t in trip]), 8, 32))
    got = jo.moe_layer(x, idx, w, *q, act_dtype="f32")
    # naive loop of dots3/ops_selftest.py:18-27 over the dequantised experts
    deq = [np.stack([jo.dequantize_affine(t[0][e], t[1][e], t[2][e], 8, 32) for e in range(E)]) for t in q]
    ref = np.zeros((T, H), np.float32)
    for t in range(T):
        for j in range(k):
            e = int(idx[t, j])
            g = x[t] @ deq[0][e].T
            u = x[t] @ deq[1][e].T
            ref[t] += w[t, j] * (((g / (1 + np.exp(-g))) * u) @ deq[2][e].T)
    assert np.abs(got - ref).max() / np.abs(ref).max() < 1e-4


def test_imatrix_affine_fit_matches_reference(golden_dir):
    """oracle.quantize_imatrix_affine against the reference's quantize_imatrix_affine_numpy
    (tests/golden/imatrix_ref.npz, made by make_golden_imatrix.py): codes, sidecars and the error bit for bit."""
    z = _load(golden_dir, "imatrix_ref.npz")
    for gs in (32, 64, 128):
        for bits in (2, 3, 4, 5, 6, 8):
            k = f"b{bits}_g{gs}"
            packed, s, b, err = jo.quantize_imatrix_affine(z[k + "_w"], z[k + "_imp"], bits, gs)
            assert np.array_equal(packed, z[k + "_packed"]), k
            assert np.array_equal(s.view(np.uint16), z[k + "_scales"].view(np.uint16)), k
            assert np.array_equal(b.view(np.uint16), z[k + "_biases"].view(np.uint16)), k
            assert err == float(z[k + "_err"]), k
    packed, s, b, _ = jo.quantize_imatrix_affine(z["it2_w"], z["it2_imp"], 3, 64, iterations=2)
    assert np.array_equal(packed, z["it2_packed"]) and np.array_equal(s, z["it2_scales"]) and np.array_equal(b, z["it2_biases"])


def test_hadamard_rotation_oracle_properties():
    """The restated rotation against an explicit Hadamard matrix, and its defining properties."""
    from scipy.linalg import hadamard
    rng = np.random.default_rng(1)
    assert jo.pow2_blocks(192) == [128, 64] and jo.pow2_blocks(11008) == [8192, 2048, 512, 256] and jo.pow2_blocks(64) == [64]
    s = jo.hadamard_signs(64, seed=42)
    assert set(np.unique(s)) <= {-1.0, 1.0} and np.array_equal(s, jo.hadamard_signs(64, seed=42))
    x = rng.standard_normal((3, 64)).astype(np.float32)
    ref = (x * s).astype(np.float64) @ hadamard(64).astype(np.float64) / 8.0
    assert np.abs(jo.hadamard_rotate(x, s) - ref).max() < 1e-5
    for dim in (192, 4096, 11008):
        s = jo.hadamard_signs(dim, seed=42)
        x = rng.standard_normal((2, dim)).astype(np.float32)
        w = rng.standard_normal((5, dim)).astype(np.float32)
        xr, wr = jo.hadamard_rotate(x, s), jo.hadamard_rotate(w, s)
        assert np.abs(np.linalg.norm(xr, axis=-1) - np.linalg.norm(x, axis=-1)).max() < 1e-3
        assert np.abs(xr @ wr.T - x @ w.T).max() < 2e-3 * np.abs(x @ w.T).max() + 1e-3      # the rotation cancels
        assert np.abs(jo.hadamard_inverse(xr, s) - x).max() < 1e-4


# ---- JANGTQ codebook weights ----------------------------------------------------------------------------------
def test_tq_codebooks_match_the_reference():
    """Oracle and package codebooks against centroids the reference's compute_codebook produced
    (tests/golden/tq_codebooks.json, written by tests/golden/make_golden_tq.py): exact, they are format data."""
    import json
    from jangq_b200 import turboquant as tq
    gold = json.load(open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "tq_codebooks.json")))
    assert len(gold) == 21
    for key, want in gold.items():
        d, b = (int(v) for v in key.split("x"))
        assert np.array_equal(jo.tq_codebook(d, b), np.array(want)), key
        assert list(tq.compute_codebook(d, b)) == want, key


def test_tq_pack_and_products_agree():
    """Packing (10 three-bit indices per word), and the two forms of the product: rotated activations against
    norm * codebook[idx] (the kernels) equals x against the de-rotated matrix (TurboQuantLinear.__call__)."""
    rng = np.random.default_rng(2)
    for bits, K in ((2, 256), (3, 320), (4, 192)):
        idx = rng.integers(0, 1 << bits, (7, K)).astype(np.uint8)
        p = jo.tq_pack(idx, bits)
        assert p.shape == (7, K // (32 // bits)) and np.array_equal(jo.tq_unpack(p, bits, K), idx)
        if bits == 3:
            assert np.all((p >> np.uint32(30)) == 0)            # the top two bits of a 3-bit word stay empty
        w = (rng.standard_normal((24, K)) * 0.05).astype(np.float32)
        packed, norms, cb, signs = jo.tq_quantize(w, bits, seed=7)
        deq = jo.tq_dequantize(packed, norms, cb, signs, bits)
        assert np.abs(deq - w).max() < {2: 0.12, 3: 0.07, 4: 0.05}[bits]
        x = rng.standard_normal((3, K)).astype(np.float32)
        a = jo.tq_matmul_rotated(jo.hadamard_rotate(x, signs), packed, norms, cb, bits)
        b = x.astype(np.float64) @ deq.astype(np.float64).T
        assert np.abs(a - b).max() <= 1e-4 * np.abs(b).max()
