"""GPU parity of the affine quantizer, the RTN fallback and the dequantizer
against the CPU oracle and the reference-made golden vectors.  Integer outputs
(packed codes) and the stored sidecars must be bit-exact."""
import os

import numpy as np
import pytest
import torch

import jangq_b200 as jq
from oracle import jang_oracle as jo

pytestmark = pytest.mark.gpu

BITS = (2, 3, 4, 5, 6, 8)
GSS = (32, 64, 128)
TORCH_DT = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}


def dev():
    return torch.device("cuda:0")


def to_np_u32(t):
    return t.cpu().numpy().view(np.uint32)


def f32(t):
    return t.float().cpu().numpy()


def adversarial(rng, rows, K, gs):
    w = (rng.standard_normal((rows, K)) * 0.02).astype(np.float32)
    g = w.reshape(rows, K // gs, gs)
    g[0, 0] = 0.0
    g[1, 0] = 0.0371
    g[2, 0] = -0.0371
    g[3, 0] = np.abs(g[3, 0])
    g[4, 0] = -np.abs(g[4, 0])
    g[5, 0, 7] = 3.5
    g[6, 0, 3] = -3.5
    g[7, -1] = np.linspace(-1.0, 1.0, gs)
    g[8, -1] = np.arange(gs) * 0.5
    g[9, -1] = np.concatenate([[0.0, 0.5, 1.5, 3.0], np.zeros(gs - 4)])
    g[10, -1] = np.where(np.arange(gs) % 2 == 0, 0.0, -0.0)
    g[11, -1] = 1e-9 * rng.standard_normal(gs)
    g[12, -1] = np.arange(gs) - gs / 2 + 0.5            # many exact .5 ties after scaling
    return g.reshape(rows, K)


@pytest.mark.parametrize("gs", GSS)
@pytest.mark.parametrize("bits", BITS)
def test_golden_reference_vectors(golden_dir, bits, gs):
    z = np.load(os.path.join(golden_dir, "affine_ref.npz"))
    key = f"b{bits}_g{gs}"
    w = torch.from_numpy(z[key + "_w"]).to(dev())
    wq, s, b = jq.quantize(w, gs, bits, f16_tiny_guard=True)
    assert np.array_equal(to_np_u32(wq), z[key + "_packed"])
    assert np.array_equal(s.cpu().numpy(), z[key + "_scales"])
    assert np.array_equal(b.cpu().numpy(), z[key + "_biases"])
    deq = jq.dequantize(wq, s, b, gs, bits, dtype=torch.float32)
    assert np.array_equal(deq.cpu().numpy(), z[key + "_deq"])


def test_mlx_golden_vector(golden_dir):
    z = np.load(os.path.join(golden_dir, "mlx_matmul_4bit_64x128.npz"))
    rng = np.random.default_rng(int(z["seed"]))
    W = rng.standard_normal((128, 64)).astype(np.float32)
    x = rng.standard_normal((64,)).astype(np.float16)
    wq, s, b = jq.quantize(torch.from_numpy(W).to(dev()), 64, 4, sidecar_dtype=torch.float16)
    assert np.array_equal(to_np_u32(wq), z["packed"])
    assert np.array_equal(s.cpu().numpy(), z["scales"])
    assert np.array_equal(b.cpu().numpy(), z["biases"])
    y = jq.quantized_matmul(torch.from_numpy(x).to(dev())[None, :], wq, s, b, group_size=64, bits=4)[0]
    y = y.float().cpu().numpy()
    y_ref = z["y_ref"]
    # tolerance of the reference's own consumer of this vector (QuantizedMatmul4Tests.swift:83-84);
    # the output here is float16, hence the extra half-ulp term
    assert np.all(np.abs(y - y_ref) < 1e-2 + 2.0 ** -11 * np.abs(y_ref))


@pytest.mark.parametrize("src", ("bf16", "f16", "f32"))
@pytest.mark.parametrize("gs", GSS)
@pytest.mark.parametrize("bits", BITS)
def test_affine_bit_exact_vs_oracle(bits, gs, src):
    rng = np.random.default_rng(bits * 1000 + gs)
    w = adversarial(rng, 48, 1280, gs)
    wt = torch.from_numpy(w).to(dev()).to(TORCH_DT[src])
    wq, s, b = jq.quantize(wt, gs, bits)
    pk, so, bo = jo.quantize_affine(f32(wt), bits, gs, src_dtype=src)
    assert np.array_equal(to_np_u32(wq), pk)
    assert np.array_equal(f32(s), so)
    assert np.array_equal(f32(b), bo)
    assert s.dtype == TORCH_DT[src]


@pytest.mark.parametrize("bits", (2, 3, 4, 6, 8))
def test_rtn_golden(golden_dir, bits):
    z = np.load(os.path.join(golden_dir, "rtn_ref.npz"))
    wq, s, b = jq.quantize(torch.from_numpy(z["w"]).to(dev()), 64, bits, mode="rtn")
    assert np.array_equal(to_np_u32(wq), z[f"b{bits}_packed"])
    assert np.array_equal(s.cpu().numpy(), z[f"b{bits}_scales"])
    assert np.array_equal(b.cpu().numpy(), z[f"b{bits}_biases"])


@pytest.mark.parametrize("bits", (2, 3, 4, 5, 6, 8))
def test_rtn_vs_oracle(bits):
    rng = np.random.default_rng(5 + bits)
    w = (rng.standard_normal((40, 768)) * 0.02).astype(np.float32)
    w[3, 64:128] = -0.125
    w[6] = 1000.0 + w[6] * 1e-3                          # quotients far outside the code range
    wq, s, b = jq.quantize(torch.from_numpy(w).to(dev()), 64, bits, mode="rtn")
    pk, so, bo = jo.quantize_rtn(w, bits, 64)
    assert np.array_equal(to_np_u32(wq), pk)
    assert np.array_equal(f32(s), so) and np.array_equal(f32(b), bo)


@pytest.mark.parametrize("src", ("f32", "f16", "bf16"))
@pytest.mark.parametrize("bits", (2, 3, 4, 5, 6, 8))
def test_affine_division_forms_agree(bits, src):
    """The quantizer computes RN(t/scale) from the reciprocal and one exact residual; JQ_QUANT_IEEE_DIV selects
    the kernel that divides per weight instead.  The two return the same codes and sidecars on 16.8 M weights per
    case: gaussians over 24 orders of magnitude (7 for float16), integer grids (exact rounding ties in most groups), a large
    common offset, all-positive and all-negative groups, zero groups, and heavy tails."""
    g = torch.Generator(device=dev())
    g.manual_seed(17 * bits + len(src))
    R, K = 4096, 4096
    w = torch.randn((R, K), generator=g, device=dev())
    span = 8.0 if src == "f16" else 27.6                # float16 overflows at 65504
    w = w * torch.exp(torch.empty((R, 1), device=dev()).uniform_(-span, span, generator=g))
    w[100:400] = torch.randint(-40, 41, (300, K), generator=g, device=dev()).float() / 64
    w[400:500] = torch.randint(0, 1 << bits, (100, K), generator=g, device=dev()).float() * 0.125 - 0.5
    w[500:600] = 100.0 + torch.randn((100, K), generator=g, device=dev())
    w[600:700] = torch.rand((100, K), generator=g, device=dev()) + 0.01
    w[700:800] = -torch.rand((100, K), generator=g, device=dev()) - 0.01
    w[800:850] = 0.0
    w[850:950] = torch.randn((100, K), generator=g, device=dev()) ** 5
    w[950:1000] = torch.randn((50, K), generator=g, device=dev()) * (1e-9 if src != "f16" else 1e-6)
    if src != "f16":                                     # groups whose scale leaves the range of the residual form
        w[1000:1050] = torch.randn((50, K), generator=g, device=dev()) * 1e37
        w[1050:1100] = torch.randn((50, K), generator=g, device=dev()) * 1e-36
    wt = w.to(TORCH_DT[src])
    assert torch.isfinite(wt).all()
    for gs in (32, 64, 128):
        for mode in ("affine", "rtn"):
            # float32 sidecars: float16 ones overflow on the 1e37 rows and NaN != NaN
            a = jq.quantize(wt, gs, bits, mode=mode, sidecar_dtype=torch.float32)
            e = jq.quantize(wt, gs, bits, mode=mode + "_ieee_div", sidecar_dtype=torch.float32)
            for x, y in zip(a, e):
                assert torch.equal(x, y), (mode, gs)


@pytest.mark.parametrize("gs", (32, 64, 128))
@pytest.mark.parametrize("bits", (2, 3, 4, 6))
def test_mse_golden(golden_dir, bits, gs):
    """quantize_tensor(method="mse") vectors made by the reference (quantize.py:153-191)."""
    z = np.load(os.path.join(golden_dir, "mse_ref.npz"))
    wq, s, b = jq.quantize(torch.from_numpy(z["w"]).to(dev()), gs, bits, mode="mse")
    key = f"g{gs}_b{bits}"
    assert np.array_equal(to_np_u32(wq), z[key + "_packed"])
    assert np.array_equal(s.cpu().numpy(), z[key + "_scales"])
    assert np.array_equal(b.cpu().numpy(), z[key + "_biases"])


@pytest.mark.parametrize("mode", ("mse", "mse_exhaustive"))
@pytest.mark.parametrize("src", ("f32", "f16", "bf16"))
@pytest.mark.parametrize("gs", (32, 64, 128))
@pytest.mark.parametrize("bits", (2, 3, 4))
def test_mse_vs_oracle(bits, gs, src, mode):
    """Clip-ratio search against the oracle: codes and sidecars bit for bit, over magnitudes from 1e-3 to
    50, with constant and zero blocks, an outlier, and a row count that leaves the last warp and the last
    CTA partly empty."""
    rng = np.random.default_rng(100 * bits + gs)
    w = rng.standard_normal((37, 640)).astype(np.float32)
    w *= np.exp(rng.uniform(np.log(1e-3), np.log(50.0), size=(37, 1))).astype(np.float32)
    w[3, 128:256] = -0.125
    w[4, :128] = 0.0
    w[5, 77] = 300.0
    wt = torch.from_numpy(w).to(dev()).to(TORCH_DT[src])
    wq, s, b = jq.quantize(wt, gs, bits, mode=mode)
    pk, so, bo = jo.quantize_mse(f32(wt), bits, gs)
    assert np.array_equal(to_np_u32(wq), pk)
    assert np.array_equal(f32(s), so) and np.array_equal(f32(b), bo)
    assert s.dtype == torch.float16


@pytest.mark.parametrize("bits", (2, 3, 4))
def test_mse_screen_never_changes_the_winner(bits):
    """The float32 screen only discards clip ratios that cannot win: on 8.4 M weights of mixed character
    the screened search returns what the exhaustive float64 search returns.  The rows cover gaussians at
    magnitudes from 1e-12 to 1e12, blocks of few distinct values (where several ratios reconstruct almost
    exactly), a large common offset with a tiny spread (where float32 cannot tell the ratios apart),
    heavy tails, and magnitudes outside the screen's float32 range."""
    g = torch.Generator(device=dev())
    g.manual_seed(bits)
    R, K = 2048, 4096
    w = torch.randn((R, K), generator=g, device=dev())
    mag = torch.exp(torch.empty((R, 1), device=dev()).uniform_(-27.6, 27.6, generator=g))
    w = w * mag
    w[100:200] = torch.randint(0, 3, (100, K), generator=g, device=dev()).float() * 0.37 - 0.2
    w[200:300] = 1000.0 + torch.randn((100, K), generator=g, device=dev()) * 1e-4
    w[300:400] = torch.randn((100, K), generator=g, device=dev()) ** 5
    w[400:450] = torch.randn((50, K), generator=g, device=dev()) * 1e-25
    w[450:500] = torch.randn((50, K), generator=g, device=dev()) * 1e25
    w[500:600] = torch.randint(-8, 8, (100, K), generator=g, device=dev()).float() / 64
    for gs in (64, 128):
        a = jq.quantize(w, gs, bits, mode="mse")
        e = jq.quantize(w, gs, bits, mode="mse_exhaustive")
        for x, y in zip(a, e):
            assert torch.equal(x, y)


def test_mse_wide_codes_take_rtn():
    """quantize.py:153: above 4 bits the search is skipped."""
    rng = np.random.default_rng(9)
    w = torch.from_numpy((rng.standard_normal((16, 256)) * 0.02).astype(np.float32)).to(dev())
    for bits in (5, 6, 8):
        a = jq.quantize(w, 64, bits, mode="mse")
        r = jq.quantize(w, 64, bits, mode="rtn")
        assert all(torch.equal(x, y) for x, y in zip(a, r))


def test_mse_full_size_vs_oracle():
    """A 2048x4096 bf16 matrix at 2 bits: identical to the oracle, and the search lowers the error."""
    rng = np.random.default_rng(0)
    wt = torch.from_numpy((rng.standard_normal((2048, 4096)) * 0.02).astype(np.float32)).to(dev()).to(torch.bfloat16)
    wq, s, b = jq.quantize(wt, 64, 2, mode="mse")
    pk, so, bo = jo.quantize_mse(f32(wt), 2, 64)
    assert np.array_equal(to_np_u32(wq), pk)
    assert np.array_equal(f32(s), so) and np.array_equal(f32(b), bo)
    wr, sr, br = jq.quantize(wt, 64, 2, mode="rtn")
    e_mse = (jq.dequantize(wq, s, b, 64, 2, dtype=torch.float32) - wt.float()).square().mean().item()
    e_rtn = (jq.dequantize(wr, sr, br, 64, 2, dtype=torch.float32) - wt.float()).square().mean().item()
    assert e_mse < e_rtn


def test_config1_full_size_bit_exact():
    """BASELINE config 1: 4096x4096 N(0,0.02) seed 0, 4-bit, group 64, bf16."""
    rng = np.random.default_rng(0)
    w = (rng.standard_normal((4096, 4096)) * 0.02).astype(np.float32)
    wt = torch.from_numpy(w).to(dev()).to(torch.bfloat16)
    wq, s, b = jq.quantize(wt, 64, 4)
    pk, so, bo = jo.quantize_affine(f32(wt), 4, 64, src_dtype="bf16")
    assert np.array_equal(to_np_u32(wq), pk)
    assert np.array_equal(f32(s), so) and np.array_equal(f32(b), bo)
    # round trip: every weight is reproduced to within one quantization step (half a step from
    # rounding, up to one at the far edge that the upper clamp pulls in) plus sidecar rounding
    deq = jq.dequantize(wq, s, b, 64, 4, dtype=torch.float32)
    err = (deq - wt.float()).abs().reshape(4096, 64, 64)
    step = s.float().abs()[..., None]
    slack = 2.0 ** -8 * (15 * step + b.float().abs()[..., None])     # bf16 rounding of the stored sidecars
    assert bool((err <= 1.0 * step + slack).all())
    assert float((err <= 0.5 * step + slack).float().mean()) > 0.99


@pytest.mark.parametrize("bits", BITS)
def test_dequantize_dtypes(bits):
    rng = np.random.default_rng(11)
    w = torch.from_numpy((rng.standard_normal((32, 512)) * 0.02).astype(np.float32)).to(dev()).to(torch.bfloat16)
    wq, s, b = jq.quantize(w, 64, bits)
    ref = jo.dequantize_affine(to_np_u32(wq), f32(s), f32(b), bits, 64)
    assert np.array_equal(jq.dequantize(wq, s, b, 64, bits, dtype=torch.float32).cpu().numpy(), ref)
    assert np.array_equal(f32(jq.dequantize(wq, s, b, 64, bits)), jo.round_to(ref, "bf16"))
    assert np.array_equal(f32(jq.dequantize(wq, s, b, 64, bits, dtype=torch.float16)), jo.round_to(ref, "f16"))


def test_stacked_experts_and_empty():
    rng = np.random.default_rng(2)
    w = torch.from_numpy((rng.standard_normal((3, 16, 256)) * 0.02).astype(np.float32)).to(dev()).to(torch.float16)
    wq, s, b = jq.quantize(w, 64, 3)
    assert wq.shape == (3, 16, 24) and s.shape == (3, 16, 4)
    pk, so, bo = jo.quantize_affine(f32(w).reshape(48, 256), 3, 64, src_dtype="f16")
    assert np.array_equal(to_np_u32(wq).reshape(48, 24), pk)
    e = torch.empty((0, 128), dtype=torch.bfloat16, device=dev())
    wq, s, b = jq.quantize(e, 64, 4)
    assert wq.shape == (0, 16) and s.shape == (0, 2)


def test_shape_errors():
    w = torch.zeros((4, 100), dtype=torch.float16, device=dev())
    with pytest.raises(jq.JangqError, match="not divisible by group_size"):
        jq.quantize(w, 64, 4)
    with pytest.raises(jq.JangqError):
        jq.quantize(torch.zeros((4, 128), dtype=torch.float16, device=dev()), 64, 7)
    with pytest.raises(jq.JangqError):
        jq.quantize(torch.zeros((4, 128), dtype=torch.float16, device=dev()), 48, 4)


@pytest.mark.parametrize("bits", (2, 3, 4, 5, 6, 8))
@pytest.mark.parametrize("gs,dtype", ((64, torch.bfloat16), (128, torch.float16), (32, torch.float32)))
def test_embedding_rows_equal_dequantize(bits, gs, dtype):
    """Row lookup = the same rows of the full dequantization, bit for bit; ids of any shape, repeated ids,
    ids outside the table give zeros; the oracle's dequantizer agrees."""
    rows, K = 301, 512
    g = torch.Generator(device="cuda").manual_seed(bits * 7 + gs)
    w = (torch.randn((rows, K), device="cuda", generator=g) * 0.02).to(torch.bfloat16)
    sd = torch.bfloat16 if dtype == torch.float32 else dtype
    wq, s, b = jq.quantize(w.to(sd), gs, bits)
    full = jq.dequantize(wq, s, b, gs, bits, dtype=dtype)
    ids = torch.tensor([[0, 300, 17, 17], [5, -1, 301, 299]], device="cuda")
    out = jq.embedding(ids, wq, s, b, gs, bits, dtype=dtype)
    assert out.shape == (2, 4, K) and out.dtype == dtype
    valid = (ids >= 0) & (ids < rows)
    assert torch.equal(out[valid], full[ids[valid]])
    assert torch.count_nonzero(out[~valid]) == 0
    ref = jo.dequantize_affine(wq.cpu().numpy().view(np.uint32), s.float().cpu().numpy(), b.float().cpu().numpy(), bits, gs)
    assert np.array_equal(out[0, 1].float().cpu().numpy(), ref[300].astype(np.float32) if dtype == torch.float32
                          else torch.from_numpy(ref[300]).to(dtype).float().numpy())
    assert jq.embedding(torch.zeros((0,), dtype=torch.int64, device="cuda"), wq, s, b, gs, bits).shape == (0, K)


@pytest.mark.parametrize("gs", (32, 64, 128))
@pytest.mark.parametrize("bits", (2, 3, 4, 5, 6, 8))
def test_imatrix_fit_bit_exact_against_reference_vectors(golden_dir, bits, gs):
    """jq_quantize_imatrix against the reference's own outputs (tests/golden/imatrix_ref.npz): packed codes and
    float16 sidecars bit for bit, including the corner groups (all-zero, constant, outlier, exact grid,
    below the scale floor) and zero-importance columns."""
    z = np.load(os.path.join(golden_dir, "imatrix_ref.npz"))
    k = f"b{bits}_g{gs}"
    w = torch.from_numpy(z[k + "_w"]).cuda()
    wq, s, b = jq.quantize_imatrix(w, z[k + "_imp"], gs, bits)
    assert np.array_equal(wq.cpu().numpy().view(np.uint32), z[k + "_packed"])
    assert np.array_equal(s.cpu().numpy().view(np.uint16), z[k + "_scales"].view(np.uint16))
    assert np.array_equal(b.cpu().numpy().view(np.uint16), z[k + "_biases"].view(np.uint16))


def test_imatrix_fit_iterations_shapes_and_oracle(golden_dir):
    z = np.load(os.path.join(golden_dir, "imatrix_ref.npz"))
    wq, s, b = jq.quantize_imatrix(torch.from_numpy(z["it2_w"]).cuda(), z["it2_imp"], 64, 3, iterations=2)
    assert np.array_equal(wq.cpu().numpy().view(np.uint32), z["it2_packed"])
    assert np.array_equal(s.cpu().numpy(), z["it2_scales"]) and np.array_equal(b.cpu().numpy(), z["it2_biases"])
    # a larger seeded case against the oracle, stacked experts, a row count that leaves a partial block
    rng = np.random.default_rng(9)
    w = (rng.standard_normal((3, 37, 1024)) * 0.02).astype(np.float32)
    imp = (rng.standard_normal(1024) ** 2).astype(np.float32)
    wq, s, b = jq.quantize_imatrix(torch.from_numpy(w).cuda(), torch.from_numpy(imp).cuda(), 64, 4)
    pk, so, bo, _ = jo.quantize_imatrix_affine(w.reshape(-1, 1024), imp, 4, 64)
    assert wq.shape == (3, 37, 128) and s.shape == (3, 37, 16)
    assert np.array_equal(wq.cpu().numpy().view(np.uint32).reshape(pk.shape), pk)
    assert np.array_equal(s.cpu().numpy().reshape(so.shape), so) and np.array_equal(b.cpu().numpy().reshape(bo.shape), bo)
    # the fit lowers the importance-weighted error of the plain min/max quantizer
    wq0, s0, b0 = jq.quantize(torch.from_numpy(w).cuda().half(), 64, 4)
    d_fit = jq.dequantize(wq, s, b, 64, 4, dtype=torch.float32).cpu().numpy()
    d_mm = jq.dequantize(wq0, s0, b0, 64, 4, dtype=torch.float32).cpu().numpy()
    assert (imp * (d_fit - w) ** 2).sum() < (imp * (d_mm - w) ** 2).sum()
    with pytest.raises(jq.JangqError):
        jq.quantize_imatrix(torch.from_numpy(w).cuda(), imp[:-1], 64, 4)


@pytest.mark.parametrize("K", (64, 192, 4096, 11008, 14336))
def test_hadamard_rotation_matches_oracle_bit_for_bit(K):
    """The GPU butterflies do the float32 operations of the restated reference in the same order: equal bits
    in float32; bf16 input/output rounds once at the end; the rotation cancels in a rotated mat-vec."""
    rng = np.random.default_rng(K)
    x = rng.standard_normal((3, K)).astype(np.float32)
    s = jo.hadamard_signs(K, seed=42)
    ref = jo.hadamard_rotate(x, s)
    out = jq.hadamard_rotate(torch.from_numpy(x).cuda(), dtype=torch.float32)
    assert np.array_equal(out.cpu().numpy(), ref)
    assert np.array_equal(jq.hadamard_signs(K).cpu().numpy(), s)
    xb = torch.from_numpy(x).cuda().to(torch.bfloat16)
    outb = jq.hadamard_rotate(xb)
    refb = torch.from_numpy(jo.hadamard_rotate(xb.float().cpu().numpy(), s)).to(torch.bfloat16)
    assert outb.dtype == torch.bfloat16 and torch.equal(outb.cpu(), refb)
    # rotated weights, rotated input: the same product (a rotated bundle, loader.py:1763-1767)
    if K % 64 == 0 and K <= 4096:
        w = (rng.standard_normal((128, K)) * 0.02).astype(np.float32)
        wr = jq.hadamard_rotate(torch.from_numpy(w).cuda(), dtype=torch.float32)
        wq, sc, bi = jq.quantize(wr.to(torch.bfloat16), 64, 8)
        y = jq.quantized_matmul(jq.hadamard_rotate(xb), wq, sc, bi, group_size=64, bits=8).float().cpu().numpy()
        plain = xb.float().cpu().numpy() @ w.T
        assert np.abs(y - plain).max() <= 2e-2 * np.abs(plain).max()
