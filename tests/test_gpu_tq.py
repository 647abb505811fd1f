"""GPU parity of the JANGTQ (rotated codebook) functor: quantizer, gather mat-vec, fused gate/up + SwiGLU and the
modules, against the CPU oracle.  Parity is unpinned for everything the reference runs through MLX (rotation,
norms, index choice); the codebooks are pinned.  Products are held to max |y-ref| / max|ref| <= 1e-2 and
cosine >= 0.9999 -- in practice they agree to float32 rounding, since both sides use the same indices."""
import numpy as np
import pytest
import torch

import jangq_b200 as jq
from jangq_b200 import _lib, turboquant as tq
from oracle import jang_oracle as jo

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def close(y, ref, tol=1e-2):
    y, ref = np.asarray(y, np.float64), np.asarray(ref, np.float64)
    assert np.abs(y - ref).max() / np.abs(ref).max() <= tol
    assert float((y * ref).sum() / (np.linalg.norm(y) * np.linalg.norm(ref))) >= 0.9999


@pytest.mark.parametrize("bits,N,K", ((2, 96, 2048), (3, 50, 640), (4, 33, 1024), (2, 40, 768)))
def test_quantizer_against_oracle(bits, N, K):
    """Indices may differ from the numpy walk only where a normalised weight sits within float32 rounding of a
    boundary (the row norm is summed in another order), and then by one step; norms agree to float16 rounding."""
    rng = np.random.default_rng(bits + N)
    w = (rng.standard_normal((N, K)) * 0.03).astype(np.float32)
    q = tq.tq_quantize_weight(torch.from_numpy(w).to(DEV), bits, seed=42)
    packed_ref, norms_ref, cb, signs = jo.tq_quantize(w, bits, seed=42)
    idx = jo.tq_unpack(q["packed"].cpu().numpy().view(np.uint32), bits, K).astype(np.int32)
    idx_ref = jo.tq_unpack(packed_ref, bits, K).astype(np.int32)
    diff = np.abs(idx - idx_ref)
    assert diff.max() <= 1 and (diff != 0).mean() <= 1e-3
    assert q["packed"].shape == packed_ref.shape
    nr = norms_ref.astype(np.float32)
    assert np.all(np.abs(q["norms"].float().cpu().numpy() - nr) <= 2.0 ** -10 * np.abs(nr) + 1e-8)
    if bits == 3:
        assert int((q["packed"].cpu().numpy().view(np.uint32) >> np.uint32(30)).max()) == 0


@pytest.mark.parametrize("bits", (2, 3, 4))
def test_gather_matmul_and_fused_swiglu(bits):
    E, I, H, T, k = 6, 200, 640, 3, 2
    rng = np.random.default_rng(bits)
    wg = torch.from_numpy((rng.standard_normal((E, I, H)) * 0.03).astype(np.float32)).to(DEV)
    wu = torch.from_numpy((rng.standard_normal((E, I, H)) * 0.03).astype(np.float32)).to(DEV)
    wd = torch.from_numpy((rng.standard_normal((E, H, I + 56)) * 0.03).astype(np.float32)).to(DEV)     # in = 256
    gate = tq.TurboQuantSwitchLinear.from_float(wg, bits)
    up = tq.TurboQuantSwitchLinear.from_float(wu, bits)
    down = tq.TurboQuantSwitchLinear.from_float(wd, bits)
    x = torch.from_numpy(rng.standard_normal((T, H)).astype(np.float32)).to(DEV)
    idx = torch.from_numpy(rng.integers(0, E, (T, k)).astype(np.int32)).to(DEV)

    def host(m):
        return (m.packed.cpu().numpy().view(np.uint32), m.norms.float().cpu().numpy(), m.codebook.cpu().numpy())

    x_rot = gate.rotate(x)
    xr_ref = jo.hadamard_rotate(x.cpu().numpy(), gate.signs.cpu().numpy())
    assert np.abs(x_rot.cpu().numpy() - xr_ref).max() <= 1e-5 * np.abs(xr_ref).max()
    pg, ng, cb = host(gate)
    pu, nu, _ = host(up)
    for lim in (0.0, 0.05):
        act = tq.tq_fused_gate_up_swiglu(x_rot, gate, up, idx, lim)
        ref = jo.tq_fused_gate_up_swiglu(xr_ref, pg, ng, pu, nu, cb, idx.cpu().numpy(), bits, k, lim)
        assert act.shape == (T * k, I)
        close(act.cpu().numpy(), ref)
    # the module call shapes: [T, in] with idx [T, k], and one row per pair
    y = gate(x, idx)
    assert y.shape == (T, k, I)
    close(y.float().cpu().numpy().reshape(T * k, I), jo.tq_gather_matmul(xr_ref, pg, ng, cb, idx.cpu().numpy(), bits, k))
    h = torch.from_numpy(rng.standard_normal((T * k, I + 56)).astype(np.float32)).to(DEV)
    pd, nd, cbd = host(down)
    yd = down(h, idx.reshape(-1))
    hr_ref = jo.hadamard_rotate(h.cpu().numpy(), down.signs.cpu().numpy())
    close(yd.float().cpu().numpy(), jo.tq_gather_matmul(hr_ref, pd, nd, cbd, idx.cpu().numpy().reshape(-1), bits, 1))
    # an expert outside the bank yields zero rows
    bad = torch.tensor([[0, E + 3]], dtype=torch.int32, device=DEV)
    yb = tq.tq_gather_matmul(x_rot[:1], gate.packed, gate.norms, gate.codebook, bad, bits, x_div=2)
    assert torch.count_nonzero(yb[1]) == 0 and torch.count_nonzero(yb[0]) > 0


@pytest.mark.parametrize("bits", (2, 4))
def test_linear_module_equals_the_derotated_product(bits):
    """TurboQuantLinear.forward (rotate x, codebook mat-vec) against x @ W^T with W the de-rotated float matrix
    the reference's module builds (linear.py:51-56)."""
    N, K = 130, 1024
    rng = np.random.default_rng(9)
    w = torch.from_numpy((rng.standard_normal((N, K)) * 0.03).astype(np.float32)).to(DEV)
    lin = tq.TurboQuantLinear.from_float(w, bits)
    x = torch.from_numpy(rng.standard_normal((5, K)).astype(np.float32)).to(DEV)
    y = lin(x)
    W = jo.tq_dequantize(lin.packed.cpu().numpy().view(np.uint32), lin.norms.float().cpu().numpy(),
                         lin.codebook.cpu().numpy(), lin.signs.cpu().numpy(), bits)
    ref = x.cpu().numpy().astype(np.float64) @ W.astype(np.float64).T
    close(y.cpu().numpy(), ref, tol=1e-3)
    assert abs(float(np.abs(W - w.cpu().numpy()).max())) < 0.2


def test_tq_argument_checks():
    lib = _lib.load()
    z = torch.zeros(64, dtype=torch.float32, device=DEV)
    rc = lib.jq_tq_gather_matmul(z.data_ptr(), 64, 1, None, 1, z.data_ptr(), z.data_ptr(), z.data_ptr(), 1, 4, 64, 5,
                                 z.data_ptr(), 4, None)
    assert rc == _lib.JQ_EUNSUPPORTED
    rc = lib.jq_tq_gather_matmul(z.data_ptr(), 32, 1, None, 1, z.data_ptr(), z.data_ptr(), z.data_ptr(), 1, 4, 64, 2,
                                 z.data_ptr(), 4, None)
    assert rc == _lib.JQ_EINVAL
