"""GPU parity of the prefill GEMM (jq_qgemm through quantized_matmul with many rows).

Gate (BASELINE north star, form of dots3/ops_selftest.py:48): max |y-ref| / max|ref| <= 1e-2 and
cosine >= 0.9999 against the f64 oracle.  The kernel feeds the tensor cores weights rounded once
to the activation type, so it is also held elementwise to that model of the arithmetic:
x . round(deq(W))^T in f64, within one output rounding step plus 1e-3 of max|ref|."""
import numpy as np
import pytest
import torch

import jangq_b200 as jq
from jangq_b200 import _lib
from oracle import jang_oracle as jo

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def make_case(M, N, K, bits, gs, dtype, seed=0):
    rng = np.random.default_rng(seed)
    w = torch.from_numpy((rng.standard_normal((N, K)) * 0.02).astype(np.float32)).to(DEV).to(dtype)
    x = torch.from_numpy(rng.standard_normal((M, K)).astype(np.float32)).to(DEV).to(dtype)
    wq, s, b = jq.quantize(w, gs, bits)
    return x, wq, s, b


def check(y, x, wq, s, b, bits, gs, dtype):
    name = "bf16" if dtype == torch.bfloat16 else "f16"
    xn = x.float().cpu().numpy().astype(np.float64)
    W = jo.dequantize_affine(wq.cpu().numpy().view(np.uint32), s.float().cpu().numpy(), b.float().cpu().numpy(),
                             bits, gs)
    ref = (xn @ W.astype(np.float64).T).astype(np.float32)
    ref_rounded = (xn @ jo.round_to(W, name).astype(np.float64).T).astype(np.float32)
    y = y.float().cpu().numpy()
    scale = np.abs(ref).max()
    assert np.abs(y - ref).max() / scale <= 1e-2
    cos = float((y.astype(np.float64) * ref).sum() / (np.linalg.norm(y.astype(np.float64)) * np.linalg.norm(ref)))
    assert cos >= 0.9999
    ulp = 2.0 ** -8 if dtype == torch.bfloat16 else 2.0 ** -11
    assert np.all(np.abs(y - ref_rounded) <= ulp * np.abs(ref_rounded) + 1e-3 * scale)


@pytest.mark.parametrize("gs", (32, 64, 128))
@pytest.mark.parametrize("bits", (2, 3, 4, 5, 6, 8))
def test_qgemm_bf16_all_widths(bits, gs):
    M, N, K = 160, 200, 512
    x, wq, s, b = make_case(M, N, K, bits, gs, torch.bfloat16, seed=bits * 10 + gs)
    y = jq.quantized_matmul(x, wq, s, b, group_size=gs, bits=bits)
    assert y.shape == (M, N) and y.dtype == torch.bfloat16
    check(y, x, wq, s, b, bits, gs, torch.bfloat16)


@pytest.mark.parametrize("bits", (2, 4, 8))
def test_qgemm_f16(bits):
    x, wq, s, b = make_case(64, 128, 256, bits, 64, torch.float16, seed=bits)
    y = jq.quantized_matmul(x, wq, s, b, group_size=64, bits=bits)
    check(y, x, wq, s, b, bits, 64, torch.float16)


@pytest.mark.parametrize("M,N,K", ((17, 128, 64), (128, 128, 1024), (129, 130, 192), (512, 384, 2048),
                                   (300, 1000, 768)))
def test_qgemm_shapes(M, N, K):
    """Single k-block, exact tiles, one-past-a-tile in M and N, rows whose byte length is not a
    multiple of 16 (the store falls back to scalars), several tiles in both directions."""
    x, wq, s, b = make_case(M, N, K, 4, 64, torch.bfloat16, seed=M + N)
    y = jq.quantized_matmul(x, wq, s, b, group_size=64, bits=4)
    check(y, x, wq, s, b, 4, 64, torch.bfloat16)


def test_qgemm_leading_dims_and_canaries():
    lib = _lib.load()
    M, N, K, bits, gs = 70, 136, 256, 6, 64
    x, wq, s, b = make_case(M, N, K, bits, gs, torch.bfloat16, seed=5)
    ldx, ldy = K + 8, N + 24
    xp = torch.full((M, ldx), 9.0, dtype=torch.bfloat16, device=DEV)
    xp[:, :K] = x
    yp = torch.full((M + 2, ldy), -3.0, dtype=torch.bfloat16, device=DEV)
    _lib.check(lib.jq_qgemm(xp.data_ptr(), _lib.JQ_BF16, M, ldx, wq.data_ptr(), s.data_ptr(), b.data_ptr(),
                            _lib.JQ_BF16, N, K, bits, gs, yp.data_ptr(), _lib.JQ_BF16, ldy, _lib.stream_ptr()))
    torch.cuda.synchronize()
    check(yp[:M, :N], x, wq, s, b, bits, gs, torch.bfloat16)
    assert bool((yp[:M, N:] == -3.0).all()) and bool((yp[M:] == -3.0).all())


def test_qgemm_matches_qgemv_rows():
    """The same activation row through both kernels: the GEMM only differs by the weight rounding."""
    x, wq, s, b = make_case(48, 256, 1024, 4, 64, torch.bfloat16, seed=77)
    y_gemm = jq.quantized_matmul(x, wq, s, b, group_size=64, bits=4).float()
    y_gemv = torch.cat([jq.quantized_matmul(x[i:i + 8], wq, s, b, group_size=64, bits=4) for i in range(0, 48, 8)])
    err = (y_gemm - y_gemv.float()).abs().max() / y_gemv.float().abs().max()
    assert float(err) < 1e-2


def test_qgemm_unsupported_row_lengths():
    """K % 64 != 0, or packed rows that are not a multiple of 16 bytes: the C entry point refuses,
    quantized_matmul falls back to the general mat-vec kernel and stays correct."""
    lib = _lib.load()
    for K, bits, gs in ((96, 4, 32), (64, 3, 64)):
        x, wq, s, b = make_case(40, 64, K, bits, gs, torch.bfloat16, seed=K)
        y = torch.empty((40, 64), dtype=torch.bfloat16, device=DEV)
        rc = lib.jq_qgemm(x.data_ptr(), _lib.JQ_BF16, 40, K, wq.data_ptr(), s.data_ptr(), b.data_ptr(), _lib.JQ_BF16,
                          64, K, bits, gs, y.data_ptr(), _lib.JQ_BF16, 64, _lib.stream_ptr())
        assert rc == _lib.JQ_EUNSUPPORTED
        y = jq.quantized_matmul(x, wq, s, b, group_size=gs, bits=bits)
        ref = jo.qmatmul(x.float().cpu().numpy(), wq.cpu().numpy().view(np.uint32), s.float().cpu().numpy(),
                         b.float().cpu().numpy(), bits, gs)
        assert np.abs(y.float().cpu().numpy() - ref).max() / np.abs(ref).max() <= 1e-2


def test_device_status_clean_after_gemm():
    torch.cuda.synchronize()
    assert _lib.load().jq_device_status() == 0


@pytest.mark.parametrize("gs", (64, 128))
@pytest.mark.parametrize("bits", (2, 3, 4, 5, 6, 8))
def test_qgemm_two_row_tiles_per_cta(bits, gs):
    """Shapes large enough for the two-accumulator form (256 rows of the activations per CTA): a ragged last
    row tile whose second half is empty, a ragged last column tile, every width and code-stage layout."""
    M, N, K = 1160, 7300, 384
    x, wq, s, b = make_case(M, N, K, bits, gs, torch.bfloat16, seed=bits + gs)
    y = jq.quantized_matmul(x, wq, s, b, group_size=gs, bits=bits)
    check(y, x, wq, s, b, bits, gs, torch.bfloat16)
    _lib.check(_lib.load().jq_device_status())


def test_qgemm_two_row_tiles_equal_one_row_tile_results():
    """The same rows through the one- and the two-accumulator form (a small N keeps one tile per CTA) are
    bit-identical: the accumulation order along K is the same."""
    M, K, bits, gs = 1024, 512, 4, 64
    x, wq, s, b = make_case(M, 8192, K, bits, gs, torch.bfloat16, seed=5)
    y2 = jq.quantized_matmul(x, wq, s, b, group_size=gs, bits=bits)                  # 32 x 4 CTAs: two tiles each
    y1 = jq.quantized_matmul(x, wq[:512].contiguous(), s[:512].contiguous(), b[:512].contiguous(), group_size=gs,
                             bits=bits)                                               # 2 x 8 CTAs: one tile each
    assert torch.equal(y2[:, :512], y1)


@pytest.mark.parametrize("bits", (2, 3, 4, 5, 6, 8))
@pytest.mark.parametrize("M,N,K,gs", ((200, 1000, 2048, 64), (130, 520, 4096, 128), (512, 4096, 4096, 64), (40, 300, 4480, 64)))
def test_qgemm_split_k_over_a_cluster(bits, M, N, K, gs):
    """Grids far below the SM count split K over a cluster of 2 or 4 CTAs whose accumulators meet in distributed
    shared memory: ragged rows and columns, K shares that are not equal (4480 = 70 k-blocks), every width."""
    if bits in (3, 5) and K % 128:
        K += 64
    x, wq, s, b = make_case(M, N, K, bits, gs, torch.bfloat16, seed=bits * 7 + M)
    y = jq.quantized_matmul(x, wq, s, b, group_size=gs, bits=bits)
    check(y, x, wq, s, b, bits, gs, torch.bfloat16)
    y2 = jq.quantized_matmul(x, wq, s, b, group_size=gs, bits=bits)
    assert torch.equal(y, y2)                                  # the partial sums are added in rank order
    _lib.check(_lib.load().jq_device_status())
