"""quantize_tensor / dequantize_tensor, the host mirror of jang_tools/quantize.py:211-337: argument checks on the
CPU, results on the GPU against the reference-made fixtures and the oracle."""
import os

import numpy as np
import pytest
import torch

import jangq_b200 as jq
from oracle import jang_oracle as jo


def test_block_count_mismatch_raises_like_the_reference():
    w = np.zeros((4, 100), np.float32)
    with pytest.raises(ValueError, match=r"bit_allocation has 6 blocks but weight has 400 values \(7 blocks at block_size=64\)"):
        jq.quantize_tensor(w, np.full(6, 4, np.uint8), 64)


def test_mixed_and_invalid_widths_raise():
    w = np.zeros((2, 128), np.float32)
    with pytest.raises(ValueError, match="uniform bit width"):
        jq.quantize_tensor(w, np.array([4, 4, 2, 4], np.uint8), 64)
    with pytest.raises(ValueError, match="Invalid bit width 7"):
        jq.quantize_tensor(w, np.full(4, 7, np.uint8), 64)
    with pytest.raises(ValueError, match="Invalid bit width 1"):
        jq.quantize_tensor(w, np.full(4, 1, np.uint8), 64)
    with pytest.raises(ValueError, match="unknown method"):
        jq.quantize_tensor(w, np.full(4, 4, np.uint8), 64, method="gptq")
    with pytest.raises(jq.JangqError):
        jq.quantize_tensor(w, np.full(16, 4, np.uint8), 16)


@pytest.mark.gpu
@pytest.mark.parametrize("bits", (2, 3, 4, 6, 8))
def test_rtn_fixture_through_the_mirror(golden_dir, bits):
    z = np.load(os.path.join(golden_dir, "rtn_ref.npz"))
    w = z["w"]
    qt = jq.quantize_tensor(w, np.full(w.size // 64, bits, np.uint8), block_size=64, method="rtn")
    assert isinstance(qt.qweight, np.ndarray) and qt.qweight.dtype == np.uint8 and qt.scales.dtype == np.float16
    assert qt.bits == bits and qt.shape == w.shape
    assert np.array_equal(qt.qweight.view(np.uint32).reshape(16, 256 * bits // 32), z[f"b{bits}_packed"])
    assert np.array_equal(qt.scales.reshape(16, 4), z[f"b{bits}_scales"])
    assert np.array_equal(qt.biases.reshape(16, 4), z[f"b{bits}_biases"])


@pytest.mark.gpu
@pytest.mark.parametrize("gs", (32, 64, 128))
@pytest.mark.parametrize("bits", (2, 3, 4, 6))
def test_default_method_is_the_clip_ratio_search(golden_dir, bits, gs):
    z = np.load(os.path.join(golden_dir, "mse_ref.npz"))
    w = z["w"]
    qt = jq.quantize_tensor(w, np.full(w.size // gs, bits, np.uint8), block_size=gs)
    key = f"g{gs}_b{bits}"
    assert np.array_equal(qt.qweight.view(np.uint32).reshape(24, 512 * bits // 32), z[key + "_packed"])
    assert np.array_equal(qt.scales.reshape(24, 512 // gs), z[key + "_scales"])
    assert np.array_equal(qt.biases.reshape(24, 512 // gs), z[key + "_biases"])


@pytest.mark.gpu
@pytest.mark.parametrize("method", ("rtn", "mse"))
def test_ragged_tail_3d_and_round_trip(method):
    """A [3, 5, 50] tensor: 750 weights = 11 full blocks and one of 46 weights padded with zeros; blocks straddle
    rows, exactly as the reference walks the flattened tensor.  CUDA tensors in, CUDA tensors out."""
    rng = np.random.default_rng(4)
    w = (rng.standard_normal((3, 5, 50)) * 0.05).astype(np.float32)
    n_blocks = (w.size + 63) // 64
    qt = jq.quantize_tensor(torch.from_numpy(w).cuda(), np.full(n_blocks, 3, np.uint8), 64, method=method)
    assert qt.qweight.is_cuda and qt.shape == (3, 5, 50)
    padded = np.concatenate([w.reshape(-1), np.zeros(n_blocks * 64 - w.size, np.float32)]).reshape(n_blocks, 64)
    pk, so, bo = (jo.quantize_rtn if method == "rtn" else jo.quantize_mse)(padded, 3, 64)
    assert np.array_equal(qt.qweight.cpu().numpy().view(np.uint32).reshape(n_blocks, 6), pk)
    assert np.array_equal(qt.scales.float().cpu().numpy(), so.reshape(-1))
    assert np.array_equal(qt.biases.float().cpu().numpy(), bo.reshape(-1))
    deq = jq.dequantize_tensor(qt, 64)
    ref = jo.dequantize_affine(pk, so, bo, 3, 64).reshape(-1)[:w.size].reshape(w.shape)
    assert deq.shape == (3, 5, 50) and np.array_equal(deq.cpu().numpy(), ref)
    # numpy in, numpy out
    qn = jq.quantize_tensor(w, np.full(n_blocks, 3, np.uint8), 64, method=method)
    assert np.array_equal(qn.qweight, qt.qweight.cpu().numpy())
    assert np.array_equal(jq.dequantize_tensor(qn, 64), ref)
