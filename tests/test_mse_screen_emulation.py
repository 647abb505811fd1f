"""CPU emulation of the clip-ratio search's float32 screen (quantize_mse_kernel): for every block the ratio that wins
the float64 search (jang_tools/quantize.py:163-185) must lie inside the window the screen keeps, i.e. its float32
root-mean-square error is at most rms_min * (1 + 1e-4) + 2^-16 * max|x|.  The emulation follows the kernel's float32
operations (reciprocal rounded from float64, magic-number rint, clamp, fused error) with numpy; it is the bound that
is under test, not bit equality with the device."""
import numpy as np
import pytest

from oracle import jang_oracle as jo

MAGIC = np.float32(12582912.0)


def _mse64(blk, bits):
    """[20, n_blocks] float64 mean squared errors exactly as the reference forms them, plus scale and zero point."""
    L = (1 << bits) - 1
    wmin, wmax = blk.min(axis=1), blk.max(axis=1)
    x = blk.astype(np.float64)
    out, scales, zeros = [], [], []
    for ratio in jo.MSE_CLIP_RATIOS:
        c_min, c_max = wmin.astype(np.float64) * ratio, wmax.astype(np.float64) * ratio
        c_range = c_max - c_min
        c_range[c_range == 0] = 1.0
        scale = c_range / L
        zero = np.clip(np.round(-c_min / scale), 0, L)
        q = np.clip(np.round(x / scale[:, None] + zero[:, None]), 0, L)
        err = x - (q - zero[:, None]) * scale[:, None]
        out.append(jo._sum_like_numpy(err * err) / blk.shape[1])
        scales.append(scale)
        zeros.append(zero)
    return np.array(out), np.array(scales), np.array(zeros)


def _mse32(blk, bits, scales, zeros):
    L = np.float32((1 << bits) - 1)
    out = []
    for scale64, zero in zip(scales, zeros):
        scale = scale64.astype(np.float32)[:, None]
        rcp = (1.0 / scale64).astype(np.float32)[:, None]
        z = zero.astype(np.float32)[:, None]
        r = ((blk.astype(np.float64) * rcp.astype(np.float64) + np.float64(MAGIC)).astype(np.float32) - MAGIC)
        c = np.minimum(np.maximum(r, -z), L - z)
        e = (blk.astype(np.float64) - c.astype(np.float64) * scale.astype(np.float64)).astype(np.float32)
        out.append((e.astype(np.float64) ** 2).sum(axis=1).astype(np.float32) / np.float32(blk.shape[1]))
    return np.array(out)


@pytest.mark.parametrize("bits", (2, 3, 4))
@pytest.mark.parametrize("gs", (32, 64, 128))
def test_screen_window_contains_the_float64_winner(bits, gs):
    rng = np.random.default_rng(1000 * bits + gs)
    n = 6000
    blk = rng.standard_normal((n, gs)).astype(np.float32)
    blk *= np.exp(rng.uniform(np.log(1e-12), np.log(1e12), size=(n, 1))).astype(np.float32)
    blk[100:400] = (rng.integers(0, 3, (300, gs)) * 0.37 - 0.2).astype(np.float32)        # few distinct values
    blk[400:700] = (1000.0 + rng.standard_normal((300, gs)) * 1e-4).astype(np.float32)    # offset >> spread
    blk[700:1000] = (rng.standard_normal((300, gs)) ** 5).astype(np.float32)              # heavy tails
    blk[1000:1300] = (rng.integers(-8, 8, (300, gs)) / 64).astype(np.float32)             # integer grid
    blk[1300:1600] = rng.standard_normal((300, gs)).astype(np.float16).astype(np.float32)
    keep = blk.max(axis=1) != blk.min(axis=1)
    blk = blk[keep]
    mse64, scales, zeros = _mse64(blk, bits)
    winner = np.argmin(mse64, axis=0)                      # first index of the minimum = the strict '<' winner
    mse32 = _mse32(blk, bits, scales, zeros)
    amax = np.abs(blk).max(axis=1)
    lim = np.sqrt(mse32.min(axis=0)) * np.float32(1.0001) + amax * np.float32(2.0 ** -16)
    thr = lim * lim * np.float32(1.00001)
    inside = mse32[winner, np.arange(blk.shape[0])] <= thr
    assert inside.all(), f"{(~inside).sum()} winners fall outside the screen's window"
    # the window is also selective: on plain gaussian blocks it keeps few of the 20 ratios
    kept = (mse32 <= thr[None, :]).sum(axis=0)
    assert np.median(kept[1600:]) <= 3
