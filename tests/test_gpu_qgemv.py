"""GPU parity of the decode mat-vec (jq_qgemv through quantized_matmul) against
the CPU oracle.  Tolerance (BASELINE north star): max |y-ref| / max|ref| <= 1e-2
and cosine >= 0.9999; the tensor-core path is additionally held to an
elementwise bound of one output rounding step plus 2e-3 of max|ref|."""
import ctypes
import os

import numpy as np
import pytest
import torch

import jangq_b200 as jq
from jangq_b200 import _lib
from oracle import jang_oracle as jo

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def make_case(N, K, bits, gs, M, dtype, seed=0):
    rng = np.random.default_rng(seed)
    w = torch.from_numpy((rng.standard_normal((N, K)) * 0.02).astype(np.float32)).to(DEV).to(dtype)
    x = torch.from_numpy(rng.standard_normal((M, K)).astype(np.float32)).to(DEV).to(dtype)
    wq, s, b = jq.quantize(w, gs, bits)
    return x, wq, s, b


def reference(x, wq, s, b, bits, gs):
    return jo.qmatmul(x.float().cpu().numpy(), wq.cpu().numpy().view(np.uint32), s.float().cpu().numpy(),
                      b.float().cpu().numpy(), bits, gs)


def check(y, ref, dtype, tight=True):
    y = y.float().cpu().numpy()
    scale = np.abs(ref).max()
    assert np.abs(y - ref).max() / scale <= 1e-2
    cos = float((y * ref).sum() / (np.linalg.norm(y) * np.linalg.norm(ref)))
    assert cos >= 0.9999
    if tight:
        ulp = 2.0 ** -8 if dtype == torch.bfloat16 else 2.0 ** -11
        assert np.all(np.abs(y - ref) <= ulp * np.abs(ref) + 2e-3 * scale)


@pytest.mark.parametrize("M", (1, 3, 8, 13))
@pytest.mark.parametrize("gs", (64, 128))
@pytest.mark.parametrize("bits", (2, 3, 4, 5, 6, 8))
def test_qgemv_bf16(bits, gs, M):
    x, wq, s, b = make_case(176, 2048, bits, gs, M, torch.bfloat16, seed=bits + gs + M)
    y = jq.quantized_matmul(x, wq, s, b, group_size=gs, bits=bits)
    assert y.shape == (M, 176) and y.dtype == torch.bfloat16
    check(y, reference(x, wq, s, b, bits, gs), torch.bfloat16)


@pytest.mark.parametrize("bits", (2, 3, 4, 6, 8))
def test_qgemv_f16(bits):
    x, wq, s, b = make_case(96, 1024, bits, 64, 2, torch.float16, seed=bits)
    y = jq.quantized_matmul(x, wq, s, b, group_size=64, bits=bits)
    check(y, reference(x, wq, s, b, bits, 64), torch.float16)


@pytest.mark.parametrize("N,K", ((50, 1472), (1, 64), (17, 11008), (333, 768), (16, 8192)))
@pytest.mark.parametrize("bits", (2, 3, 4, 6, 8))
def test_qgemv_ragged_shapes(bits, N, K):
    """Row counts that are not a multiple of the 16-row tile, K that is not a
    multiple of the stage length, single-group rows; 3-bit rows whose pitch is not
    16-byte aligned take the general kernel."""
    x, wq, s, b = make_case(N, K, bits, 64, 2, torch.bfloat16, seed=N + K)
    y = jq.quantized_matmul(x, wq, s, b, group_size=64, bits=bits)
    check(y, reference(x, wq, s, b, bits, 64), torch.bfloat16)


@pytest.mark.parametrize("bits", (2, 4, 5, 8))
def test_qgemv_group32_general_kernel(bits):
    x, wq, s, b = make_case(40, 512, bits, 32, 3, torch.bfloat16, seed=9)
    y = jq.quantized_matmul(x, wq, s, b, group_size=32, bits=bits)
    check(y, reference(x, wq, s, b, bits, 32), torch.bfloat16)


def test_qgemv_mixed_sidecar_dtype_general_kernel():
    x, wq, s, b = make_case(64, 512, 4, 64, 1, torch.bfloat16, seed=4)
    s16, b16 = s.to(torch.float16), b.to(torch.float16)
    y = jq.quantized_matmul(x, wq, s16, b16, group_size=64, bits=4)
    check(y, reference(x, wq, s16, b16, 4, 64), torch.bfloat16)


def test_qgemv_config1_full_size():
    """BASELINE config 1: y = W.x for the 4096x4096 4-bit group-64 tensor, batch 1."""
    x, wq, s, b = make_case(4096, 4096, 4, 64, 1, torch.bfloat16, seed=0)
    y = jq.quantized_matmul(x, wq, s, b, group_size=64, bits=4)
    check(y, reference(x, wq, s, b, 4, 64), torch.bfloat16)
    # linearity in x at full size: W.(2x) == 2 W.x exactly (power-of-two scaling)
    y2 = jq.quantized_matmul(x * 2, wq, s, b, group_size=64, bits=4)
    assert torch.equal(y2, y * 2)


def test_qgemv_leading_dimensions_and_canaries():
    """Call the C ABI directly with ldx/ldy larger than the row length; the
    padding must come back untouched."""
    lib = _lib.load()
    N, K, M, bits, gs = 70, 1024, 3, 4, 64
    x, wq, s, b = make_case(N, K, bits, gs, M, torch.bfloat16, seed=21)
    ldx, ldy = K + 64, N + 10
    xp = torch.full((M, ldx), 7.0, dtype=torch.bfloat16, device=DEV)
    xp[:, :K] = x
    yp = torch.full((M + 1, ldy), -3.0, dtype=torch.bfloat16, device=DEV)
    rc = lib.jq_qgemv(xp.data_ptr(), _lib.JQ_BF16, M, ldx, wq.data_ptr(), s.data_ptr(), b.data_ptr(), _lib.JQ_BF16,
                      N, K, bits, gs, yp.data_ptr(), _lib.JQ_BF16, ldy, _lib.stream_ptr())
    _lib.check(rc)
    torch.cuda.synchronize()
    check(yp[:M, :N], reference(x, wq, s, b, bits, gs), torch.bfloat16)
    assert bool((yp[:M, N:] == -3.0).all()) and bool((yp[M] == -3.0).all())


def test_general_kernel_matches_on_standard_shape():
    x, wq, s, b = make_case(128, 1024, 6, 64, 4, torch.bfloat16, seed=6)
    ref = reference(x, wq, s, b, 6, 64)
    os.environ["JANGQ_FORCE_SIMPLE_GEMV"] = "1"
    try:
        y = jq.quantized_matmul(x, wq, s, b, group_size=64, bits=6)
    finally:
        os.environ.pop("JANGQ_FORCE_SIMPLE_GEMV")
    check(y, ref, torch.bfloat16)


def test_device_status_clean():
    torch.cuda.synchronize()
    assert _lib.load().jq_device_status() == 0


def test_static_weights_overlapped_launches_keep_stream_order():
    """JQ_GEMV_STATIC_WEIGHTS lets a launch start before its predecessor has finished; the
    activations it reads (the predecessor's output) must still be the finished ones."""
    from jangq_b200.ops import _qgemv
    N = 1024
    lins = []
    for i in range(4):
        _, wq, s, b = make_case(N, N, (2, 4, 6, 8)[i], 64, 1, torch.bfloat16, seed=40 + i)
        lins.append((wq, s * 8, b * 8, (2, 4, 6, 8)[i]))      # gain ~1 so that the chain neither dies nor blows up
    x0 = torch.randn((1, N), device=DEV).to(torch.bfloat16)

    def chain(flags):
        bufs = [x0] + [torch.empty((1, N), dtype=torch.bfloat16, device=DEV) for _ in range(8)]
        for rep in range(8):
            wq, s, b, bits = lins[rep % 4]
            _qgemv(bufs[rep], wq, s, b, N, bits, 64, bufs[rep + 1], flags)
        torch.cuda.synchronize()
        return bufs[-1]

    ref = chain(0)
    for _ in range(5):
        assert torch.equal(chain(_lib.JQ_GEMV_STATIC_WEIGHTS), ref)
    assert float(ref.float().abs().max()) > 0


# ---- fused launches (jq_qgemv_batched_ex): several matrices over the same activations -----------------------
@pytest.mark.parametrize("M", (1, 3))
@pytest.mark.parametrize("bits", (2, 4, 6, 8))
def test_fused_matches_oracle_and_single_calls(bits, M):
    """q/k/v-like: three matrices of different row counts (one ragged) in one call; every output must
    match the oracle and agree with the single-matrix call to an output rounding step (the split of K over
    clusters and warps, hence the f32 summation order, depends on the size of the launch)."""
    from jangq_b200.ops import qgemv_fused
    K, gs = 1024, 64
    x = None
    lins, refs = [], []
    for i, N in enumerate((384, 200, 128)):
        xi, wq, s, b = make_case(N, K, bits, gs, M, torch.bfloat16, seed=10 + i)
        x = xi if x is None else x
        lin = jq.JANGLinear(K, N, bits, gs, dtype=torch.bfloat16, device=DEV)
        lin.weight.copy_(wq); lin.scales.copy_(s); lin.biases.copy_(b)
        lins.append(lin)
        refs.append(reference(x, wq, s, b, bits, gs))
    outs = [torch.full((M, l.out_features), float("nan"), dtype=torch.bfloat16, device=DEV) for l in lins]
    qgemv_fused(x, lins, outs)
    torch.cuda.synchronize()
    for lin, out, ref in zip(lins, outs, refs):
        check(out, ref, torch.bfloat16)
        single = jq.quantized_matmul(x, lin.weight, lin.scales, lin.biases, group_size=gs, bits=bits)
        assert (single.float() - out.float()).abs().max() <= 2.0 ** -7 * out.float().abs().max()


def test_fused_mixed_widths_split_into_runs():
    """Entries whose width or K differ cannot share a launch: the call must still compute all of them."""
    from jangq_b200.ops import qgemv_fused
    gs, M = 64, 1
    lins, refs, x = [], [], None
    for i, (N, bits) in enumerate(((256, 8), (256, 8), (192, 2), (128, 4), (128, 4))):
        xi, wq, s, b = make_case(N, 512, bits, gs, M, torch.bfloat16, seed=30 + i)
        x = xi if x is None else x
        lin = jq.JANGLinear(512, N, bits, gs, dtype=torch.bfloat16, device=DEV)
        lin.weight.copy_(wq); lin.scales.copy_(s); lin.biases.copy_(b)
        lins.append(lin)
        refs.append(reference(x, wq, s, b, bits, gs))
    outs = [torch.empty((M, l.out_features), dtype=torch.bfloat16, device=DEV) for l in lins]
    qgemv_fused(x, lins, outs, _lib.JQ_GEMV_STATIC_WEIGHTS)
    torch.cuda.synchronize()
    for out, ref in zip(outs, refs):
        check(out, ref, torch.bfloat16)


def test_plan_groups_fuse_and_match_ungrouped():
    """GemvPlan with groups (q/k/v fused, o alone) replays to the outputs of the ungrouped plan (to one
    output rounding step: the summation order depends on the launch size)."""
    torch.manual_seed(3)
    lins = [jq.JANGLinear.from_float((torch.randn(n, 1024, device=DEV) * 0.02).to(torch.bfloat16), bits=b, group_size=64)
            for n, b in ((256, 8), (256, 8), (128, 8), (256, 8), (512, 2), (512, 2))]
    xin = torch.randn(1, 1024, device=DEV).to(torch.bfloat16)
    plans = [jq.GemvPlan(lins, m=1, device=DEV), jq.GemvPlan(lins, m=1, device=DEV, groups=[[0, 1, 2], [3], [4, 5]])]
    assert plans[0].launches_per_run == 6 and plans[1].launches_per_run == 3
    outs = []
    for p in plans:
        for buf in p._xbuf.values():
            buf.copy_(xin)
        p.capture()
        p.run()
        torch.cuda.synchronize()
        outs.append([y.clone() for y in p.y])
    for a, b in zip(*outs):
        assert (a.float() - b.float()).abs().max() <= 2.0 ** -7 * a.float().abs().max()
    _lib.check(_lib.load().jq_device_status())


# ---- every fast kernel, selected explicitly ------------------------------------------------------------------
@pytest.mark.parametrize("kernel", ("tc", "mma", "pint", "one"))
@pytest.mark.parametrize("bits,N,K,M", ((8, 4096, 4096, 1), (2, 5000, 4096, 1), (4, 300, 11008, 2), (8, 130, 2048, 2),
                                        (2, 96, 512, 1), (4, 4100, 1024, 1), (2, 4096, 11008, 2)))
def test_each_kernel_against_oracle(monkeypatch, kernel, bits, N, K, M):
    """The dispatcher picks a kernel per shape from measurements; JANGQ_GEMV_KERNEL forces one (where the
    shape fits it), so every kernel is checked on shapes it would not get by default: ragged row blocks,
    K split over clusters, rows longer than one ring."""
    monkeypatch.setenv("JANGQ_GEMV_KERNEL", kernel)
    x, wq, s, b = make_case(N, K, bits, 64, M, torch.bfloat16, seed=bits + N + M)
    y = jq.quantized_matmul(x, wq, s, b, group_size=64, bits=bits)
    check(y, reference(x, wq, s, b, bits, 64), torch.bfloat16)
    _lib.check(_lib.load().jq_device_status())


# ---- the launches of the benchmarked decode stream, at their real sizes ----------------------------------------
@pytest.mark.parametrize("names,N,K,bits", ((("q", "k", "v"), 4096, 4096, 8), (("gate", "up"), 11008, 4096, 2),
                                            (("down",), 4096, 11008, 2), (("lm_head",), 32000, 4096, 6)))
def test_bench_stream_launches_against_oracle(names, N, K, bits):
    """The fused launches bench.py times (q/k/v 3 x 4096x4096 @8-bit and gate/up 2 x 11008x4096 @2-bit as one
    jq_qgemv_batched_ex call each, down 4096x11008 @2-bit, lm_head 32000x4096 @6-bit; one activation row) on
    the default kernel choice, against the f64 oracle."""
    from jangq_b200.ops import qgemv_fused
    torch.manual_seed(len(names) * 100 + bits)
    lins = [jq.JANGLinear.from_float((torch.randn(N, K, device=DEV) * 0.02).to(torch.bfloat16), bits=bits, group_size=64)
            for _ in names]
    x = torch.randn(1, K, device=DEV).to(torch.bfloat16)
    outs = [torch.empty((1, N), dtype=torch.bfloat16, device=DEV) for _ in names]
    qgemv_fused(x, lins, outs, _lib.JQ_GEMV_STATIC_WEIGHTS)
    torch.cuda.synchronize()
    for lin, out in zip(lins, outs):
        check(out, reference(x, lin.weight, lin.scales, lin.biases, bits, 64), torch.bfloat16)
    _lib.check(_lib.load().jq_device_status())


@pytest.mark.parametrize("kernel", ("pint", "tc", "mma", "one"))
@pytest.mark.parametrize("bits", (2, 4, 8))
def test_wide_dynamic_range_group(monkeypatch, kernel, bits):
    """One 1e4 outlier among N(0,1) activations in a group: the integer kernels cut the group's activations to
    24-bit fixed point under one shared exponent, so the small ones keep 2^-22 of the outlier (about 2e-3
    absolute) -- float32-accumulation grade.  Held to the same bar as every other case."""
    monkeypatch.setenv("JANGQ_GEMV_KERNEL", kernel)
    x, wq, s, b = make_case(512, 2048, bits, 64, 2, torch.bfloat16, seed=40 + bits)
    x[0, 70] = 1.0e4
    x[1, 1999] = -3.0e4
    y = jq.quantized_matmul(x, wq, s, b, group_size=64, bits=bits)
    check(y, reference(x, wq, s, b, bits, 64), torch.bfloat16)
    _lib.check(_lib.load().jq_device_status())


def test_nonfinite_activation_poisons_only_its_outputs(monkeypatch):
    """An infinite activation must not turn into a finite garbage value: the integer kernels mark the group's
    exponent NaN, so every output row of that activation row is NaN, the other activation row is untouched."""
    for kernel, bits in (("tc", 8), ("pint", 8), ("pint", 4), ("pint", 2)):
        monkeypatch.setenv("JANGQ_GEMV_KERNEL", kernel)
        x, wq, s, b = make_case(256, 1024, bits, 64, 2, torch.bfloat16, seed=5)
        ref = reference(x, wq, s, b, bits, 64)
        x[1, 77] = float("inf")
        y = jq.quantized_matmul(x, wq, s, b, group_size=64, bits=bits).float().cpu().numpy()
        assert np.all(np.isnan(y[1]))
        assert np.abs(y[0] - ref[0]).max() <= 1e-2 * np.abs(ref[0]).max()
    # the one-row integer kernel (the default for a single activation row): every output becomes NaN
    for bits in (2, 4, 6, 8):
        monkeypatch.setenv("JANGQ_GEMV_KERNEL", "one")
        x, wq, s, b = make_case(256, 1024, bits, 64, 1, torch.bfloat16, seed=6)
        x[0, 300] = float("-inf")
        y = jq.quantized_matmul(x, wq, s, b, group_size=64, bits=bits).float().cpu().numpy()
        assert np.all(np.isnan(y))


@pytest.mark.parametrize("bits,gs", ((2, 64), (2, 128), (3, 64), (3, 128), (4, 64), (4, 128), (6, 64), (6, 128), (8, 64),
                                     (8, 128)))
def test_one_row_integer_kernel_shapes_and_extremes(monkeypatch, bits, gs):
    """The item-streaming integer kernel (one activation row): ragged row counts, rows shorter than one
    256-byte stage, rows whose last stage is short, a fused launch of three matrices, largest codes against
    largest limbs, f16."""
    from jangq_b200.ops import qgemv_fused
    monkeypatch.setenv("JANGQ_GEMV_KERNEL", "one")
    for N, K in ((333, 2048), (17, 256), (5000, 1280), (40, 11008)):
        if K % (4 * gs):
            continue
        x, wq, s, b = make_case(N, K, bits, gs, 1, torch.bfloat16, seed=bits + gs + N)
        check(jq.quantized_matmul(x, wq, s, b, group_size=gs, bits=bits), reference(x, wq, s, b, bits, gs), torch.bfloat16)
    for dtype in (torch.bfloat16, torch.float16):
        g = torch.Generator(device="cuda").manual_seed(bits * 131 + gs)
        w = (torch.rand(333, 2048, device="cuda", generator=g) > 0.2).to(dtype)
        w[:, ::gs] = 0
        wq, s, b = jq.quantize(w, group_size=gs, bits=bits)
        x = torch.full((1, 2048), 1.9921875, device="cuda", dtype=dtype)
        check(jq.quantized_matmul(x, wq, s, b, group_size=gs, bits=bits), reference(x, wq, s, b, bits, gs), dtype)
    lins = [jq.JANGLinear.from_float((torch.randn(n, 1024, device=DEV) * 0.02).to(torch.bfloat16), bits=bits, group_size=gs)
            for n in (96, 33, 2500)]
    x = torch.randn(1, 1024, device=DEV).to(torch.bfloat16)
    outs = [torch.empty((1, l.out_features), dtype=torch.bfloat16, device=DEV) for l in lins]
    qgemv_fused(x, lins, outs, _lib.JQ_GEMV_STATIC_WEIGHTS)
    torch.cuda.synchronize()
    for lin, out in zip(lins, outs):
        check(out, reference(x, lin.weight, lin.scales, lin.biases, bits, gs), torch.bfloat16)
    _lib.check(_lib.load().jq_device_status())


@pytest.mark.parametrize("bits,gs", ((2, 64), (2, 128), (4, 64), (4, 128), (8, 64), (8, 128)))
def test_persistent_integer_kernel_extremes(monkeypatch, bits, gs):
    """Largest codes against largest limbs (every code the maximum in most positions, every activation the
    same value just under a power of two), a fused launch of two matrices with ragged row counts, and f16."""
    monkeypatch.setenv("JANGQ_GEMV_KERNEL", "pint")
    K = 2048
    for dtype in (torch.bfloat16, torch.float16):
        g = torch.Generator(device="cuda").manual_seed(bits * 131 + gs)
        w = (torch.rand(333, K, device="cuda", generator=g) > 0.2).to(dtype)
        w[:, ::gs] = 0
        wq, s, b = jq.quantize(w, group_size=gs, bits=bits)
        x = torch.full((1, K), 1.9921875, device="cuda", dtype=dtype)
        y = jq.quantized_matmul(x, wq, s, b, group_size=gs, bits=bits)
        check(y, reference(x, wq, s, b, bits, gs), dtype)
    _lib.check(_lib.load().jq_device_status())


def test_modules_loaded_from_a_reference_bundle():
    """A bundle written by the reference's writer (tests/golden/bundle_v2) loads into JANGLinear / ExpertBank
    with the widths inferred from the shapes, and the modules compute what the oracle computes from the files."""
    import os
    from jangq_b200 import bundle as B, moe
    gold = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "bundle_v2")
    mods = B.load_modules(gold, device=DEV)
    b = B.open_bundle(gold)
    rng = np.random.default_rng(3)
    for name in ("model.layers.0.self_attn.q_proj", "model.layers.0.mlp.gate_proj", "lm_head"):
        lin = mods[name]
        spec = b.quant_spec(name)
        assert (lin.bits, lin.group_size) == (spec.bits, spec.group_size)
        x = torch.from_numpy(rng.standard_normal((2, lin.in_features)).astype(np.float32)).to(DEV).to(torch.float16)
        y = lin(x)
        ref = jo.qmatmul(x.float().cpu().numpy(), b.tensor(name + ".weight"), b.tensor(name + ".scales").astype(np.float32),
                         b.tensor(name + ".biases").astype(np.float32), spec.bits, spec.group_size)
        check(y, ref, torch.float16)
    bank = mods["model.layers.0.mlp.switch_mlp.up_proj"]
    assert isinstance(bank, moe.ExpertBank) and bank.expert_bits == [3] * 4 and (bank.E, bank.N, bank.K) == (4, 16, 128)
    b.close()


@pytest.mark.parametrize("bits,K,k,shapes", ((6, 2048, 8, (4096, 512, 512)), (8, 4096, 1, (256,)), (2, 1024, 3, (300, 100)),
                                             (4, 768, 8, (64,)), (3, 1024, 4, (128, 128)), (8, 2048, 16, (1000,))))
@pytest.mark.parametrize("dtype", (torch.bfloat16, torch.float16))
def test_row_formed_in_the_launch_as_residual_rmsnorm(bits, K, k, shapes, dtype):
    """jq_qgemv_batched_norm: x = rms_norm(res + sum of k rows) formed inside the mat-vec launch equals the separate
    norm launch to one rounding step of the activation type, and the products match the oracle applied to the row
    the launch stored; 3-bit takes the two-launch route."""
    from jangq_b200.ops import qgemv_fused_norm
    from jangq_b200.moe import residual_rmsnorm
    rng = np.random.default_rng(bits * 100 + k)
    res = torch.from_numpy(rng.standard_normal((1, K)).astype(np.float32)).to(DEV).to(dtype)
    y = torch.from_numpy(rng.standard_normal((k, K)).astype(np.float32) * 0.5).to(DEV).to(dtype)
    lins = []
    for i, N in enumerate(shapes):
        _, wq, s, b = make_case(N, K, bits, 64, 1, dtype, seed=400 + i)
        lin = jq.JANGLinear(K, N, bits, 64, dtype=dtype, device=DEV)
        lin.weight.copy_(wq); lin.scales.copy_(s); lin.biases.copy_(b)
        lins.append(lin)
    outs = [torch.full((1, n), float("nan"), dtype=dtype, device=DEV) for n in shapes]
    x = qgemv_fused_norm(res, y, k, lins, outs, _lib.JQ_GEMV_STATIC_WEIGHTS)
    want = residual_rmsnorm(res, y, k=k)
    torch.cuda.synchronize()
    ulp = 2.0 ** -7 if dtype == torch.bfloat16 else 2.0 ** -10
    assert ((x.float() - want.float()).abs() <= ulp * want.float().abs() + 1e-6).all()
    v = res.float().cpu().numpy().astype(np.float64) + y.float().cpu().numpy().astype(np.float64).sum(0, keepdims=True)
    ref_x = v / np.sqrt((v * v).mean() + float(torch.finfo(dtype).eps))
    assert np.abs(x.float().cpu().numpy() - ref_x).max() <= 2 * ulp * np.abs(ref_x).max()
    for lin, out in zip(lins, outs):
        check(out, reference(x, lin.weight, lin.scales, lin.biases, bits, 64), dtype)
    _lib.check(_lib.load().jq_device_status())


def test_row_formed_in_the_launch_validation():
    lib = _lib.load()
    K = 1024
    _, wq, s, b = make_case(64, K, 4, 64, 1, torch.bfloat16)
    res = torch.zeros((1, K), dtype=torch.bfloat16, device=DEV)
    y = torch.zeros((2, K), dtype=torch.bfloat16, device=DEV)
    x = torch.zeros((1, K), dtype=torch.bfloat16, device=DEV)
    out = torch.zeros((1, 64), dtype=torch.bfloat16, device=DEV)
    d = (_lib.JqGemvDesc * 1)()
    d[0].x, d[0].codes, d[0].scales, d[0].biases, d[0].y = x.data_ptr(), wq.data_ptr(), s.data_ptr(), b.data_ptr(), out.data_ptr()
    d[0].N, d[0].K, d[0].ldx, d[0].ldy, d[0].bits, d[0].group_size = 64, K, K, 64, 4, 64

    def call(xo, yy=y, ldy=K):
        return lib.jq_qgemv_batched_norm(res.data_ptr(), yy.data_ptr(), ldy, 2, 1e-6, xo, d, 1, _lib.JQ_BF16, _lib.JQ_BF16, 0,
                                         _lib.stream_ptr())

    assert call(x.data_ptr()) == _lib.JQ_OK
    assert call(res.data_ptr()) == _lib.JQ_EINVAL            # entries do not read x_out / aliasing
    d[0].x = res.data_ptr()
    assert call(res.data_ptr()) == _lib.JQ_EINVAL
    assert b"must not overlap" in lib.jq_last_error()
    d[0].x = x.data_ptr()
    assert call(x.data_ptr(), ldy=K + 8) == _lib.JQ_EUNSUPPORTED
    torch.cuda.synchronize()
