"""GPU parity of the streamed program (jq_qgemv_stream_prepare / jq_qgemv_stream_run: a whole step's
dependent one-row mat-vecs in one persistent launch) against the CPU oracle and against the same ops as
separate launches.  Tolerance as for every mat-vec: max |y-ref| / max|ref| <= 1e-2, cosine >= 0.9999, plus
the elementwise bound of one output rounding step + 2e-3 of max|ref|."""
import ctypes

import numpy as np
import pytest
import torch

import jangq_b200 as jq
from jangq_b200 import _lib
from jangq_b200.plan import StreamProgram
from oracle import jang_oracle as jo

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def make_linear(N, K, bits, gs, seed, dtype=torch.bfloat16):
    g = torch.Generator(device=DEV).manual_seed(seed)
    w = (torch.randn((N, K), generator=g, device=DEV, dtype=torch.float32) * 0.02).to(dtype)
    return jq.JANGLinear.from_float(w, bits=bits, group_size=gs)


def reference(x, lin):
    return jo.qmatmul(x.float().cpu().numpy().reshape(1, -1), lin.weight.cpu().numpy().view(np.uint32),
                      lin.scales.float().cpu().numpy(), lin.biases.float().cpu().numpy(), lin.bits, lin.group_size)


def check(y, ref, dtype=torch.bfloat16):
    y = y.float().cpu().numpy().reshape(ref.shape)
    scale = np.abs(ref).max()
    assert np.abs(y - ref).max() / scale <= 1e-2
    assert float((y * ref).sum() / (np.linalg.norm(y) * np.linalg.norm(ref))) >= 0.9999
    ulp = 2.0 ** -8 if dtype == torch.bfloat16 else 2.0 ** -11
    assert np.all(np.abs(y - ref) <= ulp * np.abs(ref) + 2e-3 * scale)


def rand_x(K, seed, dtype=torch.bfloat16):
    g = torch.Generator(device=DEV).manual_seed(seed)
    return torch.randn((1, K), generator=g, device=DEV).to(dtype)


@pytest.mark.parametrize("dtype", (torch.bfloat16, torch.float16))
def test_small_program_every_width_and_ragged_shapes(dtype):
    """Independent activations per op: every width and group size, row counts that are not a multiple of the
    16-row tile, rows shorter than one 256-byte stage, rows whose last stage is short, a fused op of three
    matrices; fewer tiles than SMs (one or two CTAs per tile)."""
    shapes = ((8, 64, 176, 1024), (2, 64, 100, 768), (4, 64, 333, 1280), (2, 128, 64, 2048), (4, 128, 40, 1024),
              (8, 128, 17, 512), (2, 64, 300, 11008), (8, 64, 1, 256), (6, 64, 200, 1024), (6, 128, 77, 2048),
              (6, 64, 50, 1280))
    ops, lins, xs = [], [], []
    for i, (bits, gs, N, K) in enumerate(shapes):
        lin = make_linear(N, K, bits, gs, 10 + i, dtype)
        x = rand_x(K, 50 + i, dtype)
        y = torch.full((1, N), float("nan"), dtype=dtype, device=DEV)
        ops.append((x, [lin], [y]))
        lins.append(lin), xs.append(x)
    fused = [make_linear(n, 1024, 8, 64, 90 + n, dtype) for n in (96, 33, 250)]
    xf = rand_x(1024, 99, dtype)
    yf = [torch.full((1, l.out_features), float("nan"), dtype=dtype, device=DEV) for l in fused]
    ops.insert(3, (xf, fused, yf))
    prog = StreamProgram(ops, dtype)
    prog.run()
    torch.cuda.synchronize()
    for x, ls, ys in ops:
        for lin, y in zip(ls, ys):
            check(y, reference(x, lin), dtype)
    _lib.check(_lib.load().jq_device_status())


def test_chained_ops_read_the_previous_output():
    """x of an op is the whole output of the op before it (the float32 accumulator path), mixed with ops on
    outside buffers and an op that reads an output from two ops back; every op is checked against the oracle
    applied to the activations the GPU actually fed it."""
    dims = ((8, 1024, 512), (2, 512, 768), (4, 768, 1024), (8, 1024, 256))      # (bits, K, N): N feeds the next K
    x0 = rand_x(1024, 1)
    ops, cur = [], x0
    for i, (bits, K, N) in enumerate(dims):
        lin = make_linear(N, K, bits, 64, 200 + i)
        y = torch.zeros((1, N), dtype=torch.bfloat16, device=DEV)
        ops.append((cur, [lin], [y]))
        cur = y
    # reads the output of ops[1] (K = 768): written two ops earlier, a plain buffer by then
    late = make_linear(128, 768, 2, 64, 300)
    ops.append((ops[1][2][0], [late], [torch.zeros((1, 128), dtype=torch.bfloat16, device=DEV)]))
    prog = StreamProgram(ops)
    for _ in range(3):                                  # replays leave the workspace as they found it
        prog.run()
    torch.cuda.synchronize()
    for x, (lin,), (y,) in ops:
        check(y, reference(x, lin))
    _lib.check(_lib.load().jq_device_status())


def test_large_ops_contiguous_item_runs_and_replay():
    """More tiles than SMs (every CTA owns a run of items that starts and ends inside a tile), a fused op, a
    row chunking of an op with more rows than one op may have, CUDA-graph replay, bit-identical repeats."""
    a = [make_linear(n, 1024, 8, 64, 400 + n) for n in (3000, 520, 2500)]
    b = [make_linear(5000, 2048, 2, 64, 411)]
    c = [make_linear(40000, 512, 4, 64, 412)]
    xa, xb, xc = rand_x(1024, 5), rand_x(2048, 6), rand_x(512, 7)
    ops = [(xa, a, [torch.zeros((1, l.out_features), dtype=torch.bfloat16, device=DEV) for l in a]),
           (xb, b, [torch.zeros((1, 5000), dtype=torch.bfloat16, device=DEV)]),
           (xc, c, [torch.zeros((1, 40000), dtype=torch.bfloat16, device=DEV)])]
    prog = StreamProgram(ops)
    assert prog.n_ops >= 4                              # the 40000-row op was cut by rows
    prog.run()
    torch.cuda.synchronize()
    first = [y.clone() for _, _, ys in ops for y in ys]
    for x, ls, ys in ops:
        for lin, y in zip(ls, ys):
            check(y, reference(x, lin))
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        prog.run()
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        prog.run()
    for _, _, ys in ops:
        for y in ys:
            y.zero_()
    g.replay()
    g.replay()
    torch.cuda.synchronize()
    again = [y for _, _, ys in ops for y in ys]
    for p, q in zip(first, again):
        assert torch.equal(p, q)
    _lib.check(_lib.load().jq_device_status())


def test_decoder_layer_shapes_match_separate_launches():
    """Two layers of the dense decoder the benchmark streams ([q,k,v] 3 x 4096x4096 @8-bit, o 4096x4096 @8,
    [gate,up] 2 x 11008x4096 @2, down 4096x11008 @2) as one program, against the oracle and against the
    same plan as separate launches (same arithmetic, other summation order: one output rounding step)."""
    lins, groups = [], []
    for l in range(2):
        b = len(lins)
        lins += [make_linear(4096, 4096, 8, 64, 500 + 10 * l + i) for i in range(4)]
        lins += [make_linear(11008, 4096, 2, 64, 505 + 10 * l), make_linear(11008, 4096, 2, 64, 506 + 10 * l),
                 make_linear(4096, 11008, 2, 64, 507 + 10 * l)]
        groups += [[b, b + 1, b + 2], [b + 3], [b + 4, b + 5], [b + 6]]
    plans = [jq.GemvPlan(lins, m=1, device=DEV, groups=groups, persistent=p) for p in (False, True)]
    assert plans[1].launches_per_run == 1 and plans[0].launches_per_run == 8
    outs = []
    for p in plans:
        for k, buf in p._xbuf.items():
            buf.copy_(rand_x(k, k))
        p.capture()
        p.run()
        torch.cuda.synchronize()
        outs.append([y.clone() for y in p.y])
    for i in (0, 3, 4, 6, 9, 13):
        check(outs[1][i], reference(plans[1].x[i], lins[i]))
    for a, b in zip(*outs):
        assert (a.float() - b.float()).abs().max() <= 2.0 ** -7 * a.float().abs().max()
    _lib.check(_lib.load().jq_device_status())


def test_plan_with_a_width_the_program_does_not_take():
    """A 3-bit matrix between streamable groups: programs cover the runs around it, it keeps its own launch;
    the 6-bit head rides in the second program."""
    lins = [make_linear(512, 1024, 8, 64, 601), make_linear(512, 1024, 8, 64, 602), make_linear(1024, 1024, 3, 64, 603),
            make_linear(5000, 1024, 6, 64, 604)]
    plan = jq.GemvPlan(lins, m=1, device=DEV, groups=[[0, 1], [2], [3]], persistent=True)
    assert plan.launches_per_run == 3
    for k, buf in plan._xbuf.items():
        buf.copy_(rand_x(k, 77))
    plan.capture()
    plan.run()
    torch.cuda.synchronize()
    for i, lin in enumerate(lins):
        check(plan.y[i], reference(plan.x[i], lin))


def test_program_validation():
    lib = _lib.load()
    lin = make_linear(64, 512, 4, 64, 700)
    x = rand_x(512, 1)
    y = torch.zeros((1, 512), dtype=torch.bfloat16, device=DEV)

    def op(xp, yp, bits=4, K=512, N=64):
        d = _lib.JqStreamOp()
        d.x, d.K, d.bits, d.group_size, d.count = xp, K, bits, 64, 1
        d.codes[0], d.scales[0], d.biases[0], d.y[0], d.N[0] = (lin.weight.data_ptr(), lin.scales.data_ptr(),
                                                                  lin.biases.data_ptr(), yp, N)
        return d

    ws = torch.zeros(1 << 20, dtype=torch.uint8, device=DEV)
    prog = _lib.JqStreamProgram()

    def prepare(descs, nbytes=None):
        arr = (_lib.JqStreamOp * len(descs))(*descs)
        return lib.jq_qgemv_stream_prepare(arr, len(descs), _lib.JQ_BF16, ws.data_ptr(), ws.numel() if nbytes is None else nbytes,
                                           ctypes.byref(prog), _lib.stream_ptr())

    assert prepare([op(x.data_ptr(), y.data_ptr())]) == _lib.JQ_OK
    assert prepare([op(x.data_ptr(), y.data_ptr(), bits=3)]) == _lib.JQ_EUNSUPPORTED
    assert prepare([op(x.data_ptr(), y.data_ptr())], nbytes=512) == _lib.JQ_EWORKSPACE
    # the second op reads the middle of the first op's output: refused
    assert prepare([op(x.data_ptr(), y.data_ptr()), op(y.data_ptr() + 32, x.data_ptr(), K=512)]) == _lib.JQ_EINVAL
    assert b"overlaps an output" in lib.jq_last_error()
    assert prepare([op(x.data_ptr(), y.data_ptr(), N=1 << 20)]) == _lib.JQ_EUNSUPPORTED
    assert b"split the op by rows" in lib.jq_last_error()
    assert lib.jq_qgemv_stream_run(ctypes.byref(_lib.JqStreamProgram()), _lib.stream_ptr()) == _lib.JQ_EINVAL
