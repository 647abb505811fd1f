"""Single-op micro-benchmark with an HBM-resident working set.

    python microbench.py --op qgemv --N 4096 --K 4096 --bits 4 --gs 64 --M 1
    python microbench.py --op quantize --N 8192 --K 8192 --bits 4
    python microbench.py --sweep qgemv        # BASELINE config-4 small-M sweep

Distinct copies of the weights are rotated so that the bytes touched between
two uses of the same copy exceed `--rotate-mb` (default 512 MB, 4x the L2), and
the launches are replayed from a CUDA graph.  Prints one JSON line per case
with achieved GB/s (algorithmic bytes / time) or TFLOP/s.
"""
from __future__ import annotations

import argparse
import json

import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from jangq_b200 import _lib, ops  # noqa: E402


def _time_graph(fn, iters: int, warmup: int = 3) -> float:
    """Median milliseconds of one fn() call sequence, replayed from a CUDA graph."""
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        fn()
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        fn()
    for _ in range(warmup):
        g.replay()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        e1.synchronize()
        times.append(e0.elapsed_time(e1))
    times.sort()
    return times[len(times) // 2]


def bytes_w(N, K, bits, gs, e=2):
    return N * K * bits // 8 + N * (K // gs) * 2 * e


def bench_qgemv(N, K, bits, gs, M, iters, rotate_mb, dtype=torch.bfloat16, flags=0):
    dev = torch.device("cuda")
    per = bytes_w(N, K, bits, gs)
    copies = max(2, min(64, int(rotate_mb * 2 ** 20 // per) + 1))
    g = torch.Generator(device=dev)
    g.manual_seed(0)
    w = (torch.randn((N, K), generator=g, device=dev) * 0.02).to(dtype)
    wq, s, b = ops.quantize(w, gs, bits)
    del w
    ws = [(wq.clone(), s.clone(), b.clone()) for _ in range(copies)]
    x = torch.randn((M, K), generator=g, device=dev).to(dtype)
    y = torch.empty((M, N), dtype=dtype, device=dev)

    def fn():
        for wq_, s_, b_ in ws:
            ops._qgemv(x, wq_, s_, b_, K, bits, gs, y, flags)

    ms = _time_graph(fn, iters) / copies
    alg = per + M * K * 2 + M * N * 2
    return {"op": "qgemv", "N": N, "K": K, "bits": bits, "gs": gs, "M": M, "us": ms * 1e3,
            "GBps": alg / (ms * 1e-3) / 1e9, "bytes": alg, "copies": copies}


def bench_qgemm(N, K, bits, gs, M, iters, dtype=torch.bfloat16):
    """Prefill GEMM: TFLOP/s = 2*M*N*K / time (activations and weights stay L2/HBM resident as they fall)."""
    from jangq_b200.gemm import qgemm
    dev = torch.device("cuda")
    g = torch.Generator(device=dev)
    g.manual_seed(0)
    w = (torch.randn((N, K), generator=g, device=dev) * 0.02).to(dtype)
    wq, s, b = ops.quantize(w, gs, bits)
    del w
    x = torch.randn((M, K), generator=g, device=dev).to(dtype)
    y = torch.empty((M, N), dtype=dtype, device=dev)
    reps = 4

    def fn():
        for _ in range(reps):
            qgemm(x, wq, s, b, K, bits, gs, y)

    ms = _time_graph(fn, iters) / reps
    return {"op": "qgemm", "M": M, "N": N, "K": K, "bits": bits, "gs": gs, "us": ms * 1e3,
            "TFLOPs": 2.0 * M * N * K / (ms * 1e-3) / 1e12}


def bench_quantize(N, K, bits, gs, iters, rotate_mb, dtype=torch.bfloat16, op="quantize"):
    dev = torch.device("cuda")
    per = N * K * 2
    copies = max(2, min(16, int(rotate_mb * 2 ** 20 // per) + 1))
    g = torch.Generator(device=dev)
    g.manual_seed(0)
    wsrc = [(torch.randn((N, K), generator=g, device=dev) * 0.02).to(dtype) for _ in range(copies)]
    if op in ("quantize", "quantize_ieee_div", "quantize_rtn", "quantize_rtn_ieee_div", "quantize_mse", "quantize_mse_exhaustive"):
        mode = {"quantize": "affine", "quantize_ieee_div": "affine_ieee_div", "quantize_rtn": "rtn", "quantize_rtn_ieee_div": "rtn_ieee_div", "quantize_mse": "mse",
                "quantize_mse_exhaustive": "mse_exhaustive"}[op]

        def fn():
            for w in wsrc:
                ops.quantize(w, gs, bits, mode=mode)
        alg = per + bytes_w(N, K, bits, gs)
    elif op == "quantize_imatrix":
        # the C entry point directly: the Python wrapper floors the importance vector on the host
        lib = _lib.load()
        imp = (torch.randn((K,), generator=g, device=dev) ** 2 + 1e-3).float()
        outs = [(torch.empty((N, K * bits // 32), dtype=torch.int32, device=dev),
                 torch.empty((N, K // gs), dtype=torch.float16, device=dev),
                 torch.empty((N, K // gs), dtype=torch.float16, device=dev)) for _ in wsrc]

        def fn():
            for w, (q, s, b) in zip(wsrc, outs):
                _lib.check(lib.jq_quantize_imatrix(w.data_ptr(), _lib.dtype_id(w.dtype), imp.data_ptr(), N, K, bits, gs, 6,
                                                   q.data_ptr(), s.data_ptr(), b.data_ptr(), _lib.stream_ptr(dev)))
        alg = per + bytes_w(N, K, bits, gs)
    else:
        trip = [ops.quantize(w, gs, bits) for w in wsrc]
        del wsrc

        def fn():
            for wq, s, b in trip:
                ops.dequantize(wq, s, b, gs, bits)
        alg = per + bytes_w(N, K, bits, gs)
    ms = _time_graph(fn, iters) / copies
    return {"op": op, "N": N, "K": K, "bits": bits, "gs": gs, "us": ms * 1e3, "GBps": alg / (ms * 1e-3) / 1e9,
            "bytes": alg, "copies": copies}


def bench_moe_decode(layers, T, iters):
    """Few-token decode through `layers` layers of the config-3 MoE stack (stacks.MoEDecodeStack, one GPU): one
    eager pass (plain launches, what a launch-list capture sees), then the median time of a graph replay."""
    from jangq_b200.stacks import MoEDecodeStack
    dev = torch.device("cuda")
    stack = MoEDecodeStack(layers=layers, device=dev)
    g = torch.Generator(device=dev)
    g.manual_seed(11)
    x = torch.randn((T, stack.H), generator=g, device=dev).to(torch.bfloat16)
    stack.step(x)
    torch.cuda.synchronize()
    ms = _time_graph(lambda: stack.step(x), iters)
    return {"op": "moe_decode", "layers": layers, "T": T, "us_per_layer": ms * 1e3 / layers, "ms_per_step": ms,
            "bytes_per_token": stack.bytes_per_token}


def bench_moe_prefill(tokens, iters):
    """The routed-expert block of one config-3 layer over `tokens` tokens (router, sort, gather, grouped GEMMs,
    SwiGLU, combine), timed as eager launches with CUDA events (its tile counts live on the device, so it is not
    graph-captured)."""
    from jangq_b200.stacks import MoEDecodeStack
    dev = torch.device("cuda")
    stack = MoEDecodeStack(layers=1, device=dev)
    g = torch.Generator(device=dev)
    g.manual_seed(12)
    x = torch.randn((tokens, stack.H), generator=g, device=dev).to(torch.bfloat16)
    for _ in range(3):
        stack.prefill_layer(x)
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        stack.prefill_layer(x)
        e1.record()
        e1.synchronize()
        times.append(e0.elapsed_time(e1))
    times.sort()
    ms = times[len(times) // 2]
    flops = 2.0 * tokens * stack.k * 3 * stack.I * stack.H
    return {"op": "moe_prefill", "tokens": tokens, "ms_per_layer": ms, "expert_TFLOPs": flops / (ms * 1e-3) / 1e12}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", default="qgemv", choices=("qgemv", "qgemm", "quantize", "quantize_ieee_div", "quantize_rtn", "quantize_rtn_ieee_div", "quantize_mse", "quantize_mse_exhaustive", "quantize_imatrix", "dequantize", "moe_decode", "moe_prefill"))
    ap.add_argument("--sweep", default=None, choices=(None, "qgemv", "qgemv-small", "qgemm"))
    ap.add_argument("--N", type=int, default=4096)
    ap.add_argument("--K", type=int, default=4096)
    ap.add_argument("--bits", type=int, default=4)
    ap.add_argument("--gs", type=int, default=64)
    ap.add_argument("--M", type=int, default=1)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--rotate-mb", type=float, default=512.0)
    ap.add_argument("--layers", type=int, default=4, help="moe_decode: layers of the stack")
    ap.add_argument("--pdl", action="store_true", help="launch with JQ_GEMV_STATIC_WEIGHTS (overlapped launches)")
    a = ap.parse_args()
    _lib.load()
    flags = _lib.JQ_GEMV_STATIC_WEIGHTS if a.pdl else 0
    if a.sweep == "qgemm":
        for N in (4096, 14336):
            for bits in (2, 4, 8):
                for M in (64, 512, 4096):
                    print(json.dumps(bench_qgemm(N, 4096, bits, 64, M, a.iters)), flush=True)
        return
    if a.sweep:
        Ks = (2048, 4096, 8192) if a.sweep == "qgemv" else (4096,)
        Ns = (4096, 14336, 28672) if a.sweep == "qgemv" else (4096, 14336)
        for K in Ks:
            for N in Ns:
                for bits in (2, 3, 4, 6, 8):
                    for gs in (64, 128):
                        for M in (1, 8):
                            print(json.dumps(bench_qgemv(N, K, bits, gs, M, a.iters, a.rotate_mb, flags=flags)), flush=True)
        return
    if a.op == "moe_decode":
        print(json.dumps(bench_moe_decode(a.layers, a.M, a.iters)))
    elif a.op == "moe_prefill":
        print(json.dumps(bench_moe_prefill(a.M if a.M > 1 else 2048, a.iters)))
    elif a.op == "qgemv":
        print(json.dumps(bench_qgemv(a.N, a.K, a.bits, a.gs, a.M, a.iters, a.rotate_mb, flags=flags)))
    elif a.op == "qgemm":
        print(json.dumps(bench_qgemm(a.N, a.K, a.bits, a.gs, a.M, a.iters)))
    else:
        print(json.dumps(bench_quantize(a.N, a.K, a.bits, a.gs, a.iters, a.rotate_mb, op=a.op)))
    _lib.check(_lib.load().jq_device_status())


if __name__ == "__main__":
    main()
