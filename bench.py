#!/usr/bin/env python3
"""Benchmark of the JANG quantized decode hot path on B200.

    python bench.py --gpus N --steps K --warmup W            # CUDA arm (this repo)
    python bench.py --impl reference --gpus N --steps K --warmup W   # reference's CPU path

Workload (N=1): BASELINE config 2, the dense Llama-shaped decoder's batch-1
decode weight stream — per layer q/k/v/o 4096x4096 @8-bit, gate/up 11008x4096
@2-bit, down 4096x11008 @2-bit, 32 layers, lm_head 32000x4096 @6-bit, group 64,
bf16 sidecars — i.e. the 225 quantized mat-vecs of one decoded token
(3.74 GB of algorithmic bytes, far larger than L2, so no flush is needed).
One step = one pass over all 225 matrices.  Weights are random N(0, 0.02)
quantized on the GPU by this repo's quantizer; activations are N(0,1).
Attention, norms and sampling are outside the path and are not run.

metric: achieved GB/s = algorithmic bytes / time.  `value` has inputs resident
in HBM and replays a CUDA graph; `e2e` goes through GemvPlan.run_host() with
pinned host activations in and the logits row out every step.
For N>1 the dense stack is replicated (weak scaling, no collective on this part
of the path).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LAYERS, HIDDEN, INTER, VOCAB, GS = 32, 4096, 11008, 32000, 64
METRIC, UNIT = "jang_qgemv_hbm_gbs", "GB/s"


def stack_spec():
    """(name, N, K, bits) of every quantized matrix one decoded token streams."""
    spec = []
    for l in range(LAYERS):
        for p in ("q", "k", "v", "o"):
            spec.append((f"layers.{l}.self_attn.{p}_proj", HIDDEN, HIDDEN, 8))
        spec.append((f"layers.{l}.mlp.gate_proj", INTER, HIDDEN, 2))
        spec.append((f"layers.{l}.mlp.up_proj", INTER, HIDDEN, 2))
        spec.append((f"layers.{l}.mlp.down_proj", HIDDEN, INTER, 2))
    spec.append(("lm_head", VOCAB, HIDDEN, 6))
    return spec


def stack_groups():
    """Indices into stack_spec() of the matrices that read the same activations and have no data
    dependency on each other in a real decoder layer: [q, k, v], [o], [gate, up], [down]; lm_head alone.
    Each group is one call of the batched mat-vec (one launch per run of equal shapes)."""
    groups = []
    for l in range(LAYERS):
        b = 7 * l
        groups += [[b, b + 1, b + 2], [b + 3], [b + 4, b + 5], [b + 6]]
    groups.append([7 * LAYERS])
    return groups


def alg_bytes(N, K, bits, gs=GS, m=1, sidecar=2):
    return N * K * bits // 8 + N * (K // gs) * 2 * sidecar + m * K * 2 + m * N * 2


CONFIG = {"workload": "config2 dense decoder, batch-1 decode weight stream: 225 qGEMVs/token "
                      "(32x[q,k,v,o 4096x4096@8b; gate,up 11008x4096@2b; down 4096x11008@2b] + lm_head 32000x4096@6b), "
                      "group 64, bf16; q/k/v and gate/up of a layer are fused launches (129 launches/token)",
          "matrices": 225, "bytes_per_step": sum(alg_bytes(n, k, b) for _, n, k, b in stack_spec()),
          "l2": "working set 3.7 GB per step >> 126 MB L2, no flush needed", "parallelism": "replicated"}


# --------------------------------------------------------------------------------------
# CPU arm: the reference's numpy path, dequantize_affine_numpy(...) @ x (jang_tools/affine.py:445-463), on a
# bounded sample of the workload, row chunks spread over one worker process per host core with the BLAS
# library held to one thread per worker (no oversubscription).  The reference's own function is used where
# its tree can be imported ($JANGQ_REF, or the build container's mount of it; widths 2/4/8 -- its 3/5/6-bit
# unpack is a per-element Python loop); elsewhere, and for the 6-bit rows, the restatement in oracle/jang_oracle.py.
# --------------------------------------------------------------------------------------
_CPU = {}


def _cpu_cores():
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


_REFERENCE_MOUNT = os.path.join(os.sep, "root", "reference")


def _reference_dequant():
    for root in (os.environ.get("JANGQ_REF", ""), _REFERENCE_MOUNT):
        pkg = os.path.join(root, "jang-tools")
        if root and os.path.isdir(os.path.join(pkg, "jang_tools")):
            if pkg not in sys.path:
                sys.path.insert(0, pkg)
            try:
                from jang_tools.affine import dequantize_affine_numpy
                return dequantize_affine_numpy
            except Exception:
                pass
    return None


def cpu_sample_setup():
    from oracle import jang_oracle as jo
    rng = np.random.default_rng(0)
    sample = []
    for name, N, K, bits in (("q_proj", HIDDEN, HIDDEN, 8), ("gate_proj", INTER, HIDDEN, 2),
                             ("lm_head[:4096]", 4096, HIDDEN, 6)):
        w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
        packed, s, b = jo.quantize_affine(w, bits, GS, src_dtype="bf16")
        x = jo.round_to(rng.standard_normal((1, K)).astype(np.float32), "bf16")
        sample.append((name, packed, s, b, x, bits, N, K))
    return sample


def _cpu_worker_init():
    try:
        from threadpoolctl import threadpool_limits
        _CPU["limit"] = threadpool_limits(limits=1)
    except Exception:
        pass


def _cpu_part(job):
    i, r0, r1 = job
    _, packed, s, b, x, bits, _, _ = _CPU["sample"][i]
    ref = _CPU["ref"]
    if ref is not None and bits in (2, 4, 8):
        W = ref(packed[r0:r1], s[r0:r1], b[r0:r1], bits=bits, group_size=GS)
        return float((x.astype(np.float32) @ W.T).sum())
    from oracle import jang_oracle as jo
    return float(jo.qmatmul(x, packed[r0:r1], s[r0:r1], b[r0:r1], bits, GS, acc=np.float32).sum())


def cpu_arm(steps, warmup):
    """Times the sample; returns (GB/s, ms per step, description).  Worker processes are forked after the
    sample exists, so they share it without copies; this process holds no CUDA context."""
    import multiprocessing as mp
    cores = _cpu_cores()
    _CPU["sample"] = cpu_sample_setup()
    _CPU["ref"] = _reference_dequant()
    jobs = []
    for i, (_, _, _, _, _, _, N, _) in enumerate(_CPU["sample"]):
        chunk = max(64, (N + 2 * cores - 1) // (2 * cores))
        jobs += [(i, r0, min(N, r0 + chunk)) for r0 in range(0, N, chunk)]
    nbytes = sum(alg_bytes(N, K, bits) for _, _, _, _, _, bits, N, K in _CPU["sample"])
    with mp.get_context("fork").Pool(cores, initializer=_cpu_worker_init) as pool:
        for _ in range(max(warmup, 1)):
            pool.map(_cpu_part, jobs)
        t0 = time.perf_counter()
        for _ in range(steps):
            pool.map(_cpu_part, jobs)
        dt = time.perf_counter() - t0
    kind = "reference" if _CPU["ref"] is not None else "port"
    desc = {"value": nbytes * steps / dt / 1e9, "unit": UNIT, "cores": cores, "blas_threads_per_worker": 1,
            "workers": cores, "kind": kind,
            "sample": "per step: one q_proj 4096x4096@8b + one gate_proj 11008x4096@2b + 4096 rows of lm_head@6b; "
                      "dequantize + f32 mat-vec in numpy, row chunks over one process per core"
                      + ("; jang_tools.affine.dequantize_affine_numpy for the 2/8-bit matrices, its restatement for "
                         "the 6-bit rows" if kind == "reference" else "; numpy restatement of jang_tools/affine.py:445-463"),
            "ms_per_step": dt / steps * 1e3}
    return desc


def cpu_baseline(steps=3, warmup=1):
    """The CPU arm in a process of its own (this one holds a CUDA context; workers are forked)."""
    import subprocess
    out = subprocess.run([sys.executable, os.path.abspath(__file__), "--impl", "reference", "--steps", str(steps),
                          "--warmup", str(warmup)], capture_output=True, text=True, timeout=900,
                         env={k: v for k, v in os.environ.items() if k not in ("RANK", "WORLD_SIZE", "LOCAL_RANK")})
    for line in out.stdout.splitlines():
        if line.startswith("{"):
            return json.loads(line)["cpu_baseline"]
    return {"error": (out.stderr or out.stdout)[-300:]}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    desc = cpu_arm(args.steps, args.warmup)
    v = desc["value"]
    line = {"impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": desc["ms_per_step"], "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": CONFIG,
            "cpu_baseline": desc,
            "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------
# clocks sampling (read-only NVML)
# --------------------------------------------------------------------------------------
class ClockSampler:
    def __init__(self, index):
        self.samples, self.reasons, self._stop = [], set(), threading.Event()
        self.max_mhz = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            try:
                import torch
                uuid = str(torch.cuda.get_device_properties(index).uuid)
                self.h = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid) if not uuid.startswith("GPU-") else uuid)
            except Exception:
                self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None
        self.t = threading.Thread(target=self._run, daemon=True)

    def _run(self):
        nv = self.nv
        names = {"hw_slowdown": 0x8, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40,
                 "hw_power_brake_slowdown": 0x80, "sw_power_cap": 0x4}
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                for k, bit in names.items():
                    if r & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            time.sleep(0.001)      # the timed region is tens of milliseconds: sample as fast as NVML answers

    def __enter__(self):
        if self.nv is not None:
            self.t.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self.nv is not None:
            self.t.join(timeout=1)

    def summary(self):
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


# --------------------------------------------------------------------------------------
# CUDA arm
# --------------------------------------------------------------------------------------
def build_stack(device):
    import torch
    import jangq_b200 as jq
    linears = []
    for i, (name, N, K, bits) in enumerate(stack_spec()):
        g = torch.Generator(device=device)
        g.manual_seed(1000 + i)
        w = (torch.randn((N, K), generator=g, device=device, dtype=torch.float32) * 0.02).to(torch.bfloat16)
        linears.append(jq.JANGLinear.from_float(w, bits=bits, group_size=GS))
        del w
    return linears


def run_cuda(args):
    import torch
    import torch.distributed as dist
    import jangq_b200 as jq

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        # the peer exchange uses plain peer loads and stores: keep its buffers off NVLink multicast objects
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback for the CUDA arm)")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    linears = build_stack(device)
    plan = jq.GemvPlan(linears, m=1, dtype=torch.bfloat16, device=device, groups=stack_groups(),
                       persistent=args.persistent)
    g = torch.Generator(device=device)
    g.manual_seed(7)
    for buf in plan._xbuf.values():
        buf.copy_(torch.randn(buf.shape, generator=g, device=device).to(torch.bfloat16))
    for k, hb in plan._host_in.items():
        hb.copy_(plan._xbuf[k].cpu())
    plan.capture()

    W, K = max(args.warmup, 3), args.steps
    for _ in range(W):
        plan.run()
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clk:
        barrier()
        ev0.record()
        for _ in range(K):
            plan.run()
        ev1.record()
        barrier()
    ms = ev0.elapsed_time(ev1)
    t = torch.tensor([ms], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    bytes_step = plan.algorithmic_bytes
    value = world * bytes_step * K / (ms * 1e-3) / 1e9

    # end to end through the public API with host buffers
    for _ in range(3):
        plan.run_host()
    barrier()
    t0 = time.perf_counter()
    ev0.record()
    for _ in range(K):
        plan.run_host()
    ev1.record()
    barrier()
    e2e_ms = max(ev0.elapsed_time(ev1), (time.perf_counter() - t0) * 1e3)
    t = torch.tensor([e2e_ms], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_ms = float(t.item())
    e2e = world * bytes_step * K / (e2e_ms * 1e-3) / 1e9

    moe_res = None
    if not args.no_moe:
        moe_res = run_moe(args, device, world, rank, barrier)

    jq._lib.check(jq._lib.load().jq_device_status())

    if rank == 0:
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except Exception:
            pass
        peak = float(peaks.get("hbm_gbs", 6650.0))
        per_gpu = value / world
        # DRAM bytes of one step = sum over the step's five launch shapes of (bytes ncu counted for one launch of
        # that shape) x (launches of that shape per step); the captures are per kernel, not of this run
        traffic = None
        try:
            shapes = json.load(open(os.path.join(ROOT, "profiles", "qgemv_one_dram_bytes.json")))["launch_shapes"]
            traffic = sum(int(v["dram_bytes"]) * int(v["launches_per_step"]) for v in shapes.values())
        except Exception:
            pass
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W,
                "ms_per_step": ms / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "bf16", "data": "synthetic", "config": CONFIG,
                "tokens_per_s_weight_stream_bound": world * K / (ms * 1e-3),
                "roofline": {"bound": "hbm", "achieved": per_gpu, "peak": peak, "unit": "GB/s",
                             "frac": per_gpu / peak,
                             "peak_source": "measured (MEASURED_PEAKS.json)" if peaks else "fallback 6650",
                             "traffic": traffic,
                             "traffic_note": "ESTIMATED: per step, the sum over the five launch shapes of one captured launch's "
                             "dram__bytes_read + dram__bytes_write (ncu, per kernel) x launches per step "
                             "(profiles/qgemv_one_dram_bytes.json); not a capture of this run",
                             "kernel": ("qgemv_stream_kernel (the step as one persistent launch)" if args.persistent else
                                        "qgemv_one_kernel (225 matrices in 129 launches per step, averaged)")},
                "e2e": {"value": e2e, "unit": UNIT, "h2d_bytes_per_step": plan.h2d_bytes,
                        "d2h_bytes_per_step": plan.d2h_bytes, "ms_per_step": e2e_ms / K},
                "gpu_launches": plan.launches_per_run * K, "clocks": clk.summary()}
        if moe_res is not None:
            line["moe_decode"] = moe_res
        if world == 1 and not args.no_extras:
            try:
                line["other_configs"] = run_extras(peaks, quick=args.quick_extras)
            except Exception as e:                        # the headline stands without the side measurements
                line["other_configs"] = {"error": f"{type(e).__name__}: {e}"}
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline()
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_moe(args, device, world, rank, barrier):
    """BASELINE config 3, batch-1 decode per GPU through the quantized hot path (attention
    projections 6-bit, router, top-8 of 128 experts 2-bit), experts sharded over the ranks;
    aggregate tokens/s = world tokens per step / step time (weak scaling: one token per GPU)."""
    import torch
    import torch.distributed as dist
    from jangq_b200.stacks import MoEDecodeStack
    ep_mode = os.environ.get("JANGQ_EP_MODE", "peer")
    try:
        stack = MoEDecodeStack(device=device, rank=rank, world=world, ep_mode=ep_mode)
    except Exception as e:                                # no symmetric memory on this box: NCCL all-reduce instead
        if rank == 0:
            print(f"# peer exchange not available ({type(e).__name__}: {e}); using the NCCL all-reduce", file=sys.stderr)
        ep_mode = "replicated"
        stack = MoEDecodeStack(device=device, rank=rank, world=world, ep_mode=ep_mode)
    g = torch.Generator(device=device)
    g.manual_seed(11)
    # one token per GPU and step; with N > 1 every rank carries the rows of all N tokens (same seed everywhere)
    x = torch.randn((world, stack.H), generator=g, device=device).to(torch.bfloat16)
    out = stack.step(x)                                   # eager warm-up (sets function attributes)
    torch.cuda.synchronize()
    graph = None
    try:
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            stack.step(x)
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr):
            out = stack.step(x)
        graph = gr
    except Exception as e:                                # capture of the collectives not available: run eagerly
        if rank == 0:
            print(f"# MoE step not captured ({type(e).__name__}: {e}); timing eager launches", file=sys.stderr)
        torch.cuda.synchronize()

    def one():
        if graph is not None:
            graph.replay()
        else:
            stack.step(x)

    W, K = max(args.warmup, 3), args.steps
    for _ in range(W):
        one()
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(K):
        one()
    ev1.record()
    barrier()
    t = torch.tensor([ev0.elapsed_time(ev1)], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item()) / K
    finite = bool(torch.isfinite(out.float()).all())
    # strong scaling: ONE token per step on all N GPUs (every rank runs the dense blocks on it, its own experts, one
    # exchange per layer): the batch-1 latency the path is named for, next to the weak-scaling throughput above
    strong = None
    if world > 1:
        try:
            x1 = x[:1].contiguous()
            stack.step(x1)
            torch.cuda.synchronize()
            s1 = torch.cuda.Stream()
            s1.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s1):
                stack.step(x1)
            torch.cuda.current_stream().wait_stream(s1)
            torch.cuda.synchronize()
            g1 = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g1):
                stack.step(x1)
            for _ in range(W):
                g1.replay()
            barrier()
            ev0.record()
            for _ in range(K):
                g1.replay()
            ev1.record()
            barrier()
            t1 = torch.tensor([ev0.elapsed_time(ev1)], device=device, dtype=torch.float64)
            dist.all_reduce(t1, op=dist.ReduceOp.MAX)
            ms1 = float(t1.item()) / K
            strong = {"tokens_per_step": 1, "ms_per_step": ms1, "tok_s": 1.0 / (ms1 * 1e-3),
                      "note": "one token on all N GPUs: per-token latency; the dense half is replicated, so N GPUs buy no "
                              "latency on this path"}
        except Exception as e:
            strong = {"error": f"{type(e).__name__}: {e}"}
    peak = 6464.6
    try:
        peak = float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["hbm_gbs"])
    except Exception:
        pass
    # routed-expert block over a 2048-token prefill batch per GPU (sorted grouped-GEMM path)
    Tp = 2048
    xp = torch.randn((Tp, stack.H), generator=g, device=device).to(torch.bfloat16)
    nl = min(4, stack.L)
    layer_fn = stack.prefill_layer
    for l in range(nl):
        layer_fn(xp, l)
    if stack.prefill_overflowed():       # a destination got more rows than its slots hold: the exact exchange instead
        layer_fn = stack.prefill_layer_exact
    barrier()
    ev0.record()
    for _ in range(3):
        for l in range(nl):
            layer_fn(xp, l)
    ev1.record()
    barrier()
    exchange = "one GPU" if world == 1 else ("fixed-capacity slots, two equal-split all_to_all_single, no host read-back"
                                             if layer_fn == stack.prefill_layer and not stack.prefill_overflowed()
                                             else "exact split sizes (host read-back per layer): slots overflowed")
    tp = torch.tensor([ev0.elapsed_time(ev1)], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(tp, op=dist.ReduceOp.MAX)
    ms_layer = float(tp.item()) / (3 * nl)
    flops_layer = 2.0 * Tp * stack.k * 3 * stack.I * stack.H
    prefill = {"tokens_per_gpu": Tp, "ms_per_layer": ms_layer, "tok_s_per_layer": world * Tp / (ms_layer * 1e-3),
               "expert_TFLOPs_per_gpu": flops_layer / (ms_layer * 1e-3) / 1e12,
               "note": "router + sort + gather + gate/up/down grouped GEMMs + SwiGLU + combine of one layer; "
                       "N>1: all-to-all dispatch/combine of the rank's 2048 tokens", "exchange": exchange}
    gbs = stack.bytes_per_token / (ms * 1e-3) / 1e9
    parity = moe_parity(stack, x, xp, device, world, rank) if world > 1 else None
    return {"parity": parity, "prefill": prefill, "strong_scaling": strong, "scaling_of_tok_s": "weak (one token per GPU and step)",
            "tok_s": world / (ms * 1e-3), "ms_per_step": ms, "tokens_per_step": world, "bytes_per_token": stack.bytes_per_token,
            "per_gpu_GBps": gbs, "hbm_frac": gbs / peak, "graph": graph is not None, "finite": finite,
            "ep_mode": ep_mode if world > 1 else None,
            "workload": "config3 MoE stack, batch-1 decode per GPU: 48 layers x [q,k,v,o @6b + bf16 router + top-8 of "
                        "128 experts (768x2048 gate/up, 2048x768 down) @2b], group 64; experts sharded E/N per GPU, "
                        "N>1: every rank runs the replicated dense blocks on the N tokens of the step, its own experts on "
                        "them, and the partial sums are added per layer over NVLink peer loads inside the residual+norm "
                        "kernel (ep_mode peer) or by one NCCL all-reduce (ep_mode replicated); attention core not run"}


def run_extras(peaks, quick=False):
    """The other BASELINE configurations on one GPU, as sub-records of the bench line (CUDA events, graph
    replay, weights rotated over more than twice the L2 where a case would fit it):
      config1   4096x4096 bf16 weight: quantize at 4 bits (GB/s) and the batch-1 mat-vec over it;
      qgemm     the prefill GEMM at the config-2 layer shapes with M = 512, and 4096 x 14336 x 4096 at 4 bits;
      sweep     config 4: K in {2048,4096,8192} x N in {4096,14336,28672} x bits {2,3,4,6,8} x group {64,128},
                M in {1,8} as GB/s against the HBM peak, M in {64,512,4096} as TFLOP/s against the bf16 peak;
                per width the minimum and the median fraction over the 18 (K, N, group) cases."""
    import torch
    import microbench as mb
    hbm = float(peaks.get("hbm_gbs", 6650.0))
    tf_burst = float(peaks.get("bf16_tflops", 1590.0))
    tf_sus = float(peaks.get("bf16_tflops_sustained", 1400.0))
    out = {"peaks": {"hbm_gbs": hbm, "bf16_tflops_burst": tf_burst, "bf16_tflops_sustained": tf_sus,
                     "source": "measured (MEASURED_PEAKS.json)" if peaks else "fallback"}}
    q = mb.bench_quantize(4096, 4096, 4, 64, 5, 300)
    v = mb.bench_qgemv(4096, 4096, 4, 64, 1, 5, 300, flags=1)
    out["config1"] = {"quantize_GBps": q["GBps"], "quantize_us": q["us"], "quantize_frac_hbm": q["GBps"] / hbm,
                      "qgemv_GBps": v["GBps"], "qgemv_us": v["us"], "qgemv_frac_hbm": v["GBps"] / hbm,
                      "note": "HBM-resident: rotating copies; the 9.45 MB mat-vec alone would sit in L2"}
    torch.cuda.empty_cache()
    layer = []
    flops = us = 0.0
    for name, N, K, bits, cnt in (("q/k/v/o", 4096, 4096, 8, 4), ("gate/up", 11008, 4096, 2, 2), ("down", 4096, 11008, 2, 1)):
        r = mb.bench_qgemm(N, K, bits, 64, 512, 3)
        layer.append({"name": name, "M": 512, "N": N, "K": K, "bits": bits, "TFLOPs": r["TFLOPs"], "us": r["us"]})
        flops += cnt * 2.0 * 512 * N * K
        us += cnt * r["us"]
    big = mb.bench_qgemm(14336, 4096, 4, 64, 4096, 3)
    out["qgemm"] = {"config2_prefill512_layer": layer, "layer_TFLOPs": flops / (us * 1e-6) / 1e12,
                    "layer_frac_burst": flops / (us * 1e-6) / 1e12 / tf_burst,
                    "layer_frac_sustained": flops / (us * 1e-6) / 1e12 / tf_sus,
                    "M4096_N14336_K4096_4bit_TFLOPs": big["TFLOPs"], "frac_burst": big["TFLOPs"] / tf_burst,
                    "frac_sustained": big["TFLOPs"] / tf_sus}
    torch.cuda.empty_cache()
    Ks, Ns = ((4096,), (4096, 14336)) if quick else ((2048, 4096, 8192), (4096, 14336, 28672))
    sweep = {}
    for bits in (2, 3, 4, 6, 8):
        small, large, worst_s, worst_l = {1: [], 8: []}, {64: [], 512: [], 4096: []}, None, None
        for gs in (64, 128):
            for K in Ks:
                for N in Ns:
                    for M in (1, 8):
                        r = mb.bench_qgemv(N, K, bits, gs, M, 3, 256, flags=1)
                        f = r["GBps"] / hbm
                        small[M].append(f)
                        if worst_s is None or f < worst_s[0]:
                            worst_s = (f, f"M={M} N={N} K={K} gs={gs}")
                    for M in (64, 512, 4096):
                        r = mb.bench_qgemm(N, K, bits, gs, M, 2)
                        f = r["TFLOPs"] / tf_burst
                        large[M].append(f)
                        if worst_l is None or f < worst_l[0]:
                            worst_l = (f, f"M={M} N={N} K={K} gs={gs}")
                    torch.cuda.empty_cache()
        sweep[str(bits)] = {
            **{f"M{M}_hbm_frac_min_med": [min(v), statistics.median(v)] for M, v in small.items()},
            **{f"M{M}_bf16_burst_frac_min_med": [min(v), statistics.median(v)] for M, v in large.items()},
            "worst_small": worst_s[1], "worst_large": worst_l[1]}
    out["config4_sweep"] = {"cases_per_width": len(Ks) * len(Ns) * 2, "by_bits": sweep,
                            "note": "fractions of the measured HBM copy rate (M = 1, 8) and of the measured bf16 burst "
                                    "rate (M = 64, 512, 4096); [minimum, median] over K x N x group size"}
    return out


def moe_parity(stack, x, xp, device, world, rank):
    """Outside the timed region, with several ranks: two layers of the expert-parallel decode step and one
    expert-parallel prefill layer against the same layers computed on rank 0 alone from all experts (a
    one-rank stack with the same seeds: experts are drawn by global id, so it is the same model).
    Returns max |y - ref| / max |ref| and the cosine of both comparisons (north-star bar 1e-2 / 0.9999)."""
    import torch
    from jangq_b200.stacks import MoEDecodeStack
    y_ep = stack.step(x, n_layers=2).float()
    p_ep = stack.prefill_layer(xp, 0).float()
    torch.cuda.synchronize()
    if rank != 0:
        return None
    ref = MoEDecodeStack(layers=2, device=device, rank=0, world=1)
    y_ref = ref.step(x).float()
    p_ref = ref.prefill_layer(xp, 0).float()
    torch.cuda.synchronize()

    def cmp(a, b):
        return {"max_rel": float((a - b).abs().max() / b.abs().max()),
                "cos": float((a * b).sum() / (a.norm() * b.norm()))}
    return {"decode_2_layers": cmp(y_ep, y_ref), "prefill_layer_0": cmp(p_ep, p_ref),
            "reference": "the same layers on rank 0 alone with all 128 experts", "tokens": int(x.shape[0])}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="cuda", choices=("cuda", "reference"))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-moe", action="store_true", help="skip the config-3 MoE decode measurement")
    ap.add_argument("--no-extras", action="store_true", help="skip the config-1 / prefill GEMM / config-4 sweep sub-records")
    ap.add_argument("--quick-extras", action="store_true", help="a reduced config-4 sweep (K=4096, two N)")
    ap.add_argument("--persistent", action="store_true",
                    help="the whole step as one persistent launch (jq_qgemv_stream_run) instead of one launch per group of "
                         "matrices; measured slower on B200 (1.5 ms against 1.1 ms per step), kept for comparison")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_cuda(args)


if __name__ == "__main__":
    main()
