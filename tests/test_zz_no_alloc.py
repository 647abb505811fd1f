"""The workspace-free grouped GEMM (jq_moe_gemm_static) against jq_moe_gemm.

Some users of this library cannot allocate device memory where they call it: a serving process
that handed all of its device memory to weight and KV-cache arenas when it started, or a host
runtime that loads the library as a plug-in and keeps its allocator to itself.  For them the
tile list of the grouped GEMM lives in a fixed array inside the library.  This test calls the
entry point through the C ABI twice in a row with different routings (the second call must not
see anything of the first) and compares with the entry point that takes caller buffers: the same
kernel walks the same tiles, so the outputs must be identical, which is tighter than the 1e-2
bound the other MoE tests use.  The file sorts last so that a run stopping at the first failure
has already run every other test; it also passes on its own in a fresh process."""
import numpy as np
import pytest
import torch

import jangq_b200 as jq
from jangq_b200 import _lib
from jangq_b200.moe import SortedPairs, _gather_rows, _moe_gemm

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_static_grouped_gemm_matches_workspace_version_twice():
    lib = _lib.load()
    E, N, K, bits, gs = 12, 192, 256, 4, 64
    rng = np.random.default_rng(123)
    w = torch.from_numpy((rng.standard_normal((E, N, K)) * 0.05).astype(np.float32)).to(DEV).to(torch.bfloat16)
    wq, s, b = jq.quantize(w, gs, bits)
    bank = jq.ExpertBank(wq, s, b, bits, gs)
    for call, (T, k) in enumerate(((150, 4), (97, 2))):
        x = torch.from_numpy(rng.standard_normal((T, K)).astype(np.float32)).to(DEV).to(torch.bfloat16)
        # second call: a routing that leaves most experts empty, so stale tiles of call one would show
        hi = E if call == 0 else 3
        idx = torch.from_numpy(rng.integers(0, hi, T * k).astype(np.int32)).to(DEV)
        sp = SortedPairs(idx, E)
        xs = _gather_rows(x, sp, k)
        ref = _moe_gemm(xs, sp, bank)
        y = torch.full_like(ref, float("nan"))
        rc = lib.jq_moe_gemm_static(xs.data_ptr(), _lib.JQ_BF16, sp.n, xs.stride(0), sp.offsets.data_ptr(), E,
                                    bank.codes_tab.data_ptr(), bank.scales_tab.data_ptr(), bank.biases_tab.data_ptr(),
                                    None, _lib.JQ_BF16, N, K, bits, gs, y.data_ptr(), y.stride(0), _lib.stream_ptr())
        _lib.check(rc)
        torch.cuda.synchronize()
        kept = int(sp.offsets[E])
        assert kept == T * k
        assert torch.equal(y[:kept], ref[:kept])
        assert bool(torch.isfinite(y[:kept].float()).all())
    assert lib.jq_device_status() == 0


def test_static_grouped_gemm_rejects_sizes_beyond_its_array():
    lib = _lib.load()
    z = torch.zeros(8, dtype=torch.int64, device=DEV)
    rc = lib.jq_moe_gemm_static(z.data_ptr(), _lib.JQ_BF16, 16, 64, z.data_ptr(), 2000, z.data_ptr(), z.data_ptr(),
                                z.data_ptr(), None, _lib.JQ_BF16, 64, 64, 4, 64, z.data_ptr(), 64, None)
    assert rc == _lib.JQ_EUNSUPPORTED and b"at most 1024 experts" in lib.jq_last_error()
    rc = lib.jq_moe_gemm_static(z.data_ptr(), _lib.JQ_BF16, 70000, 64, z.data_ptr(), 4, z.data_ptr(), z.data_ptr(),
                                z.data_ptr(), None, _lib.JQ_BF16, 64, 64, 4, 64, z.data_ptr(), 64, None)
    assert rc == _lib.JQ_EUNSUPPORTED and b"at most 65536 rows" in lib.jq_last_error()


def test_static_grouped_gemm_mixed_widths_and_dropped_pairs():
    """A bank with two code widths (one launch per width, experts of the other width skipped) and a routing in
    which some pairs belong to experts outside the bank, so fewer rows are kept than the call's row bound:
    two calls in a row, each identical to the entry point that takes caller buffers."""
    lib = _lib.load()
    E, N, K, gs, base = 6, 128, 256, 64, 4
    widths = (4, 8, 4, 8, 8, 4)
    rng = np.random.default_rng(77)
    experts = []
    for e in range(E):
        w = torch.from_numpy((rng.standard_normal((N, K)) * 0.05).astype(np.float32)).to(DEV).to(torch.bfloat16)
        wq, s, b = jq.quantize(w, gs, widths[e])
        experts.append((wq, s, b, widths[e]))
    bank = jq.ExpertBank.from_experts(experts, gs)
    for T, k in ((140, 3), (33, 2)):
        x = torch.from_numpy(rng.standard_normal((T, K)).astype(np.float32)).to(DEV).to(torch.bfloat16)
        idx = torch.from_numpy(rng.integers(0, base + E + 3, T * k).astype(np.int32)).to(DEV)   # some ids outside the bank
        sp = SortedPairs(idx, E, base)
        xs = _gather_rows(x, sp, k)
        ref = _moe_gemm(xs, sp, bank)
        y = torch.zeros_like(ref)
        for bits in bank.distinct_bits:
            _lib.check(lib.jq_moe_gemm_static(xs.data_ptr(), _lib.JQ_BF16, sp.n, xs.stride(0), sp.offsets.data_ptr(), E,
                                              bank.codes_tab.data_ptr(), bank.scales_tab.data_ptr(),
                                              bank.biases_tab.data_ptr(), bank.bits_tab.data_ptr(), _lib.JQ_BF16, N, K,
                                              bits, gs, y.data_ptr(), y.stride(0), _lib.stream_ptr()))
        torch.cuda.synchronize()
        kept = int(sp.offsets[E])
        assert 0 < kept < T * k
        assert torch.equal(y[:kept], ref[:kept])
    assert lib.jq_device_status() == 0
