"""Routed mixture-of-experts over quantized experts.

    ExpertBank        the stacked-expert weight holder (SwitchProj, jang_tools/dsv41/model.py:847-857),
                      optionally with a different bit width per expert
    gather_qmm        <-> mx.gather_qmm call shape of jang_tools/dots3/ops.py:168-192
    route_softmax_topk  softmax -> top-k -> renormalise (dots3/ops.py:159-162 normalisation)
    moe_layer         the layer logic of dsv41/model.py:1206-1245 (sort by expert above 64 pairs,
                      SwiGLU with optional clamp, routing weight applied before down, f32 sum over
                      slots, optional shared expert)

Every matmul runs in libjangq_b200.so: the tensor-core grouped GEMM over expert-sorted rows, or
the gather mat-vec below the sort threshold.
"""
from __future__ import annotations

from typing import Sequence

import torch

from . import _lib, ops
from ._lib import JangqError

SORT_THRESHOLD = 64      # pairs; dsv41/model.py:1206 (n * topk >= 64), mlx-lm SwitchGLU indices.size >= 64


class ExpertBank:
    """Quantized weights of E experts for one projection: y = deq(W[e]) . x.

    Uniform: `weight` int32/uint32 [E, N, K*bits/32], `scales`/`biases` [E, N, K/gs], one
    (bits, group_size) for all experts (the reference's layout).  Mixed: `from_experts` takes one
    (wq, scales, biases, bits) tuple per expert.  Device pointer tables are built once.
    """

    def __init__(self, weight: torch.Tensor, scales: torch.Tensor, biases: torch.Tensor, bits: int,
                 group_size: int = 64):
        dev = _lib.require_cuda(weight, scales, biases)
        weight = ops._as_i32(weight).contiguous()
        scales, biases = scales.contiguous(), biases.contiguous()
        if weight.dim() != 3:
            raise JangqError(_lib.JQ_EINVAL, f"stacked expert weight must be [E, N, K*bits/32], got {tuple(weight.shape)}")
        self.K = ops._check_triple(weight, scales, biases, bits, group_size)
        self.E, self.N = weight.shape[0], weight.shape[1]
        self.group_size = group_size
        self.device, self.sidecar_dtype = dev, scales.dtype
        self._keep = [weight, scales, biases]
        self.weight, self.scales, self.biases = weight, scales, biases
        self.expert_bits = [bits] * self.E
        self._build_tables([weight[e] for e in range(self.E)], [scales[e] for e in range(self.E)],
                           [biases[e] for e in range(self.E)])

    @classmethod
    def from_experts(cls, experts: Sequence[tuple], group_size: int = 64) -> "ExpertBank":
        """experts[e] = (wq [N, K*bits_e/32], scales [N, K/gs], biases, bits_e): per-expert widths."""
        self = cls.__new__(cls)
        ws, ss, bs, bits = [], [], [], []
        for wq, s, b, nb in experts:
            wq = ops._as_i32(wq).contiguous()
            K = ops._check_triple(wq, s, b, nb, group_size)
            ws.append(wq), ss.append(s.contiguous()), bs.append(b.contiguous()), bits.append(int(nb))
            if len(ws) == 1:
                self.K, self.N = K, wq.shape[0]
            elif K != self.K or wq.shape[0] != self.N:
                raise JangqError(_lib.JQ_EINVAL, "all experts of a bank must share [N, K]")
        self.E, self.group_size = len(ws), group_size
        self.device = _lib.require_cuda(*ws, *ss, *bs)
        self.sidecar_dtype = ss[0].dtype
        self._keep = [ws, ss, bs]
        self.weight = self.scales = self.biases = None
        self.expert_bits = bits
        self._build_tables(ws, ss, bs)
        return self

    def _build_tables(self, ws, ss, bs):
        for t in ws + ss + bs:
            if t.data_ptr() % 16:
                raise JangqError(_lib.JQ_EINVAL, "expert tensors must be 16-byte aligned")
        dev = self.device
        self.codes_tab = torch.tensor([t.data_ptr() for t in ws], dtype=torch.int64, device=dev)
        self.scales_tab = torch.tensor([t.data_ptr() for t in ss], dtype=torch.int64, device=dev)
        self.biases_tab = torch.tensor([t.data_ptr() for t in bs], dtype=torch.int64, device=dev)
        self.distinct_bits = sorted(set(self.expert_bits))
        self.bits_tab = (torch.tensor(self.expert_bits, dtype=torch.int32, device=dev)
                         if len(self.distinct_bits) > 1 else None)

    @property
    def gemm_ok(self) -> bool:
        """Shapes the tensor-core grouped GEMM takes: K a multiple of 64, packed rows of 16-byte multiples."""
        return self.K % 64 == 0 and all((self.K * b // 8) % 16 == 0 for b in self.distinct_bits)

    def slice(self, e0: int, e1: int) -> "ExpertBank":
        """Experts [e0, e1) as their own bank (expert-parallel shard), sharing storage."""
        if self.weight is not None:
            return ExpertBank(self.weight[e0:e1], self.scales[e0:e1], self.biases[e0:e1], self.expert_bits[0],
                              self.group_size)
        ws, ss, bs = self._keep
        return ExpertBank.from_experts([(ws[e], ss[e], bs[e], self.expert_bits[e]) for e in range(e0, e1)],
                                       self.group_size)

    def _sidecars_as(self, dtype):
        """The kernels take sidecars in the activation dtype (converted once, then cached)."""
        if self.sidecar_dtype == dtype:
            return self
        cache = self.__dict__.setdefault("_converted", {})
        if dtype not in cache:
            if self.weight is not None:
                cache[dtype] = ExpertBank(self.weight, self.scales.to(dtype), self.biases.to(dtype),
                                          self.expert_bits[0], self.group_size)
            else:
                ws, ss, bs = self._keep
                cache[dtype] = ExpertBank.from_experts([(w, s.to(dtype), b.to(dtype), nb) for w, s, b, nb in
                                                        zip(ws, ss, bs, self.expert_bits)], self.group_size)
        return cache[dtype]


class SortedPairs:
    """Result of jq_moe_sort for one routing decision; reused by gate, up and down."""

    def __init__(self, idx_flat: torch.Tensor, num_experts: int, expert_base: int = 0, tile_m: int | None = None):
        lib = _lib.load()
        dev = idx_flat.device
        n = idx_flat.numel()
        self.n, self.E = n, num_experts
        self.tile_m = tile_m or _lib.MOE_TILE_M
        self.max_tiles = int(lib.jq_moe_sort_max_tiles(n, num_experts, self.tile_m))
        i32 = dict(dtype=torch.int32, device=dev)
        self.order = torch.empty(max(n, 1), **i32)
        self.inv = torch.empty(max(n, 1), **i32)
        self.offsets = torch.empty(num_experts + 1, **i32)
        self.tile_expert = torch.empty(max(self.max_tiles, 1), **i32)
        self.tile_row0 = torch.empty(max(self.max_tiles, 1), **i32)
        self.num_tiles = torch.empty(1, **i32)
        _lib.check(lib.jq_moe_sort(idx_flat.data_ptr(), n, num_experts, expert_base, self.order.data_ptr(),
                                   self.inv.data_ptr(), self.offsets.data_ptr(), self.tile_m,
                                   self.tile_expert.data_ptr(), self.tile_row0.data_ptr(), self.num_tiles.data_ptr(),
                                   _lib.stream_ptr(dev)))
        self.count_ptr = self.offsets.data_ptr() + 4 * num_experts      # device address of the kept-pair count


def _gather_rows(src: torch.Tensor, sp: SortedPairs, div: int) -> torch.Tensor:
    lib = _lib.load()
    dst = torch.empty((max(sp.n, 1), src.shape[1]), dtype=src.dtype, device=src.device)
    _lib.check(lib.jq_gather_rows(src.data_ptr(), src.stride(0), sp.order.data_ptr(), sp.count_ptr, div, dst.data_ptr(),
                                  dst.stride(0), src.shape[1], sp.n, _lib.dtype_id(src.dtype), _lib.stream_ptr(src.device)))
    return dst


def _moe_gemm(x_sorted: torch.Tensor, sp: SortedPairs, bank: ExpertBank) -> torch.Tensor:
    lib = _lib.load()
    bank = bank._sidecars_as(x_sorted.dtype)
    y = torch.empty((x_sorted.shape[0], bank.N), dtype=x_sorted.dtype, device=x_sorted.device)
    for bits in bank.distinct_bits:
        _lib.check(lib.jq_moe_gemm_tiled(x_sorted.data_ptr(), _lib.dtype_id(x_sorted.dtype), sp.n, x_sorted.stride(0),
                                         sp.offsets.data_ptr(), sp.tile_expert.data_ptr(), sp.tile_row0.data_ptr(),
                                         sp.num_tiles.data_ptr(), sp.max_tiles, sp.tile_m, bank.codes_tab.data_ptr(),
                                         bank.scales_tab.data_ptr(), bank.biases_tab.data_ptr(),
                                         bank.bits_tab.data_ptr() if bank.bits_tab is not None else None,
                                         _lib.dtype_id(bank.sidecar_dtype), bank.N, bank.K, bits, bank.group_size,
                                         y.data_ptr(), y.stride(0), _lib.stream_ptr(x_sorted.device)))
    return y


def _gather_qgemv(x: torch.Tensor, x_div: int, pair_expert: torch.Tensor, bank: ExpertBank,
                  flags: int = 0, expert_base: int = 0) -> torch.Tensor:
    """y[p] = deq(W[pair_expert[p] - expert_base]) . x[p // x_div].  Pairs whose expert is not in the bank
    get a zero row (written by the kernel)."""
    lib = _lib.load()
    bank = bank._sidecars_as(x.dtype)
    P = pair_expert.numel()
    y = torch.empty((P, bank.N), dtype=x.dtype, device=x.device)
    for bits in bank.distinct_bits:
        _lib.check(lib.jq_gather_qgemv2(x.data_ptr(), _lib.dtype_id(x.dtype), x.stride(0), x_div, pair_expert.data_ptr(),
                                        P, bank.codes_tab.data_ptr(), bank.scales_tab.data_ptr(),
                                        bank.biases_tab.data_ptr(), None, None, None,
                                        bank.bits_tab.data_ptr() if bank.bits_tab is not None else None, bank.E,
                                        _lib.dtype_id(bank.sidecar_dtype), bank.N, bank.K, bits, bank.group_size,
                                        y.data_ptr(), None, y.stride(0), expert_base, flags, _lib.stream_ptr(x.device)))
    return y


def _gather_qgemv_pair(x: torch.Tensor, x_div: int, pair_expert: torch.Tensor, bank_a: ExpertBank, bank_b: ExpertBank,
                       flags: int = 0, expert_base: int = 0):
    """Two banks of equal shape and width (gate, up) over the same rows of x in one launch."""
    same = (bank_a.N == bank_b.N and bank_a.K == bank_b.K and bank_a.group_size == bank_b.group_size and
            bank_a.E == bank_b.E and bank_a.bits_tab is None and bank_b.bits_tab is None and
            bank_a.distinct_bits == bank_b.distinct_bits and len(bank_a.distinct_bits) == 1)
    if not same:
        return (_gather_qgemv(x, x_div, pair_expert, bank_a, flags, expert_base),
                _gather_qgemv(x, x_div, pair_expert, bank_b, flags, expert_base))
    lib = _lib.load()
    a, b = bank_a._sidecars_as(x.dtype), bank_b._sidecars_as(x.dtype)
    P = pair_expert.numel()
    y = torch.empty((2, P, a.N), dtype=x.dtype, device=x.device)
    _lib.check(lib.jq_gather_qgemv2(x.data_ptr(), _lib.dtype_id(x.dtype), x.stride(0), x_div, pair_expert.data_ptr(), P,
                                    a.codes_tab.data_ptr(), a.scales_tab.data_ptr(), a.biases_tab.data_ptr(),
                                    b.codes_tab.data_ptr(), b.scales_tab.data_ptr(), b.biases_tab.data_ptr(), None, a.E,
                                    _lib.dtype_id(a.sidecar_dtype), a.N, a.K, a.distinct_bits[0], a.group_size,
                                    y[0].data_ptr(), y[1].data_ptr(), y.stride(1), expert_base, flags,
                                    _lib.stream_ptr(x.device)))
    return y[0], y[1]


def gather_qmm(x: torch.Tensor, w, scales: torch.Tensor | None = None, biases: torch.Tensor | None = None,
               rhs_indices: torch.Tensor | None = None, lhs_indices: torch.Tensor | None = None,
               transpose: bool = True, group_size: int = 64, bits: int = 4, sorted_indices: bool = False) -> torch.Tensor:
    """y[r] = x[lhs[r]] . deq(w[rhs[r]])^T for stacked experts w [E, N, K*bits/32] (or an ExpertBank).

    x is [R0, K] (singleton middle dims are squeezed); rhs_indices [R] or [T, k]; lhs_indices [R]
    or None, in which case row r of x is used when R0 == R, and row r // k when rhs is [T, k] with
    R0 == T (MLX broadcasts the batch dims the same way).  As in the reference
    (dots3/ops.py:175-176) sorted_indices=True needs lhs_indices.  Returns [R, N].
    """
    if not transpose:
        raise JangqError(_lib.JQ_EUNSUPPORTED, "gather_qmm: only transpose=True is provided")
    if rhs_indices is None:
        raise JangqError(_lib.JQ_EINVAL, "gather_qmm needs rhs_indices")
    if sorted_indices and lhs_indices is None:
        raise ValueError("sorted_indices=True requires lhs_indices")
    bank = w if isinstance(w, ExpertBank) else ExpertBank(w, scales, biases, bits, group_size)
    dev = _lib.require_cuda(x, rhs_indices)
    x2 = x.reshape(-1, x.shape[-1])
    if x2.dtype not in (torch.bfloat16, torch.float16):
        raise JangqError(_lib.JQ_EINVAL, f"activations must be bfloat16 or float16, got {x2.dtype}")
    if x2.shape[1] != bank.K:
        raise JangqError(_lib.JQ_EINVAL, f"x has {x2.shape[1]} features, experts expect {bank.K}")
    k = rhs_indices.shape[-1] if rhs_indices.dim() == 2 else 1
    rhs = rhs_indices.reshape(-1).to(torch.int32).contiguous()
    R = rhs.numel()
    if lhs_indices is not None:
        lhs = lhs_indices.reshape(-1).to(torch.int64)
        if lhs.numel() != R:
            raise JangqError(_lib.JQ_EINVAL, "lhs_indices and rhs_indices differ in length")
        x2, x_div = x2.index_select(0, lhs), 1
    elif x2.shape[0] == R:
        x_div = 1
    elif rhs_indices.dim() == 2 and x2.shape[0] == rhs_indices.shape[0]:
        x_div = k
    else:
        raise JangqError(_lib.JQ_EINVAL, f"cannot match {x2.shape[0]} rows of x with {R} indices")
    x2 = x2.contiguous()
    with torch.cuda.device(dev):
        if R < SORT_THRESHOLD or not bank.gemm_ok:
            return _gather_qgemv(x2, x_div, rhs, bank)
        sp = SortedPairs(rhs, bank.E)
        xs = _gather_rows(x2, sp, x_div)
        ys = _moe_gemm(xs, sp, bank)
        return ys.index_select(0, sp.inv.to(torch.int64))


def route_softmax_topk(logits: torch.Tensor, k: int, renorm: bool = True, scale: float = 1.0):
    """(idx int32 [T, k], w float32 [T, k]): softmax over experts in f32, top-k by score (ties to
    the lower id, as jang_tools/dsv41/metal_decode.py:1141), w / (sum w + 1e-20) * scale."""
    if logits.is_cuda and logits.dim() == 2 and logits.shape[1] <= 1024 and \
            logits.dtype in (torch.float32, torch.bfloat16, torch.float16):
        lib = _lib.load()
        if logits.stride(1) != 1:
            logits = logits.contiguous()
        T, E = logits.shape
        idx = torch.empty((T, k), dtype=torch.int32, device=logits.device)
        wts = torch.empty((T, k), dtype=torch.float32, device=logits.device)
        with torch.cuda.device(logits.device):
            _lib.check(lib.jq_moe_topk(logits.data_ptr(), _lib.dtype_id(logits.dtype), logits.stride(0), T, E, k,
                                       1 if renorm else 0, float(scale), idx.data_ptr(), wts.data_ptr(),
                                       _lib.stream_ptr(logits.device)))
        return idx, wts
    p = torch.softmax(logits.float(), dim=-1)
    w, idx = torch.topk(p, k, dim=-1, sorted=True)
    if renorm:
        w = w / (w.sum(dim=-1, keepdim=True) + 1e-20)
    return idx.to(torch.int32), (w * scale).float()


def route_from_hidden(x: torch.Tensor, router_w: torch.Tensor, k: int, renorm: bool = True, scale: float = 1.0):
    """route_softmax_topk(x @ router_w.T, k) in one launch for few tokens: (idx int32 [T, k], w f32 [T, k]).
    x [T, H] and router_w [E, H] share a 16-bit dtype; E <= 1024."""
    lib = _lib.load()
    dev = _lib.require_cuda(x, router_w)
    if x.dtype != router_w.dtype or x.dtype not in (torch.bfloat16, torch.float16):
        raise JangqError(_lib.JQ_EINVAL, "route_from_hidden: x and router_w must share a 16-bit dtype")
    T, H = x.shape
    E = router_w.shape[0]
    x, router_w = x.contiguous(), router_w.contiguous()
    idx = torch.empty((T, k), dtype=torch.int32, device=dev)
    w = torch.empty((T, k), dtype=torch.float32, device=dev)
    cnt, ws = _route_workspace(dev, T, E)
    with torch.cuda.device(dev):
        _lib.check(lib.jq_moe_route(x.data_ptr(), _lib.dtype_id(x.dtype), x.stride(0), T, H, router_w.data_ptr(), E, k,
                                    1 if renorm else 0, float(scale), idx.data_ptr(), w.data_ptr(), cnt.data_ptr(),
                                    ws.data_ptr(), _lib.stream_ptr(dev)))
    return idx, w


def route_norm_from_hidden(x: torch.Tensor, res: torch.Tensor, router_w: torch.Tensor, k: int, renorm: bool = True,
                           scale: float = 1.0, eps: float | None = None):
    """(rms_norm(x + res), idx, w): residual_rmsnorm followed by route_from_hidden in one launch."""
    lib = _lib.load()
    dev = _lib.require_cuda(x, res, router_w)
    if x.dtype != router_w.dtype or x.dtype != res.dtype or x.dtype not in (torch.bfloat16, torch.float16):
        raise JangqError(_lib.JQ_EINVAL, "route_norm_from_hidden: x, res and router_w must share a 16-bit dtype")
    T, H = x.shape
    E = router_w.shape[0]
    x, res, router_w = x.contiguous(), res.contiguous(), router_w.contiguous()
    if eps is None:
        eps = torch.finfo(x.dtype).eps
    xo = torch.empty_like(x)
    idx = torch.empty((T, k), dtype=torch.int32, device=dev)
    w = torch.empty((T, k), dtype=torch.float32, device=dev)
    cnt, ws = _route_workspace(dev, T, E)
    with torch.cuda.device(dev):
        _lib.check(lib.jq_moe_route_norm(x.data_ptr(), res.data_ptr(), _lib.dtype_id(x.dtype), T, H, float(eps),
                                         xo.data_ptr(), router_w.data_ptr(), E, k, 1 if renorm else 0, float(scale),
                                         idx.data_ptr(), w.data_ptr(), cnt.data_ptr(), ws.data_ptr(), _lib.stream_ptr(dev)))
    return xo, idx, w


_ROUTE_WS = {}


def _route_workspace(dev, T: int, E: int):
    """(counters, logits scratch) of the router kernel, kept per device and stream: calls on one stream
    follow each other, and the kernel leaves the counters at zero."""
    key = (dev.type, dev.index, torch.cuda.current_stream(dev).cuda_stream)
    cnt, ws = _ROUTE_WS.get(key, (None, None))
    if cnt is None or cnt.numel() < T:
        cnt = torch.zeros(max(T, 1024), dtype=torch.int32, device=dev)
    if ws is None or ws.numel() < T * E:
        ws = torch.empty(max(T * E, 1 << 16), dtype=torch.float32, device=dev)
    _ROUTE_WS[key] = (cnt, ws)
    return cnt, ws


def residual_rmsnorm(x: torch.Tensor, y: torch.Tensor, eps: float | None = None, k: int = 1) -> torch.Tensor:
    """rms_norm(x + y) without weight, f32 arithmetic, one launch; y [T, H] may be f32 or x's dtype, or
    (k > 1, x's dtype) the [T*k, H] slot rows of the routed experts, which are summed in slot order.  Glue of
    the synthetic decode stacks, not part of the reference's quantized path."""
    lib = _lib.load()
    dev = _lib.require_cuda(x, y)
    T, H = x.shape
    x, y = x.contiguous(), y.contiguous()
    if y.shape != (T * k, H):
        raise JangqError(_lib.JQ_EINVAL, f"residual_rmsnorm: y must be [{T * k}, {H}], got {tuple(y.shape)}")
    if eps is None:
        eps = torch.finfo(x.dtype).eps
    out = torch.empty_like(x)
    yf = y.dtype == torch.float32
    with torch.cuda.device(dev):
        _lib.check(lib.jq_residual_rmsnorm(x.data_ptr(), None if yf else y.data_ptr(), y.data_ptr() if yf else None, k, T, H,
                                           float(eps), out.data_ptr(), _lib.dtype_id(x.dtype), _lib.stream_ptr(dev)))
    return out


def _shared_expert(x: torch.Tensor, shared, swiglu_limit: float) -> torch.Tensor:
    """down(silu(gate x) * up x) of the always-on expert (`_shared`, dsv41/model.py:1237-1245): gate and up
    as one fused mat-vec launch for few rows, the SwiGLU kernel without routing weights, then down.  All three
    products run in libjangq_b200.so."""
    lib = _lib.load()
    sg, su, sd = shared
    T = x.shape[0]
    dev = x.device
    same = (sg.in_features == su.in_features and sg.out_features == su.out_features and sg.bits == su.bits and
            sg.group_size == su.group_size)
    if T <= _lib.QGEMV_MAX_M and same and sg.scales.dtype == x.dtype and su.scales.dtype == x.dtype:
        gu = torch.empty((2, T, sg.out_features), dtype=x.dtype, device=dev)
        flags = _lib.JQ_GEMV_STATIC_WEIGHTS if (getattr(sg, "static_weights", False) and
                                                getattr(su, "static_weights", False)) else 0
        ops.qgemv_fused(x, [sg, su], [gu[0], gu[1]], flags)
        g2, u2 = gu[0], gu[1]
    else:
        g2, u2 = sg(x), su(x)
    I2 = g2.shape[1]
    h2 = torch.empty((T, I2), dtype=x.dtype, device=dev)
    _lib.check(lib.jq_moe_swiglu(g2.data_ptr(), u2.data_ptr(), g2.stride(0), None, None, None, h2.data_ptr(),
                                 h2.stride(0), I2, T, float(swiglu_limit), _lib.dtype_id(x.dtype), _lib.stream_ptr(dev)))
    return sd(h2)


def moe_layer(x: torch.Tensor, idx: torch.Tensor, w: torch.Tensor, gate: ExpertBank, up: ExpertBank,
              down: ExpertBank, swiglu_limit: float = 0.0, shared=None, expert_base: int = 0,
              out_f32: bool = False, all_local: bool | None = None, return_slots: bool = False,
              static_weights: bool = False, few_token_path: bool | None = None, few_local: bool = False) -> torch.Tensor:
    """Routed SwiGLU experts: out[t] = sum_j down_e( silu(gate_e x_t) * up_e x_t * w[t, j] ), e = idx[t, j].

    x [T, H] bf16/f16; idx [T, k] int; w [T, k] f32.  Follows dsv41/model.py:1206-1245.  With
    `expert_base` the banks hold experts [expert_base, expert_base + E) only and the other
    pairs contribute nothing (expert parallelism).  `shared` = (gate, up, down) JANGLinear-like
    modules of an always-on expert, added in f32.  Returns [T, H] in x.dtype (f32 if out_f32).
    all_local is accepted for compatibility and ignored (the kernels zero the rows of skipped pairs
    themselves).  return_slots=True
    (few-token path only) returns the [T*k, H] rows before the combine, for a caller that fuses the sum.
    static_weights=True promises that the expert weights are not written by earlier work on the stream, so
    the few-token mat-vecs may prefetch them while their predecessor still runs.  few_local says that most
    pairs name experts of other ranks (up to 128 pairs then stay on the integer gather).  few_token_path forces
    (True) or forbids (False) the unsorted gather mat-vec path; default: below 64 pairs, as the reference.
    """
    lib = _lib.load()
    dev = _lib.require_cuda(x, idx, w)
    T, H = x.shape
    k = idx.shape[1]
    P = T * k
    idx32 = idx.reshape(-1).to(torch.int32).contiguous()
    wf = w.reshape(-1).float().contiguous()
    # rows with a leading dimension are taken as they are (the slot rows of the expert-parallel exchange carry
    # 16 bytes of routing data behind each row); anything else is made contiguous
    if not (x.dim() == 2 and x.stride(1) == 1 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0):
        x = x.contiguous()
    dt = _lib.dtype_id(x.dtype)
    st = _lib.stream_ptr(dev)
    I = gate.N
    with torch.cuda.device(dev):
        use_sorted = P >= SORT_THRESHOLD if few_token_path is None else not few_token_path
        if use_sorted and gate.gemm_ok and up.gemm_ok and down.gemm_ok:
            # experts with at least 256 rows on average: 256-row tiles, two accumulators per CTA share every
            # dequantized weight tile (bf16, all three projections at least 256 wide)
            big = (x.dtype == torch.bfloat16 and min(gate.N, up.N, down.N) >= 256 and P >= 256 * gate.E)
            sp = SortedPairs(idx32, gate.E, expert_base, tile_m=256 if big else 128)
            xs = _gather_rows(x, sp, k)
            g = _moe_gemm(xs, sp, gate)
            u = _moe_gemm(xs, sp, up)
            h = torch.empty((max(P, 1), I), dtype=x.dtype, device=dev)
            _lib.check(lib.jq_moe_swiglu(g.data_ptr(), u.data_ptr(), g.stride(0), wf.data_ptr(), sp.order.data_ptr(),
                                         sp.count_ptr, h.data_ptr(), h.stride(0), I, P, float(swiglu_limit), dt, st))
            y = _moe_gemm(h, sp, down)
            inv_ptr = sp.inv.data_ptr()
        else:
            flags = _lib.JQ_GEMV_STATIC_WEIGHTS if static_weights else 0
            if few_local:        # experts sharded over ranks: most pairs are other ranks' (JQ_GATHER_FEW_LOCAL)
                flags |= _lib.JQ_GATHER_FEW_LOCAL
            g, u = _gather_qgemv_pair(x, k, idx32, gate, up, flags, expert_base)
            if len(down.distinct_bits) == 1 and down.bits_tab is None:
                # SwiGLU folded into the down gather (one launch for up to 16 pairs, two through h otherwise)
                dn = down._sidecars_as(x.dtype)
                y = torch.empty((P, dn.N), dtype=x.dtype, device=dev)
                h = torch.empty((P, I), dtype=x.dtype, device=dev)     # only shapes off the one-launch path touch it
                _lib.check(lib.jq_gather_qgemv_swiglu(g.data_ptr(), u.data_ptr(), dt, g.stride(0), wf.data_ptr(),
                                                      float(swiglu_limit), idx32.data_ptr(), P, dn.codes_tab.data_ptr(),
                                                      dn.scales_tab.data_ptr(), dn.biases_tab.data_ptr(), None, dn.E,
                                                      _lib.dtype_id(dn.sidecar_dtype), dn.N, dn.K, dn.distinct_bits[0],
                                                      dn.group_size, y.data_ptr(), y.stride(0), expert_base, flags,
                                                      h.data_ptr(), st))
            else:
                h = torch.empty((P, I), dtype=x.dtype, device=dev)
                _lib.check(lib.jq_moe_swiglu(g.data_ptr(), u.data_ptr(), g.stride(0), wf.data_ptr(), None, None,
                                             h.data_ptr(), h.stride(0), I, P, float(swiglu_limit), dt, st))
                y = _gather_qgemv(h, 1, idx32, down, flags, expert_base)
            if return_slots and shared is None:
                return y        # [T*k, H]: the caller sums the k rows of a token (routing weights already applied)
            # pairs of other ranks' experts were skipped by the kernels and their rows stay zero
            inv_ptr = None
        ys = _shared_expert(x, shared, swiglu_limit) if shared is not None else None
        acc = torch.empty((T, H), dtype=torch.float32, device=dev) if out_f32 else None
        out = None if out_f32 else torch.empty((T, H), dtype=x.dtype, device=dev)
        _lib.check(lib.jq_moe_combine_shared(y.data_ptr(), y.stride(0), inv_ptr, None, T, k, H,
                                             ys.data_ptr() if ys is not None else None,
                                             ys.stride(0) if ys is not None else 0,
                                             out.data_ptr() if out is not None else None, H,
                                             acc.data_ptr() if acc is not None else None, dt, st))
        return acc if out_f32 else out
