"""Expert parallelism for the routed-MoE path: experts sharded E/G per GPU, one process per GPU.

The reference has no multi-device code; this is the one place the path shards naturally (by
expert), with exactly one exchange each way:

  replicated tokens (batch-1 / small-batch decode: every rank holds the same rows):
      each rank runs its own experts on all rows (pairs of other ranks' experts are skipped by the
      kernels) and the partial sums are added over NVLink: by `peer_combine_residual_rmsnorm` (peer stores
      inside the kernel that also does the residual and the norm) or with one NCCL all-reduce;
  sharded tokens (prefill / large batches: every rank holds its own rows):
      dispatch  = all_to_all_single of the (row, local expert id, routing weight) triples, ordered by
                  destination rank, split sizes from a histogram of the top-k ids;
      local     = the rank's experts on the rows it received;
      combine   = the reverse all_to_all_single and the sum over each token's k slots.

`local_fn(x_rows, e_local, w_rows) -> y_rows` does the expert math; on GPUs it is
`local_experts_fn(gate, up, down)` (the CUDA kernels); the process-group logic itself is
device-agnostic so that it is tested with gloo on CPU ranks.
"""
from __future__ import annotations

import ctypes
from typing import Callable

import torch
import torch.distributed as dist

from . import _lib


def validate_splits(send_counts: torch.Tensor, recv_counts: torch.Tensor, n_pairs: int) -> None:
    """Host-side check of the all-to-all split tables before anything is launched."""
    if int(send_counts.sum()) != n_pairs:
        raise ValueError(f"dispatch splits cover {int(send_counts.sum())} pairs, expected {n_pairs}")
    if bool((send_counts < 0).any()) or bool((recv_counts < 0).any()):
        raise ValueError("negative split size")


def dispatch_combine(x: torch.Tensor, idx: torch.Tensor, w: torch.Tensor, num_experts: int, local_fn: Callable,
                     group=None) -> torch.Tensor:
    """Sharded-token expert parallelism.  x [T, H] (this rank's rows), idx [T, k] global expert ids,
    w [T, k] f32.  Returns this rank's [T, H] output in float32."""
    world = dist.get_world_size(group)
    if num_experts % world:
        raise ValueError(f"{num_experts} experts do not shard over {world} ranks")
    e_local = num_experts // world
    T, H = x.shape
    k = idx.shape[1]
    flat = idx.reshape(-1).to(torch.int64)
    if bool(((flat < 0) | (flat >= num_experts)).any()):
        raise ValueError("expert id out of range")
    dest = flat // e_local
    order = torch.argsort(dest, stable=True)                       # pairs grouped by destination rank
    send_counts = torch.bincount(dest, minlength=world)
    recv_counts = torch.empty_like(send_counts)
    dist.all_to_all_single(recv_counts, send_counts, group=group)
    validate_splits(send_counts, recv_counts, T * k)
    s_list, r_list = send_counts.tolist(), recv_counts.tolist()
    n_recv = sum(r_list)

    x_send = x.index_select(0, order // k).contiguous()
    meta_send = torch.stack([(flat[order] % e_local).to(torch.float32),
                             w.reshape(-1).to(torch.float32)[order]], dim=1).contiguous()
    x_recv = torch.empty((n_recv, H), dtype=x.dtype, device=x.device)
    meta_recv = torch.empty((n_recv, 2), dtype=torch.float32, device=x.device)
    dist.all_to_all_single(x_recv, x_send, r_list, s_list, group=group)
    dist.all_to_all_single(meta_recv, meta_send, r_list, s_list, group=group)

    y_recv = local_fn(x_recv, meta_recv[:, 0].to(torch.int32), meta_recv[:, 1].contiguous())
    y_recv = y_recv.to(x.dtype).contiguous()

    y_back = torch.empty((T * k, H), dtype=x.dtype, device=x.device)
    dist.all_to_all_single(y_back, y_recv, s_list, r_list, group=group)
    out = torch.zeros((T, H), dtype=torch.float32, device=x.device)
    out.index_add_(0, order // k, y_back.float())                   # sum over each token's slots
    return out


def slot_capacity(n_pairs: int, world: int, factor: float = 1.25) -> int:
    """Slots per (source, destination) pair of ranks for dispatch_combine_slots: the mean share of a rank's
    pairs times `factor`, plus slack for small batches, a multiple of 8, never more than all pairs."""
    c = int(n_pairs / world * factor) + 32
    return min(max(n_pairs, 8), (c + 7) // 8 * 8)


def dispatch_combine_slots(x: torch.Tensor, idx: torch.Tensor, w: torch.Tensor, num_experts: int, local_fn: Callable,
                           capacity: int, group=None):
    """Sharded-token expert parallelism without a host read-back: every (source, destination) pair of ranks owns
    `capacity` row slots (the same number on every rank), so both exchanges are equal-split all_to_all_single calls
    of fixed size and no split table ever reaches the host.  A row travels with its local expert id and routing
    weight packed behind its H values (16 bytes), so the dispatch is ONE collective; empty slots carry expert id
    -1 and local_fn ignores them (the CUDA kernels drop pairs whose expert is outside the bank).  The return trip
    sends the slot rows back and each token adds its k slots in slot order.

    Returns (out [T, H] float32, overflow): `overflow` is a 0-dim bool tensor on x's device, true when some
    destination got more than `capacity` pairs -- their rows are missing from `out`; the caller reads it after
    the step (not in its middle) and repeats the step with dispatch_combine or a larger capacity."""
    world = dist.get_world_size(group)
    if num_experts % world:
        raise ValueError(f"{num_experts} experts do not shard over {world} ranks")
    e_local = num_experts // world
    T, H = x.shape
    k = idx.shape[1]
    P, C = T * k, int(capacity)
    es = x.element_size()
    if C < 1 or (H * es) % 4:
        raise ValueError("capacity must be positive and rows a multiple of 4 bytes")
    dev = x.device
    Hp = H + 16 // es                                               # row + 16 bytes: expert id, weight, 8 spare
    mcol = H * es // 4                                              # int32 / float32 column of the expert id
    if x.is_cuda and es == 2 and H % 8 == 0:
        return _dispatch_combine_slots_cuda(x, idx, w, num_experts, local_fn, C, group, world, Hp, mcol)
    flat = idx.reshape(-1).to(torch.int64)
    dest = torch.div(flat, e_local, rounding_mode="floor").clamp_(0, world - 1)
    order = torch.sort(dest, stable=True).indices                  # pairs grouped by destination rank
    counts = torch.zeros(world, dtype=torch.int64, device=dev).scatter_add_(0, dest, torch.ones_like(dest))
    first = torch.cumsum(counts, 0) - counts
    sdest = dest[order]
    pos = torch.arange(P, device=dev) - first[sdest]               # position among the pairs of its destination
    valid = pos < C
    slot = torch.where(valid, sdest * C + pos, torch.full_like(pos, world * C))   # row world*C: never sent
    overflow = (counts > C).any()

    send = torch.empty((world * C + 1, Hp), dtype=x.dtype, device=dev)
    send_i, send_f = send.view(torch.int32), send.view(torch.float32)
    send_i[:, mcol] = -1
    send[:, :H].index_copy_(0, slot, x.index_select(0, torch.div(order, k, rounding_mode="floor")))
    send_i[:, mcol].index_copy_(0, slot, (flat[order] % e_local).to(torch.int32))
    send_f[:, mcol + 1].index_copy_(0, slot, w.reshape(-1).to(torch.float32)[order])
    recv = torch.empty((world * C, Hp), dtype=x.dtype, device=dev)
    dist.all_to_all_single(recv, send[:world * C], group=group)

    y_recv = local_fn(recv[:, :H], recv.view(torch.int32)[:, mcol], recv.view(torch.float32)[:, mcol + 1])
    y_recv = y_recv.to(x.dtype).contiguous()
    y_back = torch.empty_like(y_recv)
    dist.all_to_all_single(y_back, y_recv, group=group)

    slot_of_pair = torch.empty(P, dtype=torch.int32, device=dev)
    slot_of_pair.index_copy_(0, order, torch.where(valid, slot, torch.full_like(slot, -1)).to(torch.int32))
    out = torch.empty((T, y_back.shape[1]), dtype=torch.float32, device=dev)
    if x.is_cuda:
        lib = _lib.load()
        with torch.cuda.device(dev):
            _lib.check(lib.jq_moe_combine(y_back.data_ptr(), y_back.stride(0), slot_of_pair.data_ptr(), None, T, k,
                                          y_back.shape[1], None, y_back.shape[1], out.data_ptr(),
                                          _lib.dtype_id(x.dtype), _lib.stream_ptr(dev)))
    else:
        sp = slot_of_pair.long().reshape(T, k)
        rows = y_back.float()[sp.clamp(min=0)]                     # [T, k, D]; slot -1 (dropped) reads row 0: masked
        rows = torch.where((sp >= 0)[..., None], rows, torch.zeros((), dtype=rows.dtype))
        out = rows.sum(1) if T else out
    return out, overflow


def _dispatch_combine_slots_cuda(x, idx, w, num_experts, local_fn, C, group, world, Hp, mcol):
    """dispatch_combine_slots on a GPU: the slot rows are packed by jq_ep_pack_slots (two launches), the k slots of
    a token are added by jq_moe_combine; in between only the two collectives and local_fn."""
    lib = _lib.load()
    T, H = x.shape
    k = idx.shape[1]
    dev = x.device
    if x.stride(1) != 1 or x.stride(0) % 8 or x.data_ptr() % 16:
        x = x.contiguous()
    idx32 = idx.reshape(-1).to(torch.int32).contiguous()
    wf = w.reshape(-1).to(torch.float32).contiguous()
    send = torch.empty((world * C, Hp), dtype=x.dtype, device=dev)
    recv = torch.empty_like(send)
    slot_of_pair = torch.empty(max(T * k, 1), dtype=torch.int32, device=dev)
    scratch = torch.empty(world + 1, dtype=torch.int32, device=dev)           # counters, then the overflow word
    st = _lib.stream_ptr(dev)
    with torch.cuda.device(dev):
        _lib.check(lib.jq_ep_pack_slots(x.data_ptr(), x.stride(0), idx32.data_ptr(), wf.data_ptr(), T, k, H, num_experts,
                                        world, C, send.data_ptr(), slot_of_pair.data_ptr(), scratch.data_ptr(),
                                        scratch[world:].data_ptr(), st))
        dist.all_to_all_single(recv, send, group=group)
        y_recv = local_fn(recv[:, :H], recv.view(torch.int32)[:, mcol], recv.view(torch.float32)[:, mcol + 1])
        y_recv = y_recv.to(x.dtype).contiguous()
        y_back = torch.empty_like(y_recv)
        dist.all_to_all_single(y_back, y_recv, group=group)
        D = y_back.shape[1]
        out = torch.empty((T, D), dtype=torch.float32, device=dev)
        _lib.check(lib.jq_moe_combine(y_back.data_ptr(), y_back.stride(0), slot_of_pair.data_ptr(), None, T, k, D, None, D,
                                      out.data_ptr(), _lib.dtype_id(x.dtype), st))
    return out, scratch[world] != 0


def replicated_tokens(x: torch.Tensor, idx: torch.Tensor, w: torch.Tensor, partial_fn: Callable, group=None) -> torch.Tensor:
    """Replicated-token expert parallelism: partial_fn(x, idx, w) -> f32 [T, H] over this rank's experts
    only; one all-reduce adds the ranks' partial sums."""
    out = partial_fn(x, idx, w)
    dist.all_reduce(out, op=dist.ReduceOp.SUM, group=group)
    return out


def gathered_tokens(x: torch.Tensor, idx: torch.Tensor, w: torch.Tensor, partial_fn: Callable, group=None) -> torch.Tensor:
    """Small-batch expert parallelism without any host synchronisation (CUDA-graph capturable):
    every rank holds its own T rows; all-gather rows, ids and weights (fixed sizes), run this rank's
    experts over all world*T rows, reduce-scatter the f32 partial sums.  Returns this rank's [T, H]."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    T, H = x.shape
    k = idx.shape[1]
    x_all = torch.empty((world * T, H), dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(x_all, x.contiguous(), group=group)
    meta = torch.cat([idx.to(torch.float32), w.to(torch.float32)], dim=1).contiguous()       # [T, 2k]
    meta_all = torch.empty((world * T, 2 * k), dtype=torch.float32, device=x.device)
    dist.all_gather_into_tensor(meta_all, meta, group=group)
    part = partial_fn(x_all, meta_all[:, :k].to(torch.int32), meta_all[:, k:].contiguous())   # [world*T, H] f32
    out = torch.empty((T, H), dtype=torch.float32, device=x.device)
    try:
        dist.reduce_scatter_tensor(out, part.contiguous(), op=dist.ReduceOp.SUM, group=group)
    except (RuntimeError, NotImplementedError):       # backends without reduce-scatter (gloo)
        dist.all_reduce(part, op=dist.ReduceOp.SUM, group=group)
        out = part[rank * T:(rank + 1) * T].clone()
    return out


def local_experts_fn(gate, up, down, swiglu_limit: float = 0.0, out_f32: bool = True):
    """local_fn for dispatch_combine / dispatch_combine_slots on a GPU: rows with one (local) expert and weight
    each; rows whose expert id is outside the bank (the empty slots, id -1) give zero rows."""
    from .moe import moe_layer

    def fn(x_rows, e_local, w_rows):
        if x_rows.shape[0] == 0:
            return torch.zeros_like(x_rows, dtype=torch.float32)
        return moe_layer(x_rows, e_local[:, None], w_rows[:, None], gate, up, down, swiglu_limit=swiglu_limit,
                         out_f32=out_f32)
    return fn


def partial_experts_fn(gate, up, down, expert_base: int, swiglu_limit: float = 0.0):
    """partial_fn for replicated_tokens on a GPU: this rank's experts [expert_base, expert_base + E_local)."""
    from .moe import moe_layer

    def fn(x, idx, w):
        return moe_layer(x, idx, w, gate, up, down, swiglu_limit=swiglu_limit, expert_base=expert_base, out_f32=True)
    return fn


class PeerExchange:
    """Exchange buffers for `peer_combine_residual_rmsnorm`: one buffer per rank, every rank holding the device
    addresses of all of them.  `PeerExchange.connect(group, tcap, H, device)` allocates this rank's buffer in
    torch's symmetric memory (which maps the peers' buffers for plain loads and stores over NVLink) and
    exchanges the addresses; `PeerExchange.emulated(world, tcap, H, device)` puts every rank's buffer on one
    GPU for the single-launch emulation used by the tests."""

    def __init__(self, buffers, ptrs, rank, world, tcap, H, device, handle=None):
        self.buffers, self.ptrs, self.rank, self.world, self.tcap, self.H = buffers, ptrs, rank, world, tcap, H
        self.device, self.handle = device, handle
        self.counters = torch.zeros((world if rank < 0 else 1) * tcap, dtype=torch.int32, device=device)
        self._ptr_array = (ctypes.c_uint64 * world)(*ptrs)

    @staticmethod
    def nbytes(tcap: int, H: int) -> int:
        return int(_lib.load().jq_ep_buffer_bytes(tcap, H))

    @classmethod
    def connect(cls, group, tcap: int, H: int, device) -> "PeerExchange":
        import torch.distributed._symmetric_memory as symm_mem
        group = group if group is not None else dist.group.WORLD
        n = cls.nbytes(tcap, H) // 4
        buf = symm_mem.empty(n, dtype=torch.float32, device=device)
        buf.zero_()
        handle = symm_mem.rendezvous(buf, group)
        torch.cuda.synchronize(device)
        dist.barrier(group=group)          # every rank's buffer is zero before anyone signals into it
        ptrs = [int(p) for p in handle.buffer_ptrs]
        return cls([buf], ptrs, dist.get_rank(group), dist.get_world_size(group), tcap, H, device, handle)

    @classmethod
    def emulated(cls, world: int, tcap: int, H: int, device) -> "PeerExchange":
        n = cls.nbytes(tcap, H) // 4
        bufs = [torch.zeros(n, dtype=torch.float32, device=device) for _ in range(world)]
        return cls(bufs, [b.data_ptr() for b in bufs], -1, world, tcap, H, device)


def peer_combine_residual_rmsnorm(x: torch.Tensor, y: torch.Tensor, k: int, ex: PeerExchange,
                                  eps: float | None = None) -> torch.Tensor:
    """rms_norm(x + sum over ranks and slots of y): x [T, H] (the same on every rank), y [T*k, H] this rank's
    expert outputs (zero rows for pairs owned elsewhere).  One launch; the ranks' partial sums cross NVLink
    as peer stores inside it.  With an emulated exchange x and y carry a leading rank dimension."""
    lib = _lib.load()
    dev = _lib.require_cuda(x, y)
    emul = ex.rank < 0
    T, H = x.shape[-2], x.shape[-1]
    x, y = x.contiguous(), y.contiguous()
    if eps is None:
        eps = torch.finfo(x.dtype).eps
    out = torch.empty_like(x)
    with torch.cuda.device(dev):
        _lib.check(lib.jq_ep_combine_residual_rmsnorm(
            x.data_ptr(), y.data_ptr(), k, T, H, float(eps), out.data_ptr(), _lib.dtype_id(x.dtype), ex._ptr_array,
            0 if emul else ex.rank, ex.world, ex.tcap, ex.counters.data_ptr(), ex.world if emul else 0,
            _lib.stream_ptr(dev)))
    return out
