"""Expert parallelism for the routed-MoE path: experts sharded E/G per GPU, one process per GPU.

The reference has no multi-device code; this is the one place the path shards naturally (by
expert), with exactly one exchange each way:

  replicated tokens (batch-1 / small-batch decode: every rank holds the same rows):
      each rank runs its own experts on all rows (pairs of other ranks' experts are skipped by the
      kernels) and the partial sums are added over NVLink: by `peer_combine_residual_rmsnorm` (peer loads
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


def local_experts_fn(gate, up, down, swiglu_limit: float = 0.0):
    """local_fn for dispatch_combine on a GPU: rows with one (local) expert and weight each."""
    from .moe import moe_layer

    def fn(x_rows, e_local, w_rows):
        if x_rows.shape[0] == 0:
            return torch.zeros_like(x_rows, dtype=torch.float32)
        return moe_layer(x_rows, e_local[:, None], w_rows[:, None], gate, up, down, swiglu_limit=swiglu_limit,
                         out_f32=True)
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
    as peer loads inside it.  With an emulated exchange x and y carry a leading rank dimension."""
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
