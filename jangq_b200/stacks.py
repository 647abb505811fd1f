"""Synthetic random-init weight stacks with the shapes of the BASELINE configurations, for
benchmarks and smoke tests.  Only the quantized hot path is modelled: attention's softmax(QK)V,
norms, RoPE and sampling are outside it, so the attention block is its four projections with the
query projection's output standing in for the attention result.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import moe, moe_ep
from .linear import JANGLinear


def _rand_linear(out_f, in_f, bits, gs, device, seed):
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    w = (torch.randn((out_f, in_f), generator=g, device=device, dtype=torch.float32) * 0.02).to(torch.bfloat16)
    return JANGLinear.from_float(w, bits=bits, group_size=gs)


def _rand_bank(E, out_f, in_f, bits, gs, device, seed, e0=0, e1=None):
    """Experts [e0, e1) of a bank of E random experts.  The whole bank is drawn from one seed and then cut, so
    the experts a rank holds are the same tensors whatever the number of ranks."""
    from .ops import quantize
    e1 = E if e1 is None else e1
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    w = (torch.randn((E, out_f, in_f), generator=g, device=device, dtype=torch.float32)[e0:e1] * 0.02).to(torch.bfloat16)
    wq, s, b = quantize(w, gs, bits)
    return moe.ExpertBank(wq, s, b, bits, gs)


class MoEDecodeStack:
    """BASELINE config 3 (default arguments): 48 layers, hidden 2048, 32 query / 4 KV heads of 128,
    128 experts of SwiGLU intermediate 768, top-8 softmax routing, experts 2-bit, attention 6-bit,
    group 64.  With world > 1 the experts are sharded E/world per rank (expert parallelism); the
    attention projections and the router are replicated.  Decode modes for world > 1:
      "replicated" (default)  every rank carries the rows of ALL tokens of the step through the replicated
                   dense blocks (a decode mat-vec streams the same weights for 1 or 8 rows), runs its own
                   experts on them and one all-reduce per layer adds the partial sums;
      "peer"       as "replicated", but the partial sums cross NVLink as peer loads inside the kernel that also
                   does the residual and the norm (moe_ep.peer_combine_residual_rmsnorm): no library collective;
      "gathered"   every rank carries its own rows; all-gather before, reduce-scatter after the experts."""

    def __init__(self, layers=48, hidden=2048, q_heads=32, kv_heads=4, head_dim=128, experts=128, inter=768, topk=8,
                 expert_bits=2, attn_bits=6, gs=64, device="cuda", rank=0, world=1, seed=0, group=None,
                 ep_mode="replicated"):
        self.L, self.H, self.E, self.I, self.k = layers, hidden, experts, inter, topk
        self.slot_factor, self._overflow = 1.25, None
        self.world, self.rank, self.group = world, rank, group
        self.ep_mode = ep_mode
        self.e_local = experts // world
        self.exchange = None
        if world > 1 and ep_mode == "peer":
            self.exchange = moe_ep.PeerExchange.connect(group, 16, hidden, device)
        self.base = rank * self.e_local
        dq, dkv = q_heads * head_dim, kv_heads * head_dim
        self.layers = []
        for l in range(layers):
            s0 = seed + 1000 * l
            lay = {
                "q": _rand_linear(dq, hidden, attn_bits, gs, device, s0 + 1),
                "k": _rand_linear(dkv, hidden, attn_bits, gs, device, s0 + 2),
                "v": _rand_linear(dkv, hidden, attn_bits, gs, device, s0 + 3),
                "o": _rand_linear(hidden, dq, attn_bits, gs, device, s0 + 4),
                "router": (torch.randn((experts, hidden), device=device,
                                       generator=torch.Generator(device=device).manual_seed(s0 + 5)) * 0.02).to(torch.bfloat16),
                "gate": _rand_bank(experts, inter, hidden, expert_bits, gs, device, s0 + 10, self.base, self.base + self.e_local),
                "up": _rand_bank(experts, inter, hidden, expert_bits, gs, device, s0 + 30, self.base, self.base + self.e_local),
                "down": _rand_bank(experts, hidden, inter, expert_bits, gs, device, s0 + 50, self.base, self.base + self.e_local),
            }
            self.layers.append(lay)
        torch.cuda.synchronize(device)
        for lay in self.layers:
            for n in "qkvo":
                lay[n].freeze()
        e = 2
        attn = sum(moe_bytes(lin) for lin in (self.layers[0][n] for n in "qkvo"))
        per_expert = 3 * (inter * hidden * expert_bits // 8 + (inter * hidden // gs) * 2 * e)
        self.bytes_per_token = layers * (attn + topk * per_expert + experts * hidden * 2)

    def check_status(self):
        """Raise JangqError(JQ_ETIMEOUT) if a bounded device-side wait ran out since the last check (a rank of
        the exchange that never arrived): the outputs of that step are undefined.  Reads the device status
        word, which synchronises the device; call it between graph replays in a serving loop."""
        from . import _lib
        _lib.check(_lib.load().jq_device_status())

    def step(self, x: torch.Tensor, trace: list | None = None, n_layers: int | None = None) -> torch.Tensor:
        """One token per row of x ([T, H] bf16) through every layer's quantized matmuls.  With several ranks
        and outside stream capture, the step first checks that the previous one did not time out.  `trace`
        (a list) receives every layer's routing decision (idx, w), for checks against a reference walk;
        `n_layers` stops after the first layers."""
        from .ops import qgemv_fused, qgemv_fused_norm
        T = x.shape[0]
        if self.world > 1 and not torch.cuda.is_current_stream_capturing():
            self.check_status()
        pending = None      # (x, slot rows) of a layer whose combine + residual + norm rides in the next q/k/v launch
        for lay in self.layers[:n_layers]:
            if T <= 16:     # q/k/v read the same activations: one fused launch
                outs = [torch.empty((T, lay[n].out_features), dtype=x.dtype, device=x.device) for n in "qkv"]
                if pending is not None:
                    x = qgemv_fused_norm(pending[0], pending[1], self.k, [lay[n] for n in "qkv"], outs, 1)
                    pending = None
                else:
                    qgemv_fused(x, [lay[n] for n in "qkv"], outs, 1)
                q = outs[0]
            else:
                q = lay["q"](x)
                lay["k"](x)
                lay["v"](x)
            if T <= 16 and self.H <= 4096:       # residual + norm folded into the router launch
                x, idx, w = moe.route_norm_from_hidden(x, lay["o"](q), lay["router"], self.k)
            else:
                x = moe.residual_rmsnorm(x, lay["o"](q))
                idx, w = moe.route_from_hidden(x, lay["router"], self.k)
            if trace is not None:
                trace.append((idx, w))
            if self.world == 1 and T * self.k < moe.SORT_THRESHOLD:
                y = moe.moe_layer(x, idx, w, lay["gate"], lay["up"], lay["down"], all_local=True, return_slots=True,
                                  static_weights=True)
                if T == 1 and self.H <= 4096:
                    pending = (x, y)
                else:
                    x = moe.residual_rmsnorm(x, y, k=self.k)     # combine + residual + norm in one launch
                continue
            if self.world == 1:
                y = moe.moe_layer(x, idx, w, lay["gate"], lay["up"], lay["down"], out_f32=True, all_local=True)
            elif self.ep_mode == "peer" and T <= self.exchange.tcap:
                y = moe.moe_layer(x, idx, w, lay["gate"], lay["up"], lay["down"], expert_base=self.base,
                                  return_slots=True, static_weights=True, few_token_path=True, few_local=True)
                x = moe_ep.peer_combine_residual_rmsnorm(x, y, self.k, self.exchange)
                continue
            elif self.ep_mode in ("replicated", "peer"):
                y = moe.moe_layer(x, idx, w, lay["gate"], lay["up"], lay["down"], expert_base=self.base, out_f32=True,
                                  static_weights=True, few_token_path=T <= 16, few_local=True)
                dist.all_reduce(y, op=dist.ReduceOp.SUM, group=self.group)
            else:
                y = moe_ep.gathered_tokens(x, idx, w, moe_ep.partial_experts_fn(lay["gate"], lay["up"], lay["down"],
                                                                                self.base), group=self.group)
            x = moe.residual_rmsnorm(x, y)
        if pending is not None:
            x = moe.residual_rmsnorm(pending[0], pending[1], k=self.k)
        return x


    def prefill_layer(self, x: torch.Tensor, layer: int = 0) -> torch.Tensor:
        """The routed-expert block of one layer over many tokens (sorted tensor-core path); with
        world > 1 the tokens of this rank are dispatched to the expert owners and combined back."""
        lay = self.layers[layer]
        logits = torch.matmul(x, lay["router"].t())          # library GEMM; the selection is jq_moe_topk (one launch)
        idx, w = moe.route_softmax_topk(logits, self.k)
        if self.world == 1:
            return moe.moe_layer(x, idx, w, lay["gate"], lay["up"], lay["down"])
        # fixed-capacity slots: two equal-split collectives, nothing read back by the host inside the layer; the
        # overflow flags of a step are OR-ed on the device and read by prefill_overflowed() after it
        cap = moe_ep.slot_capacity(x.shape[0] * self.k, self.world, self.slot_factor)
        y, over = moe_ep.dispatch_combine_slots(x, idx, w, self.E,
                                                moe_ep.local_experts_fn(lay["gate"], lay["up"], lay["down"], out_f32=False),
                                                cap, group=self.group)
        self._overflow = over if self._overflow is None else (self._overflow | over)
        return y.to(x.dtype)

    def prefill_layer_exact(self, x: torch.Tensor, layer: int = 0) -> torch.Tensor:
        """prefill_layer with exact split sizes (a host read-back per layer): the route to repeat a step on whose
        slots overflowed."""
        lay = self.layers[layer]
        logits = torch.matmul(x, lay["router"].t())          # library GEMM; the selection is jq_moe_topk (one launch)
        idx, w = moe.route_softmax_topk(logits, self.k)
        if self.world == 1:
            return moe.moe_layer(x, idx, w, lay["gate"], lay["up"], lay["down"])
        y = moe_ep.dispatch_combine(x, idx, w, self.E, moe_ep.local_experts_fn(lay["gate"], lay["up"], lay["down"]),
                                    group=self.group)
        return y.to(x.dtype)

    def prefill_overflowed(self) -> bool:
        """True when a prefill_layer call since the last check ran out of slots on any rank (one host read; the
        ranks agree through one all-reduce, so that they repeat the step together)."""
        if self._overflow is None:
            return False
        flag = self._overflow.to(torch.int32).reshape(1)
        self._overflow = None
        if self.world > 1:
            dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=self.group)
        return bool(flag.item())


def moe_bytes(lin: JANGLinear) -> int:
    n, k = lin.out_features, lin.in_features
    return n * k * lin.bits // 8 + n * (k // lin.group_size) * 2 * lin.scales.element_size()
