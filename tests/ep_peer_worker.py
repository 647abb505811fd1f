"""Worker of tests/test_gpu_ep_peer.py: one process per GPU (torchrun).  Checks the peer-memory exchange fused
with residual + norm against an NCCL all-reduce of the same partial sums, eagerly and from a CUDA graph, and
the expert-parallel decode stack in "peer" mode against "replicated" mode."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from jangq_b200 import _lib, moe, moe_ep  # noqa: E402
from jangq_b200.stacks import MoEDecodeStack  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    T, k, H = 8, 8, 2048
    ex = moe_ep.PeerExchange.connect(None, 16, H, dev)
    g = torch.Generator(device=dev).manual_seed(5)              # x: the same on every rank
    gy = torch.Generator(device=dev).manual_seed(100 + rank)    # y: the rank's own
    eps = torch.finfo(torch.bfloat16).eps
    failures = []       # recorded, not raised: every rank runs the same sequence of collectives to the end

    def expect(cond, what):
        if not bool(cond):
            failures.append(what)

    def reference(x, y):
        part = y.float().reshape(T, k, H).sum(dim=1)
        dist.all_reduce(part)
        tot = x.float() + part
        return tot * torch.rsqrt((tot * tot).mean(dim=-1, keepdim=True) + eps)

    for rep in range(6):
        x = torch.randn((T, H), device=dev, generator=g).to(torch.bfloat16)
        y = (torch.randn((T * k, H), device=dev, generator=gy) * 0.3).to(torch.bfloat16)
        out = moe_ep.peer_combine_residual_rmsnorm(x, y, k, ex)
        ref = reference(x, y)
        expect((out.float() - ref).abs().max() <= 2.0 ** -7 * ref.abs().max(), f"eager exchange, rep {rep}")
        gathered = [torch.empty_like(out) for _ in range(world)]
        dist.all_gather(gathered, out)
        expect(all(torch.equal(gathered[0], o) for o in gathered), "ranks disagree bit-wise")
    # the same call replayed from a CUDA graph
    x = torch.randn((T, H), device=dev, generator=g).to(torch.bfloat16)
    y = (torch.randn((T * k, H), device=dev, generator=gy) * 0.3).to(torch.bfloat16)
    ref = reference(x, y)
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        moe_ep.peer_combine_residual_rmsnorm(x, y, k, ex)
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    gr = torch.cuda.CUDAGraph()
    with torch.cuda.graph(gr):
        out = moe_ep.peer_combine_residual_rmsnorm(x, y, k, ex)
    for _ in range(5):
        gr.replay()
    torch.cuda.synchronize()
    expect((out.float() - ref).abs().max() <= 2.0 ** -7 * ref.abs().max(), "graph replay")
    # the decode stack: peer mode against the NCCL mode, two layers
    xs = torch.randn((world, H), device=dev, generator=g).to(torch.bfloat16)
    outs = {}
    for mode in ("replicated", "peer"):
        st = MoEDecodeStack(layers=2, device=dev, rank=rank, world=world, ep_mode=mode)
        outs[mode] = st.step(xs).float()
    torch.cuda.synchronize()
    expect((outs["peer"] - outs["replicated"]).abs().max() <= 2.0 ** -5 * outs["replicated"].abs().max(),
           "decode stack: peer against replicated")
    expect(_lib.load().jq_device_status() == _lib.JQ_OK, "device status word set")
    # the ranks agree on pass or fail between steps, with nothing in flight, and all leave through the same door
    bad = torch.tensor([len(failures)], device=dev, dtype=torch.int32)
    dist.all_reduce(bad, op=dist.ReduceOp.MAX)
    if failures:
        print(f"EP_PEER_FAIL rank {rank}: {failures}", flush=True)
    if rank == 0 and int(bad.item()) == 0:
        print("EP_PEER_OK")
    dist.destroy_process_group()
    sys.exit(1 if int(bad.item()) else 0)


if __name__ == "__main__":
    main()
