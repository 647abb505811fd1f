"""Expert-parallel dispatch/combine logic on two CPU ranks (gloo).  The expert math is a dense
torch reference passed in as `local_fn`; what is under test is the exchange: split tables, the
ordering by destination, the return trip, the sum over slots, and the host-side validation."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from jangq_b200 import moe_ep


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _dense_moe(x, idx, w, Wg, Wu, Wd):
    out = torch.zeros(x.shape[0], Wd.shape[1], dtype=torch.float32)
    for t in range(x.shape[0]):
        for j in range(idx.shape[1]):
            e = int(idx[t, j])
            g, u = Wg[e] @ x[t].float(), Wu[e] @ x[t].float()
            out[t] += float(w[t, j]) * (Wd[e] @ (torch.nn.functional.silu(g) * u))
    return out


def _worker(rank, world, port, mode, ret):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        E, k, H, I = 8, 2, 16, 8
        g = torch.Generator().manual_seed(0)
        Wg, Wu, Wd = torch.randn(E, I, H, generator=g), torch.randn(E, I, H, generator=g), torch.randn(E, H, I, generator=g)
        e_local = E // world
        lo = rank * e_local

        def local_fn(x_rows, e_loc, w_rows):
            live = e_loc >= 0                                     # empty slots of the fixed-capacity exchange: id -1
            # empty slots hold whatever the buffer held: compute on zeros there, never multiply garbage by 0
            xr = torch.where(live[:, None], x_rows, torch.zeros(()))
            wr = torch.where(live, w_rows, torch.zeros(()))
            return _dense_moe(xr, (e_loc.long().clamp(min=0) + lo)[:, None], wr[:, None], Wg, Wu, Wd)

        if mode == "sharded":
            T = 5 + 3 * rank                                     # ragged: ranks hold different row counts
            gr = torch.Generator().manual_seed(100 + rank)
            x = torch.randn(T, H, generator=gr)
            idx = torch.randint(0, E, (T, k), generator=gr)
            if rank == 0:
                idx[:] = torch.tensor([6, 7])                    # rank 0 sends everything to rank 1's experts
            w = torch.rand(T, k, generator=gr)
            out = moe_ep.dispatch_combine(x, idx, w, E, local_fn)
            ref = _dense_moe(x, idx, w, Wg, Wu, Wd)
        elif mode in ("slots", "slots_overflow"):
            T = 6                                                # capacity is a contract: the same on every rank
            gr = torch.Generator().manual_seed(200 + rank)
            x = torch.randn(T, H, generator=gr)
            idx = torch.randint(0, E, (T, k), generator=gr)
            if rank == 0:
                idx[:] = torch.tensor([6, 7])                    # all 12 pairs of rank 0 go to rank 1
            else:
                idx[:] = torch.tensor([1, 5])                    # rank 1: six pairs each way
            w = torch.rand(T, k, generator=gr)
            cap = 12 if mode == "slots" else 8
            out, over = moe_ep.dispatch_combine_slots(x, idx, w, E, local_fn, cap)
            ref = _dense_moe(x, idx, w, Wg, Wu, Wd)
            if mode == "slots_overflow":
                # rank 0 loses its pairs past the 8th slot (sorted by destination, then pair order) and says so
                assert bool(over) == (rank == 0)
                if rank == 0:
                    keep = torch.zeros(T * k, dtype=torch.bool)
                    keep[:8] = True
                    ref = _dense_moe(x, idx, w * keep.reshape(T, k), Wg, Wu, Wd)
            else:
                assert not bool(over)
        elif mode == "empty":
            x = torch.zeros(0, H)
            idx = torch.zeros(0, k, dtype=torch.long)
            w = torch.zeros(0, k)
            out = moe_ep.dispatch_combine(x, idx, w, E, local_fn)
            ref = torch.zeros(0, H)
        elif mode == "gathered":
            gr = torch.Generator().manual_seed(50 + rank)        # every rank its own rows, fixed count
            x = torch.randn(2, H, generator=gr)
            idx = torch.randint(0, E, (2, k), generator=gr)
            w = torch.rand(2, k, generator=gr)

            def partial_fn(x_, idx_, w_):
                mine = (idx_ >= lo) & (idx_ < lo + e_local)
                return _dense_moe(x_, idx_, w_ * mine, Wg, Wu, Wd)
            out = moe_ep.gathered_tokens(x, idx, w, partial_fn)
            ref = _dense_moe(x, idx, w, Wg, Wu, Wd)
        else:
            gr = torch.Generator().manual_seed(7)                # same rows on every rank
            x = torch.randn(3, H, generator=gr)
            idx = torch.randint(0, E, (3, k), generator=gr)
            w = torch.rand(3, k, generator=gr)

            def partial_fn(x_, idx_, w_):
                mine = (idx_ >= lo) & (idx_ < lo + e_local)
                return _dense_moe(x_, idx_, w_ * mine, Wg, Wu, Wd)
            out = moe_ep.replicated_tokens(x, idx, w, partial_fn)
            ref = _dense_moe(x, idx, w, Wg, Wu, Wd)
        ret[rank] = bool(torch.allclose(out, ref, rtol=1e-5, atol=1e-5))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode", ("sharded", "replicated", "gathered", "empty", "slots", "slots_overflow"))
def test_expert_parallel_two_ranks(mode):
    world, port = 2, _free_port()
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(world, port, mode, ret), nprocs=world, join=True)
    assert dict(ret) == {0: True, 1: True}


def test_split_validation():
    with pytest.raises(ValueError, match="expected 10"):
        moe_ep.validate_splits(torch.tensor([3, 3]), torch.tensor([1, 2]), 10)
    with pytest.raises(ValueError, match="negative"):
        moe_ep.validate_splits(torch.tensor([11, -1]), torch.tensor([1, 2]), 10)


def test_slot_capacity_is_a_multiple_of_8_between_the_mean_share_and_all_pairs():
    for n_pairs, world in ((16384, 8), (16384, 2), (64, 8), (8, 4), (100000, 3)):
        c = moe_ep.slot_capacity(n_pairs, world)
        assert c % 8 == 0 or c == n_pairs
        assert c <= max(n_pairs, 8)
        assert c >= min(n_pairs, n_pairs // world)
    assert moe_ep.slot_capacity(16384, 8) == 2592          # 1.25 x 2048 + 32
    assert moe_ep.slot_capacity(16384, 8, factor=2.0) == 4128
