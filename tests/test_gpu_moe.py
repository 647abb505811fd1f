"""GPU parity of the routed-MoE path (sort, gather, grouped GEMM, SwiGLU, combine, gather
mat-vec) against the CPU oracle.  Index outputs are bit-exact; floating-point outputs are held to
max |y-ref| / max|ref| <= 1e-2 and cosine >= 0.9999 (BASELINE north star)."""
import numpy as np
import pytest
import torch

import jangq_b200 as jq
from jangq_b200 import _lib
from jangq_b200.moe import SORT_THRESHOLD, SortedPairs
from oracle import jang_oracle as jo

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def close(y, ref):
    y = np.asarray(y, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    assert np.abs(y - ref).max() / np.abs(ref).max() <= 1e-2
    assert float((y * ref).sum() / (np.linalg.norm(y) * np.linalg.norm(ref))) >= 0.9999


def make_bank(E, N, K, bits, gs, seed, dtype=torch.bfloat16):
    rng = np.random.default_rng(seed)
    w = torch.from_numpy((rng.standard_normal((E, N, K)) * 0.05).astype(np.float32)).to(DEV).to(dtype)
    wq, s, b = jq.quantize(w, gs, bits)
    return jq.ExpertBank(wq, s, b, bits, gs), (wq.cpu().numpy().view(np.uint32), s.float().cpu().numpy(),
                                               b.float().cpu().numpy(), bits, gs)


@pytest.mark.parametrize("n,E,base", ((0, 4, 0), (1, 4, 0), (37, 8, 0), (4096, 128, 0), (16384, 128, 0), (40960, 512, 0),
                                      (5000, 16, 16), (3000, 64, 128)))
def test_sort_matches_stable_argsort(n, E, base):
    rng = np.random.default_rng(n + E)
    total = E if base == 0 else 4 * E + base
    idx = rng.integers(0, total, n).astype(np.int32)
    sp = SortedPairs(torch.from_numpy(idx).to(DEV), E, base)
    torch.cuda.synchronize()
    local = idx - base
    keep = (local >= 0) & (local < E)
    order_ref = np.argsort(np.where(keep, local, E), kind="stable").astype(np.int32)[: keep.sum()]
    off_ref = np.concatenate([[0], np.cumsum(np.bincount(local[keep], minlength=E))]).astype(np.int32)
    kept = int(sp.offsets[E])
    assert kept == keep.sum()
    assert np.array_equal(sp.offsets.cpu().numpy(), off_ref)
    assert np.array_equal(sp.order.cpu().numpy()[:kept], order_ref)
    inv = sp.inv.cpu().numpy()[:n]
    inv_ref = np.full(n, -1, np.int32)
    inv_ref[order_ref] = np.arange(kept, dtype=np.int32)
    assert np.array_equal(inv, inv_ref)
    # tile list: every expert's rows are covered by ceil(count / 128) tiles in order
    nt = int(sp.num_tiles)
    te, tr = sp.tile_expert.cpu().numpy()[:nt], sp.tile_row0.cpu().numpy()[:nt]
    exp_te, exp_tr = [], []
    for e in range(E):
        for r in range(off_ref[e], off_ref[e + 1], 128):
            exp_te.append(e), exp_tr.append(r)
    assert nt == len(exp_te) <= sp.max_tiles
    assert np.array_equal(te, np.array(exp_te, np.int32)) and np.array_equal(tr, np.array(exp_tr, np.int32))


@pytest.mark.parametrize("R", (8, 63, 64, 300))
@pytest.mark.parametrize("bits", (2, 4, 6))
def test_gather_qmm_both_paths(bits, R):
    """Below and above the sort threshold (the reference's ops_selftest sweeps T across it)."""
    E, N, K = 8, 96, 256
    bank, (pk, s, b, _, gs) = make_bank(E, N, K, bits, 64, seed=bits)
    rng = np.random.default_rng(R)
    x = torch.from_numpy(rng.standard_normal((R, K)).astype(np.float32)).to(DEV).to(torch.bfloat16)
    rhs = torch.from_numpy(rng.integers(0, E, R).astype(np.int32)).to(DEV)
    y = jq.gather_qmm(x, bank, rhs_indices=rhs)
    ref = jo.gather_qmm(x.float().cpu().numpy(), pk, s, b, rhs.cpu().numpy(), bits, gs)
    assert (R >= SORT_THRESHOLD) == (R >= 64)
    close(y.float().cpu().numpy(), ref)
    # the MLX call shape: stacked tensors + lhs_indices
    lhs = torch.from_numpy(rng.integers(0, R, R).astype(np.int32)).to(DEV)
    y2 = jq.gather_qmm(x, bank.weight, bank.scales, bank.biases, rhs_indices=rhs, lhs_indices=lhs, group_size=64,
                       bits=bits)
    ref2 = jo.gather_qmm(x.float().cpu().numpy(), pk, s, b, rhs.cpu().numpy(), bits, gs, lhs.cpu().numpy())
    close(y2.float().cpu().numpy(), ref2)


def test_gather_qmm_sorted_flag_needs_lhs():
    bank, _ = make_bank(2, 16, 64, 4, 64, seed=0)
    x = torch.zeros((4, 64), dtype=torch.bfloat16, device=DEV)
    with pytest.raises(ValueError):
        jq.gather_qmm(x, bank, rhs_indices=torch.zeros(4, dtype=torch.int32, device=DEV), sorted_indices=True)


@pytest.mark.parametrize("T", (1, 7, 8, 64, 300))
def test_moe_layer_vs_oracle(T):
    """E=16 experts, top-4, H=256, I=128: decode path (T*k < 64) and sorted tensor-core path."""
    E, k, H, I = 16, 4, 256, 128
    gate, qg = make_bank(E, I, H, 2, 64, seed=1)
    up, qu = make_bank(E, I, H, 2, 64, seed=2)
    down, qd = make_bank(E, H, I, 3, 64, seed=3)
    rng = np.random.default_rng(T)
    x = torch.from_numpy(rng.standard_normal((T, H)).astype(np.float32)).to(DEV).to(torch.bfloat16)
    logits = torch.from_numpy(rng.standard_normal((T, E)).astype(np.float32)).to(DEV)
    idx, w = jq.route_softmax_topk(logits, k)
    idx_ref, w_ref = jo.route_softmax_topk(logits.cpu().numpy(), k)
    assert np.array_equal(idx.cpu().numpy(), idx_ref)
    assert np.allclose(w.cpu().numpy(), w_ref, rtol=1e-5, atol=1e-7)
    out = jq.moe_layer(x, idx, w, gate, up, down)
    ref = jo.moe_layer(x.float().cpu().numpy(), idx_ref, w.cpu().numpy(), qg, qu, qd, act_dtype="bf16")
    close(out.float().cpu().numpy(), ref)
    # clamp variant (dsv41 swiglu_limit)
    out2 = jq.moe_layer(x, idx, w, gate, up, down, swiglu_limit=0.5)
    ref2 = jo.moe_layer(x.float().cpu().numpy(), idx_ref, w.cpu().numpy(), qg, qu, qd, swiglu_limit=0.5, act_dtype="bf16")
    close(out2.float().cpu().numpy(), ref2)


def test_moe_layer_zero_token_experts_and_skew():
    """All tokens routed to two experts: the other experts get no tile; one expert gets several."""
    E, k, H, I, T = 8, 2, 128, 64, 400
    gate, qg = make_bank(E, I, H, 4, 64, seed=11)
    up, qu = make_bank(E, I, H, 4, 64, seed=12)
    down, qd = make_bank(E, H, I, 4, 64, seed=13)
    rng = np.random.default_rng(0)
    x = torch.from_numpy(rng.standard_normal((T, H)).astype(np.float32)).to(DEV).to(torch.bfloat16)
    idx = torch.tensor([[5, 2]] * T, dtype=torch.int32, device=DEV)
    w = torch.from_numpy(rng.random((T, k)).astype(np.float32)).to(DEV)
    out = jq.moe_layer(x, idx, w, gate, up, down)
    ref = jo.moe_layer(x.float().cpu().numpy(), idx.cpu().numpy(), w.cpu().numpy(), qg, qu, qd, act_dtype="bf16")
    close(out.float().cpu().numpy(), ref)


def test_moe_mixed_bit_widths_per_expert():
    """Each expert with its own width (2/3/4/6/8): one launch per distinct width."""
    E, k, H, I, T = 5, 2, 128, 64, 96
    widths = (2, 3, 4, 6, 8)
    rng = np.random.default_rng(9)

    def mixed(N, K, seed):
        experts, ref = [], []
        for e in range(E):
            w = torch.from_numpy((np.random.default_rng(seed + e).standard_normal((N, K)) * 0.05).astype(np.float32))
            wq, s, b = jq.quantize(w.to(DEV).to(torch.bfloat16), 64, widths[e])
            experts.append((wq, s, b, widths[e]))
            ref.append(jo.dequantize_affine(wq.cpu().numpy().view(np.uint32), s.float().cpu().numpy(),
                                            b.float().cpu().numpy(), widths[e], 64))
        return jq.ExpertBank.from_experts(experts), np.stack(ref)

    gate, Wg = mixed(I, H, 100)
    up, Wu = mixed(I, H, 200)
    down, Wd = mixed(H, I, 300)
    x = torch.from_numpy(rng.standard_normal((T, H)).astype(np.float32)).to(DEV).to(torch.bfloat16)
    idx = torch.from_numpy(rng.integers(0, E, (T, k)).astype(np.int32)).to(DEV)
    w = torch.from_numpy(rng.random((T, k)).astype(np.float32)).to(DEV)
    for sl in (slice(0, T), slice(0, 5)):          # sorted path and decode path
        out = jq.moe_layer(x[sl], idx[sl], w[sl], gate, up, down).float().cpu().numpy()
        xn, idn, wn = x[sl].float().cpu().numpy(), idx[sl].cpu().numpy(), w[sl].cpu().numpy()
        ref = np.zeros_like(out)
        for t in range(xn.shape[0]):
            for j in range(k):
                e = int(idn[t, j])
                g = jo.round_to(xn[t] @ Wg[e].T, "bf16")
                u = jo.round_to(xn[t] @ Wu[e].T, "bf16")
                h = jo.round_to((g / (1 + np.exp(-g))) * u * wn[t, j], "bf16")
                ref[t] += jo.round_to(h @ Wd[e].T, "bf16")
        close(out, ref)


def test_moe_expert_parallel_shards_sum_to_full():
    """Experts split over 4 'ranks' (expert_base): the partial outputs add up to the full layer."""
    E, k, H, I = 16, 4, 128, 64
    gate, _ = make_bank(E, I, H, 2, 64, seed=21)
    up, _ = make_bank(E, I, H, 2, 64, seed=22)
    down, _ = make_bank(E, H, I, 2, 64, seed=23)
    rng = np.random.default_rng(3)
    for T in (3, 200):
        x = torch.from_numpy(rng.standard_normal((T, H)).astype(np.float32)).to(DEV).to(torch.bfloat16)
        idx, w = jq.route_softmax_topk(torch.from_numpy(rng.standard_normal((T, E)).astype(np.float32)).to(DEV), k)
        full = jq.moe_layer(x, idx, w, gate, up, down, out_f32=True)
        parts = sum(jq.moe_layer(x, idx, w, gate.slice(e0, e0 + 4), up.slice(e0, e0 + 4), down.slice(e0, e0 + 4),
                                 expert_base=e0, out_f32=True) for e0 in range(0, E, 4))
        assert float((full - parts).abs().max()) <= 1e-5 * float(full.abs().max()) + 1e-6


@pytest.mark.parametrize("T,E,k,H", ((1, 128, 8, 2048), (3, 16, 4, 256), (5, 1000, 32, 512), (2, 40, 40, 128)))
def test_route_from_hidden_matches_unfused_router(T, E, k, H):
    """The one-launch router against x @ W^T (activation-type logits) -> oracle softmax-top-k: same experts
    (up to swaps between scores closer than the accumulation error of the logits), same weights."""
    from jangq_b200.moe import route_from_hidden
    rng = np.random.default_rng(T + E)
    x = torch.from_numpy(rng.standard_normal((T, H)).astype(np.float32)).to(DEV).to(torch.bfloat16)
    wr = torch.from_numpy((rng.standard_normal((E, H)) * 0.05).astype(np.float32)).to(DEV).to(torch.bfloat16)
    idx, w = route_from_hidden(x, wr, k)
    logits = (x.float() @ wr.float().t()).to(torch.bfloat16).float().cpu().numpy()
    idx_ref, w_ref = jo.route_softmax_topk(logits, k)
    idx, w = idx.cpu().numpy(), w.cpu().numpy()
    assert idx.shape == (T, k) and w.shape == (T, k)
    for t in range(T):
        assert len(set(idx[t].tolist())) == k and idx[t].min() >= 0 and idx[t].max() < E
        # same set of experts unless the k-th and (k+1)-th logits are within one rounding step of each other
        srt = np.sort(logits[t])[::-1]
        gap = srt[k - 1] - srt[k] if k < E else 1.0
        if gap > 2.0 ** -7 * max(1.0, abs(srt[k - 1])):
            assert set(idx[t].tolist()) == set(idx_ref[t].tolist())
            order = {e: i for i, e in enumerate(idx_ref[t].tolist())}
            wr_sorted = np.array([w_ref[t][order[e]] for e in idx[t].tolist()])
            assert np.allclose(w[t], wr_sorted, rtol=2e-2, atol=1e-6)
        assert abs(w[t].sum() - 1.0) < 1e-4
        assert np.all(np.diff(w[t]) <= 1e-7)          # scores come out in descending order


def test_residual_rmsnorm_matches_torch():
    from jangq_b200.moe import residual_rmsnorm
    torch.manual_seed(0)
    x = torch.randn(5, 2048, device=DEV).to(torch.bfloat16)
    for y in (torch.randn(5, 2048, device=DEV), torch.randn(5, 2048, device=DEV).to(torch.bfloat16)):
        out = residual_rmsnorm(x, y)
        v = x.float() + y.float()
        ref = v * torch.rsqrt((v * v).mean(-1, keepdim=True) + torch.finfo(torch.bfloat16).eps)
        assert out.dtype == torch.bfloat16
        assert (out.float() - ref).abs().max() <= 2.0 ** -7 * ref.abs().max()
    # k slot rows per token (the unweighted combine of the routed experts), H not a multiple of 1024
    xs = torch.randn(3, 1536, device=DEV).to(torch.bfloat16)
    ys = torch.randn(3 * 8, 1536, device=DEV).to(torch.bfloat16)
    out = residual_rmsnorm(xs, ys, k=8)
    v = xs.float() + ys.float().view(3, 8, 1536).sum(1)
    ref = v * torch.rsqrt((v * v).mean(-1, keepdim=True) + torch.finfo(torch.bfloat16).eps)
    assert (out.float() - ref).abs().max() <= 2.0 ** -7 * ref.abs().max()


@pytest.mark.parametrize("bits", (2, 6))
def test_gather_pair_equals_two_single_gathers(bits):
    """gate and up in one launch (jq_gather_qgemv2) are bit-identical to two launches."""
    from jangq_b200.moe import _gather_qgemv, _gather_qgemv_pair
    E, I, H, P = 8, 192, 512, 6
    gate, _ = make_bank(E, I, H, bits, 64, seed=21)
    up, _ = make_bank(E, I, H, bits, 64, seed=22)
    rng = np.random.default_rng(1)
    x = torch.from_numpy(rng.standard_normal((3, H)).astype(np.float32)).to(DEV).to(torch.bfloat16)
    pe = torch.tensor([0, 7, 3, 3, 9, 1], dtype=torch.int32, device=DEV)     # 9: not in the bank, skipped
    g2, u2 = _gather_qgemv_pair(x, 2, pe, gate, up)
    g1, u1 = _gather_qgemv(x, 2, pe, gate), _gather_qgemv(x, 2, pe, up)
    assert torch.equal(g1, g2) and torch.equal(u1, u2)
    assert torch.count_nonzero(g2[4]) == 0 and torch.count_nonzero(u2[4]) == 0
    assert P == pe.numel()


def test_decode_stack_step_is_finite_and_deterministic():
    from jangq_b200.stacks import MoEDecodeStack
    st = MoEDecodeStack(layers=2, hidden=512, q_heads=4, kv_heads=2, head_dim=128, experts=16, inter=256, topk=4,
                        device=DEV)
    x = torch.randn(1, 512, device=DEV, generator=torch.Generator(device=DEV).manual_seed(0)).to(torch.bfloat16)
    a, b = st.step(x), st.step(x)
    assert torch.isfinite(a.float()).all() and torch.equal(a, b)
    _lib.check(_lib.load().jq_device_status())


def test_device_status_clean_after_moe():
    torch.cuda.synchronize()
    assert _lib.load().jq_device_status() == 0


# ---- expert-parallel exchange fused with residual + norm, every rank emulated in one cooperative launch --------
@pytest.mark.parametrize("world,T,k,H", ((1, 3, 8, 2048), (2, 8, 8, 2048), (4, 4, 2, 1024), (8, 8, 8, 2048)))
def test_peer_combine_residual_rmsnorm_emulated(world, T, k, H):
    """out[r] = rms_norm(x + sum over ranks and slots of y[r]) for every rank r, repeated launches (sequence
    numbers and the double buffer advance), against torch in f32.  All ranks must produce the same bits."""
    from jangq_b200 import moe_ep
    ex = moe_ep.PeerExchange.emulated(world, 8, H, DEV)
    g = torch.Generator(device=DEV).manual_seed(world * 100 + T)
    for rep in range(5):
        x1 = torch.randn((T, H), device=DEV, generator=g).to(torch.bfloat16)
        x = x1.unsqueeze(0).repeat(world, 1, 1).contiguous()
        y = (torch.randn((world, T * k, H), device=DEV, generator=g) * 0.3).to(torch.bfloat16)
        out = moe_ep.peer_combine_residual_rmsnorm(x, y, k, ex)
        torch.cuda.synchronize()
        tot = x1.float() + y.float().reshape(world, T, k, H).sum(dim=2).sum(dim=0)
        ref = tot * torch.rsqrt((tot * tot).mean(dim=-1, keepdim=True) + torch.finfo(torch.bfloat16).eps)
        for r in range(world):
            assert torch.equal(out[r], out[0])
        assert (out[0].float() - ref).abs().max() <= 2.0 ** -7 * ref.abs().max()
    _lib.check(_lib.load().jq_device_status())


def test_peer_exchange_missing_rank_times_out(monkeypatch):
    """Failure detection without a fault: rank 0 of a world of 2 runs alone, nobody sets rank 1's flags, the
    bounded wait runs out (20 ms here), the kernel returns, the status word reports it and can be cleared."""
    from jangq_b200 import moe_ep
    monkeypatch.setenv("JANGQ_EP_WAIT_MS", "20")
    lib = _lib.load()
    T, k, H = 2, 2, 1024
    ex = moe_ep.PeerExchange.emulated(2, 8, H, DEV)
    ex.rank = 0                                            # a real rank 0 whose peer never shows up
    x = torch.randn((T, H), device=DEV).to(torch.bfloat16)
    y = torch.randn((T * k, H), device=DEV).to(torch.bfloat16)
    out = moe_ep.peer_combine_residual_rmsnorm(x, y, k, ex)
    torch.cuda.synchronize()
    assert out.shape == x.shape
    with pytest.raises(jq.JangqError) as err:
        _lib.check(lib.jq_device_status())
    assert err.value.status == _lib.JQ_ETIMEOUT
    _lib.check(lib.jq_device_status_clear())
    _lib.check(lib.jq_device_status())
    # the context is still usable
    ex1 = moe_ep.PeerExchange.emulated(1, 8, H, DEV)
    moe_ep.peer_combine_residual_rmsnorm(x.unsqueeze(0), y.unsqueeze(0), k, ex1)
    torch.cuda.synchronize()
    _lib.check(lib.jq_device_status())


@pytest.mark.parametrize("T,H,E,k", ((1, 2048, 128, 8), (8, 2048, 128, 8), (3, 4096, 64, 6), (5, 1024, 512, 10)))
def test_route_with_folded_residual_norm(T, H, E, k):
    """route_norm_from_hidden = residual_rmsnorm then route_from_hidden: the normalised rows agree to one
    rounding of the activation type and, fed the fused kernel's own rows, the unfused router returns the
    same experts and weights."""
    from jangq_b200 import moe
    g = torch.Generator(device=DEV).manual_seed(T * 31 + H)
    x = torch.randn((T, H), device=DEV, generator=g).to(torch.bfloat16)
    res = torch.randn((T, H), device=DEV, generator=g).to(torch.bfloat16)
    wr = (torch.randn((E, H), device=DEV, generator=g) * 0.05).to(torch.bfloat16)
    xo, idx, w = moe.route_norm_from_hidden(x, res, wr, k)
    ref = moe.residual_rmsnorm(x, res)
    assert (xo.float() - ref.float()).abs().max() <= 2.0 ** -7 * ref.float().abs().max()
    idx2, w2 = moe.route_from_hidden(xo, wr, k)
    torch.cuda.synchronize()
    assert torch.equal(idx, idx2) and torch.equal(w, w2)


# ---- the BASELINE MoE configurations at their real layer shapes ------------------------------------------------
def _bank_from_seed(E, N, K, bits, gs, seed):
    """A bank of E random experts quantized on the GPU, and its packed tensors on the host for the oracle."""
    g = torch.Generator(device=DEV).manual_seed(seed)
    w = (torch.randn((E, N, K), generator=g, device=DEV, dtype=torch.float32) * 0.02).to(torch.bfloat16)
    wq, s, b = jq.quantize(w, gs, bits)
    del w
    return jq.ExpertBank(wq, s, b, bits, gs), (wq.cpu().numpy().view(np.uint32), s.float().cpu().numpy(),
                                               b.float().cpu().numpy(), bits, gs)


def _linear_from_seed(N, K, bits, gs, seed):
    g = torch.Generator(device=DEV).manual_seed(seed)
    w = (torch.randn((N, K), generator=g, device=DEV, dtype=torch.float32) * 0.02).to(torch.bfloat16)
    lin = jq.JANGLinear.from_float(w, bits=bits, group_size=gs)
    return lin, (lin.weight.cpu().numpy().view(np.uint32), lin.scales.float().cpu().numpy(),
                 lin.biases.float().cpu().numpy(), bits, gs)


@pytest.mark.parametrize("name,E,k,H,I,shared_bits,Ts", (("config3", 128, 8, 2048, 768, 0, (1, 8, 2048)),
                                                         ("config5", 512, 10, 4096, 1024, 8, (1, 32, 4096))))
def test_moe_layer_at_baseline_shapes(name, E, k, H, I, shared_bits, Ts):
    """One routed layer of BASELINE config 3 (128 experts, top-8, hidden 2048, intermediate 768, 2-bit) and of
    config 5 (512 experts, top-10, hidden 4096, intermediate 1024, 2-bit experts plus one 8-bit shared expert)
    through moe_layer -- the few-token gather path at batch 1 / 8 / 32 and the sorted tensor-core path at the
    prefill sizes -- against the oracle.  Tokens are independent, so the oracle walks a sample of them
    (all of them for the small batches); every GPU row outside the sample is still checked for finiteness."""
    gate, qg = _bank_from_seed(E, I, H, 2, 64, 101)
    up, qu = _bank_from_seed(E, I, H, 2, 64, 102)
    down, qd = _bank_from_seed(E, H, I, 2, 64, 103)
    shared = shared_q = None
    if shared_bits:
        mods = [_linear_from_seed(I, H, shared_bits, 64, 104), _linear_from_seed(I, H, shared_bits, 64, 105),
                _linear_from_seed(H, I, shared_bits, 64, 106)]
        shared, shared_q = tuple(m for m, _ in mods), tuple(q for _, q in mods)
    for T in Ts:
        g = torch.Generator(device=DEV).manual_seed(T)
        x = torch.randn((T, H), generator=g, device=DEV).to(torch.bfloat16)
        logits = torch.randn((T, E), generator=g, device=DEV)
        idx, w = jq.route_softmax_topk(logits, k)
        out = jq.moe_layer(x, idx, w, gate, up, down, shared=shared)
        torch.cuda.synchronize()
        assert out.shape == (T, H) and bool(torch.isfinite(out.float()).all())
        sample = np.arange(T) if T <= 32 else np.random.default_rng(T).choice(T, 24, replace=False)
        ref = jo.moe_layer(x.float().cpu().numpy()[sample], idx.cpu().numpy()[sample], w.cpu().numpy()[sample],
                           qg, qu, qd, act_dtype="bf16", shared=shared_q)
        close(out.float().cpu().numpy()[sample], ref)
    _lib.check(_lib.load().jq_device_status())


def test_moe_layer_shared_expert_small():
    """The always-on expert through the CUDA path (fused gate/up mat-vec, SwiGLU kernel, down, added in f32
    inside the combine) with and without the clamp, few tokens and many, against the oracle's `shared=`."""
    E, k, H, I = 8, 2, 256, 128
    gate, qg = make_bank(E, I, H, 4, 64, seed=31)
    up, qu = make_bank(E, I, H, 4, 64, seed=32)
    down, qd = make_bank(E, H, I, 4, 64, seed=33)
    mods = [_linear_from_seed(I, H, 8, 64, 34), _linear_from_seed(I, H, 8, 64, 35), _linear_from_seed(H, I, 8, 64, 36)]
    shared, shared_q = tuple(m for m, _ in mods), tuple(q for _, q in mods)
    rng = np.random.default_rng(5)
    for T in (1, 5, 200):
        x = torch.from_numpy(rng.standard_normal((T, H)).astype(np.float32)).to(DEV).to(torch.bfloat16)
        idx, w = jq.route_softmax_topk(torch.from_numpy(rng.standard_normal((T, E)).astype(np.float32)).to(DEV), k)
        for lim in (0.0, 0.4):
            out = jq.moe_layer(x, idx, w, gate, up, down, swiglu_limit=lim, shared=shared)
            ref = jo.moe_layer(x.float().cpu().numpy(), idx.cpu().numpy(), w.cpu().numpy(), qg, qu, qd,
                               swiglu_limit=lim, act_dtype="bf16", shared=shared_q)
            close(out.float().cpu().numpy(), ref)


def _rms(v):
    v = v.astype(np.float64)
    return (v / np.sqrt((v * v).mean(axis=-1, keepdims=True) + float(torch.finfo(torch.bfloat16).eps))).astype(np.float32)


@pytest.mark.parametrize("T", (1, 4))
def test_decode_stack_two_layers_against_numpy_walk(T):
    """MoEDecodeStack (what bench.py times for MoE decode) at config-3 layer shapes, two layers, against a
    numpy walk of the same layers through the oracle: fused q/k/v, o, residual + norm folded into the router,
    top-8 of 128 experts through the gate/up gather, SwiGLU, down gather, combine + residual + norm.  The walk
    recomputes the router logits itself and accepts the GPU's choice of experts only where it agrees with them
    (or where the k-th and (k+1)-th logits are within one rounding step of the activation type)."""
    from jangq_b200.stacks import MoEDecodeStack
    st = MoEDecodeStack(layers=2, device=DEV)
    g = torch.Generator(device=DEV).manual_seed(100 + T)
    x0 = torch.randn((T, st.H), generator=g, device=DEV).to(torch.bfloat16)
    trace = []
    out = st.step(x0, trace=trace)
    torch.cuda.synchronize()

    def host(lin):
        return (lin.weight.cpu().numpy().view(np.uint32), lin.scales.float().cpu().numpy(),
                lin.biases.float().cpu().numpy(), lin.bits, lin.group_size)

    def bank(b):
        return (b.weight.cpu().numpy().view(np.uint32), b.scales.float().cpu().numpy(), b.biases.float().cpu().numpy(),
                b.expert_bits[0], b.group_size)

    x = x0.float().cpu().numpy()
    for lay, (idx_g, _) in zip(st.layers, trace):
        q = jo.round_to(jo.qmatmul(x, *host(lay["q"])), "bf16")
        o = jo.round_to(jo.qmatmul(q, *host(lay["o"])), "bf16")
        x = jo.round_to(_rms(x + o), "bf16")
        logits = jo.round_to((x.astype(np.float64) @ lay["router"].float().cpu().numpy().astype(np.float64).T)
                             .astype(np.float32), "bf16")
        idx_ref, _ = jo.route_softmax_topk(logits, st.k)
        idx_g = idx_g.cpu().numpy()
        for t in range(T):
            srt = np.sort(logits[t])[::-1]
            if srt[st.k - 1] - srt[st.k] > 2.0 ** -7 * max(1.0, abs(srt[st.k - 1])):
                assert set(idx_g[t].tolist()) == set(idx_ref[t].tolist())
        # routing weights of the experts the GPU chose, from the walk's own logits
        z = logits - logits.max(axis=-1, keepdims=True)
        p = np.exp(z) / np.exp(z).sum(axis=-1, keepdims=True)
        w = np.take_along_axis(p, idx_g.astype(np.int64), axis=-1)
        w = (w / (w.sum(axis=-1, keepdims=True) + 1e-20)).astype(np.float32)
        y = jo.moe_layer(x, idx_g, w, bank(lay["gate"]), bank(lay["up"]), bank(lay["down"]), act_dtype="bf16")
        x = jo.round_to(_rms(x + y), "bf16")
    close(out.float().cpu().numpy(), x)
    _lib.check(_lib.load().jq_device_status())


def test_switch_linear_module_matches_gather_qmm():
    """JANGSwitchLinear with SwitchProj's call shapes (jang_tools/dsv41/model.py:1207-1230): x [T,1,1,D] with
    idx [T,k] below the sort threshold, x [R,1,D] with a sorted idx [R] above it."""
    E, N, K, bits = 8, 96, 256, 4
    rng = np.random.default_rng(12)
    w = torch.from_numpy((rng.standard_normal((E, N, K)) * 0.05).astype(np.float32)).to(DEV).to(torch.bfloat16)
    mod = jq.JANGSwitchLinear.from_float(w, bits=bits, group_size=64)
    pk = (mod.weight.cpu().numpy().view(np.uint32), mod.scales.float().cpu().numpy(), mod.biases.float().cpu().numpy())
    T, k = 5, 3
    x = torch.from_numpy(rng.standard_normal((T, K)).astype(np.float32)).to(DEV).to(torch.bfloat16)
    idx = torch.from_numpy(rng.integers(0, E, (T, k)).astype(np.int32)).to(DEV)
    y = mod(x[:, None, None, :], idx, False)
    assert y.shape == (T, k, 1, N)
    ref = jo.gather_qmm(x.float().cpu().numpy(), *pk, idx.cpu().numpy().reshape(-1), bits, 64, np.repeat(np.arange(T), k))
    close(y.float().cpu().numpy().reshape(T * k, N), ref)
    R = 100
    xr = torch.from_numpy(rng.standard_normal((R, K)).astype(np.float32)).to(DEV).to(torch.bfloat16)
    e_idx = torch.sort(torch.from_numpy(rng.integers(0, E, R).astype(np.int32)).to(DEV)).values
    y2 = mod(xr[:, None, :], e_idx, True)
    assert y2.shape == (R, 1, N)
    close(y2.float().cpu().numpy().reshape(R, N), jo.gather_qmm(xr.float().cpu().numpy(), *pk, e_idx.cpu().numpy(), bits, 64))


def test_route_norm_rejects_in_place_output():
    from jangq_b200 import moe
    lib = _lib.load()
    x = torch.randn((2, 1024), device=DEV).to(torch.bfloat16)
    res = torch.randn((2, 1024), device=DEV).to(torch.bfloat16)
    wr = torch.randn((16, 1024), device=DEV).to(torch.bfloat16)
    idx = torch.empty((2, 4), dtype=torch.int32, device=DEV)
    w = torch.empty((2, 4), dtype=torch.float32, device=DEV)
    cnt, ws = moe._route_workspace(x.device, 2, 16)
    rc = lib.jq_moe_route_norm(x.data_ptr(), res.data_ptr(), _lib.JQ_BF16, 2, 1024, 1e-3, x.data_ptr(), wr.data_ptr(), 16, 4,
                               1, 1.0, idx.data_ptr(), w.data_ptr(), cnt.data_ptr(), ws.data_ptr(), _lib.stream_ptr())
    assert rc == _lib.JQ_EINVAL and b"must not overlap" in lib.jq_last_error()


def _np_swiglu(g, u, w, limit):
    g = g.astype(np.float32)
    u = u.astype(np.float32)
    if limit > 0:
        g = np.minimum(g, limit)
        u = np.clip(u, -limit, limit)
    h = g / (1.0 + np.exp(-g)) * u * w[:, None]
    return jo.round_to(h, "bf16")


@pytest.mark.parametrize("bits,gs,N,K", ((2, 64, 768, 2048), (4, 64, 200, 1024), (6, 64, 334, 1280), (8, 128, 40, 2048),
                                         (2, 128, 2048, 768), (6, 64, 2048, 768), (3, 64, 336, 1280), (3, 128, 96, 2048)))
@pytest.mark.parametrize("P,x_div", ((8, 8), (1, 1), (6, 1), (16, 16), (16, 8), (12, 4)))
def test_one_token_gather_on_the_item_kernel(bits, gs, N, K, P, x_div, monkeypatch):
    """Up to 16 pairs of one token (a shared row, or one row per pair) take the item-streaming integer kernel:
    against the oracle, against the warp-MMA kernel forced by the environment switch, pairs outside the bank
    written as zero rows, an expert named twice, and the two-bank form."""
    from jangq_b200.moe import _gather_qgemv, _gather_qgemv_pair
    E, base = 6, 10
    a, ref_a = make_bank(E, N, K, bits, gs, seed=31)
    b, ref_b = make_bank(E, N, K, bits, gs, seed=32)
    rng = np.random.default_rng(P * 7 + bits)
    rows = P // x_div
    x = torch.from_numpy(rng.standard_normal((rows, K)).astype(np.float32)).to(DEV).to(torch.bfloat16)
    pe_np = rng.integers(base, base + E, size=P).astype(np.int32)
    if P >= 6:
        pe_np[1], pe_np[4], pe_np[5] = 3, pe_np[0], base + E       # below the bank, a repeat, above the bank
    pe = torch.from_numpy(pe_np).to(DEV)
    y = _gather_qgemv(x, x_div, pe, a, 0, base)
    ya, yb = _gather_qgemv_pair(x, x_div, pe, a, b, 0, base)
    # same arithmetic, another split of a row's stages over the warps: one output rounding step
    assert (y.float() - ya.float()).abs().max() <= 2.0 ** -7 * ya.float().abs().max()
    local = (pe_np >= base) & (pe_np < base + E)
    lhs = np.arange(P) // x_div
    for out, ref in ((ya, ref_a), (yb, ref_b)):
        want = np.zeros((P, N), np.float32)
        want[local] = jo.gather_qmm(x.float().cpu().numpy(), ref[0], ref[1], ref[2], pe_np[local] - base, bits, gs,
                                    lhs_indices=lhs[local])
        close(out.float().cpu().numpy(), want)
        assert torch.count_nonzero(out[torch.from_numpy(~local).to(DEV)]) == 0
    monkeypatch.setenv("JANGQ_GEMV_KERNEL", "mma")
    ym = _gather_qgemv(x, x_div, pe, a, 0, base)
    monkeypatch.delenv("JANGQ_GEMV_KERNEL")
    assert (y.float() - ym.float()).abs().max() <= 2.0 ** -6 * ym.float().abs().max()
    _lib.check(_lib.load().jq_device_status())


@pytest.mark.parametrize("bits,N,K", ((2, 2048, 768), (6, 2048, 768), (4, 300, 1024), (8, 64, 512), (3, 256, 512), (5, 256, 512)))
@pytest.mark.parametrize("P", (1, 8, 16, 24))
@pytest.mark.parametrize("limit", (0.0, 1.5))
def test_gather_with_folded_swiglu(bits, N, K, P, limit):
    """jq_gather_qgemv_swiglu against the oracle's SwiGLU followed by its gather, and against the two library
    calls it replaces; 5-bit banks and more than 16 pairs take the two-launch route through h_scratch, which
    is refused when the scratch is missing."""
    lib = _lib.load()
    E, base = 5, 3
    bank, ref = make_bank(E, N, K, bits, 64, seed=41)
    bank = bank._sidecars_as(torch.bfloat16)
    rng = np.random.default_rng(P + bits)
    g = torch.from_numpy(rng.standard_normal((P, K)).astype(np.float32) * 2).to(DEV).to(torch.bfloat16)
    u = torch.from_numpy(rng.standard_normal((P, K)).astype(np.float32) * 2).to(DEV).to(torch.bfloat16)
    w = torch.from_numpy(rng.random(P).astype(np.float32) + 0.1).to(DEV)
    pe_np = rng.integers(base, base + E, size=P).astype(np.int32)
    if P >= 8:
        pe_np[2] = 0                                               # not in the bank: a zero row
    pe = torch.from_numpy(pe_np).to(DEV)
    y = torch.full((P, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    h = torch.empty((P, K), dtype=torch.bfloat16, device=DEV)

    def call(scratch):
        return lib.jq_gather_qgemv_swiglu(g.data_ptr(), u.data_ptr(), _lib.JQ_BF16, g.stride(0), w.data_ptr(), limit,
                                          pe.data_ptr(), P, bank.codes_tab.data_ptr(), bank.scales_tab.data_ptr(),
                                          bank.biases_tab.data_ptr(), None, E, _lib.JQ_BF16, N, K, bits, 64, y.data_ptr(),
                                          y.stride(0), base, 0, scratch, _lib.stream_ptr())

    two_launch = bits == 5 or P > 16
    if two_launch:
        assert call(None) == _lib.JQ_EWORKSPACE
    _lib.check(call(h.data_ptr() if two_launch else None))
    local = (pe_np >= base) & (pe_np < base + E)
    hn = _np_swiglu(g.float().cpu().numpy(), u.float().cpu().numpy(), w.cpu().numpy(), limit)
    want = np.zeros((P, N), np.float32)
    want[local] = jo.gather_qmm(hn[local], ref[0], ref[1], ref[2], pe_np[local] - base, bits, 64)
    close(y.float().cpu().numpy(), want)
    assert torch.count_nonzero(y[torch.from_numpy(~local).to(DEV)]) == 0
    # the two calls it replaces
    _lib.check(lib.jq_moe_swiglu(g.data_ptr(), u.data_ptr(), g.stride(0), w.data_ptr(), None, None, h.data_ptr(), K, K, P,
                                 limit, _lib.JQ_BF16, _lib.stream_ptr()))
    from jangq_b200.moe import _gather_qgemv
    y2 = _gather_qgemv(h, 1, pe, bank, 0, base)
    assert (y.float() - y2.float()).abs().max() <= 2.0 ** -6 * y2.float().abs().max()
    _lib.check(lib.jq_device_status())


@pytest.mark.parametrize("world,C", ((2, 40), (4, 16), (8, 64), (2, 7)))
def test_ep_slot_packing_covers_every_pair_once(world, C):
    """jq_ep_pack_slots: every pair lands in exactly one slot of its destination rank with its row, local expert id
    and weight; empty slots carry id -1; a destination with more pairs than slots drops the surplus, reports them
    as -1 and sets the overflow word."""
    lib = _lib.load()
    T, k, H, E = 9, 4, 256, 16
    rng = np.random.default_rng(world * 100 + C)
    x = torch.from_numpy(rng.standard_normal((T, H)).astype(np.float32)).to(DEV).to(torch.bfloat16)
    idx = torch.from_numpy(rng.integers(0, E, size=(T, k)).astype(np.int32)).to(DEV)
    w = torch.from_numpy(rng.random((T, k)).astype(np.float32)).to(DEV)
    Hp = H + 8
    send = torch.full((world * C, Hp), 7.0, dtype=torch.bfloat16, device=DEV)
    sop = torch.full((T * k,), -5, dtype=torch.int32, device=DEV)
    scratch = torch.full((world + 1,), 99, dtype=torch.int32, device=DEV)
    _lib.check(lib.jq_ep_pack_slots(x.data_ptr(), H, idx.data_ptr(), w.data_ptr(), T, k, H, E, world, C, send.data_ptr(),
                                    sop.data_ptr(), scratch.data_ptr(), scratch[world:].data_ptr(), _lib.stream_ptr()))
    torch.cuda.synchronize()
    e_local = E // world
    dest = idx.cpu().numpy().reshape(-1) // e_local
    counts = np.bincount(dest, minlength=world)
    assert scratch[:world].cpu().numpy().tolist() == counts.tolist()
    assert bool(scratch[world]) == bool((counts > C).any())
    sop_h = sop.cpu().numpy()
    ids = send.view(torch.int32)[:, H // 2].cpu().numpy()
    wts = send.view(torch.float32)[:, H // 2 + 1].cpu().numpy()
    rows = send[:, :H].float().cpu().numpy()
    used = sop_h[sop_h >= 0]
    assert len(set(used.tolist())) == used.size                       # no slot twice
    for r in range(world):
        assert ((sop_h >= r * C) & (sop_h < (r + 1) * C)).sum() == min(counts[r], C)
    xh, wh, ih = x.float().cpu().numpy(), w.cpu().numpy().reshape(-1), idx.cpu().numpy().reshape(-1)
    for p, s in enumerate(sop_h):
        if s < 0:
            assert counts[dest[p]] > C
            continue
        assert s // C == dest[p] and ids[s] == ih[p] - dest[p] * e_local and wts[s] == wh[p]
        assert np.array_equal(rows[s], xh[p // k])
    free = np.setdiff1d(np.arange(world * C), used)
    assert (ids[free] == -1).all()


@pytest.mark.parametrize("T,E,k,dtype", ((2048, 128, 8, torch.bfloat16), (33, 1000, 32, torch.float32), (5, 7, 7, torch.float16),
                                         (300, 512, 10, torch.bfloat16)))
def test_topk_over_logit_rows(T, E, k, dtype):
    """jq_moe_topk (one warp per token) against the oracle's softmax / top-k: ids bit-exact including ties (16-bit
    logits collide often: ties go to the lower id), weights to f32 rounding; a padded leading dimension."""
    rng = np.random.default_rng(T + E)
    full = torch.from_numpy(rng.standard_normal((T, E + 8)).astype(np.float32)).to(DEV).to(dtype)
    logits = full[:, :E]
    idx, w = jq.route_softmax_topk(logits, k)
    idx_ref, w_ref = jo.route_softmax_topk(logits.float().cpu().numpy(), k)
    assert np.array_equal(idx.cpu().numpy(), idx_ref)
    assert np.allclose(w.cpu().numpy(), w_ref, rtol=2e-5, atol=1e-7)
    idx2, w2 = jq.route_softmax_topk(logits, k, renorm=False, scale=2.5)
    _, w_ref2 = jo.route_softmax_topk(logits.float().cpu().numpy(), k, renorm=False, scale=2.5)
    assert np.array_equal(idx2.cpu().numpy(), idx_ref) and np.allclose(w2.cpu().numpy(), w_ref2, rtol=2e-5, atol=1e-7)


@pytest.mark.parametrize("bits,N,K", ((2, 768, 2048), (6, 200, 1024), (3, 96, 1280), (8, 2048, 768)))
@pytest.mark.parametrize("P,x_div,E,base,E_all", ((64, 8, 16, 32, 128), (32, 1, 4, 8, 16), (128, 8, 8, 0, 16), (40, 1, 16, 0, 16),
                                                   (24, 8, 2, 6, 64)))
def test_gather_of_many_pairs_few_of_them_local(bits, N, K, P, x_div, E, base, E_all):
    """JQ_GATHER_FEW_LOCAL: up to 128 pairs on the integer gather, the local ones compacted and walked 16 at a time
    (the (40, 1, 16, 0, 16) case has every pair local: three rounds; (24, 8, 2, 6, 64) usually has none), rows shared
    by x_div pairs or one per pair, two banks; against the oracle and the bf16 warp-MMA gather."""
    lib = _lib.load()
    a, ref_a = make_bank(E, N, K, bits, 64, seed=51)
    b, ref_b = make_bank(E, N, K, bits, 64, seed=52)
    a, b = a._sidecars_as(torch.bfloat16), b._sidecars_as(torch.bfloat16)
    rng = np.random.default_rng(P + bits + E)
    rows = P // x_div
    x = torch.from_numpy(rng.standard_normal((rows, K)).astype(np.float32)).to(DEV).to(torch.bfloat16)
    pe_np = rng.integers(0, E_all, size=P).astype(np.int32)
    pe = torch.from_numpy(pe_np).to(DEV)

    def run(flags):
        y = torch.full((2, P, N), float("nan"), dtype=torch.bfloat16, device=DEV)
        _lib.check(lib.jq_gather_qgemv2(x.data_ptr(), _lib.JQ_BF16, x.stride(0), x_div, pe.data_ptr(), P, a.codes_tab.data_ptr(),
                                        a.scales_tab.data_ptr(), a.biases_tab.data_ptr(), b.codes_tab.data_ptr(),
                                        b.scales_tab.data_ptr(), b.biases_tab.data_ptr(), None, E, _lib.JQ_BF16, N, K, bits, 64,
                                        y[0].data_ptr(), y[1].data_ptr(), y.stride(1), base, flags, _lib.stream_ptr()))
        return y

    ys = run(_lib.JQ_GATHER_FEW_LOCAL | _lib.JQ_GEMV_STATIC_WEIGHTS)
    ym = run(0)
    torch.cuda.synchronize()
    local = (pe_np >= base) & (pe_np < base + E)
    lhs = np.arange(P) // x_div
    for i, ref in enumerate((ref_a, ref_b)):
        want = np.zeros((P, N), np.float32)
        if local.any():
            want[local] = jo.gather_qmm(x.float().cpu().numpy(), ref[0], ref[1], ref[2], pe_np[local] - base, bits, 64,
                                        lhs_indices=lhs[local])
            close(ys[i].float().cpu().numpy(), want)
        assert torch.count_nonzero(ys[i][torch.from_numpy(~local).to(DEV)]) == 0
        assert not torch.isnan(ys[i].float()).any()
        assert (ys[i].float() - ym[i].float()).abs().max() <= 2.0 ** -6 * max(float(ym[i].float().abs().max()), 1e-6)
    _lib.check(lib.jq_device_status())


@pytest.mark.parametrize("P,E,base,E_all", ((64, 16, 16, 128), (48, 8, 0, 8)))
def test_swiglu_gather_of_many_pairs_few_of_them_local(P, E, base, E_all):
    """jq_gather_qgemv_swiglu with JQ_GATHER_FEW_LOCAL: one set of limbs per local pair a CTA's tiles touch."""
    lib = _lib.load()
    N, K, bits = 2048, 768, 2
    bank, ref = make_bank(E, N, K, bits, 64, seed=61)
    bank = bank._sidecars_as(torch.bfloat16)
    rng = np.random.default_rng(P)
    g = torch.from_numpy(rng.standard_normal((P, K)).astype(np.float32) * 2).to(DEV).to(torch.bfloat16)
    u = torch.from_numpy(rng.standard_normal((P, K)).astype(np.float32) * 2).to(DEV).to(torch.bfloat16)
    w = torch.from_numpy(rng.random(P).astype(np.float32) + 0.1).to(DEV)
    pe_np = rng.integers(0, E_all, size=P).astype(np.int32)
    pe = torch.from_numpy(pe_np).to(DEV)
    y = torch.full((P, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    _lib.check(lib.jq_gather_qgemv_swiglu(g.data_ptr(), u.data_ptr(), _lib.JQ_BF16, g.stride(0), w.data_ptr(), 0.0,
                                          pe.data_ptr(), P, bank.codes_tab.data_ptr(), bank.scales_tab.data_ptr(),
                                          bank.biases_tab.data_ptr(), None, E, _lib.JQ_BF16, N, K, bits, 64, y.data_ptr(),
                                          y.stride(0), base, _lib.JQ_GATHER_FEW_LOCAL, None, _lib.stream_ptr()))
    torch.cuda.synchronize()
    local = (pe_np >= base) & (pe_np < base + E)
    hn = _np_swiglu(g.float().cpu().numpy(), u.float().cpu().numpy(), w.cpu().numpy(), 0.0)
    want = np.zeros((P, N), np.float32)
    want[local] = jo.gather_qmm(hn[local], ref[0], ref[1], ref[2], pe_np[local] - base, bits, 64)
    close(y.float().cpu().numpy(), want)
    assert torch.count_nonzero(y[torch.from_numpy(~local).to(DEV)]) == 0
    _lib.check(lib.jq_device_status())
