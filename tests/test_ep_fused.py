"""Fused expert-parallel dispatch / combine: the row plan against a dense statement of the MoE
data movement (CPU, all ranks emulated in one process) and the two kernels against the plain
torch statements (one GPU, one buffer per emulated rank; the kernels never wait on each other,
so launching the ranks one after another is a valid schedule)."""
import types

import pytest
import torch

from areal_b200.parallel import ep_fused as EF


def _routing(ep, E, k, T, H, seed, device="cpu", dtype=torch.float32, skew=False):
    g = torch.Generator().manual_seed(seed)
    ranks = []
    for r in range(ep):
        x = torch.randn(T + 3 * r, H, generator=g).to(dtype).to(device)
        scores = torch.rand(x.shape[0], E, generator=g)
        if skew:
            scores[:, : E // ep] += 0.5            # most tokens go to rank 0's experts
            scores[:, -1] = -1.0                   # one expert receives nothing
        topw, tope = scores.topk(k, dim=-1)
        flat_e = tope.reshape(-1).to(device)
        order = torch.argsort(flat_e, stable=True)
        ranks.append(dict(x=x, topw=topw.to(device), flat_e=flat_e, order=order))
    counts = torch.stack([torch.bincount(r["flat_e"], minlength=E) for r in ranks])
    for r, d in enumerate(ranks):
        d["plan"] = EF.build_plan(counts, d["order"], d["flat_e"][d["order"]], r, k)
    return ranks, counts


def _expert_fn(e, rows):
    return rows * (1.0 + 0.25 * e) + 0.125 * e


def _dense_expected(d, E, k):
    x, topw, flat_e = d["x"].float(), d["topw"].float(), d["flat_e"]
    out = torch.zeros_like(x)
    for t in range(x.shape[0]):
        for j in range(k):
            e = int(flat_e[t * k + j])
            out[t] += topw[t, j] * _expert_fn(e, x[t])
    return out


@pytest.mark.parametrize("ep,E,k,skew", [(2, 8, 2, False), (4, 8, 3, True), (1, 4, 2, False)])
def test_plan_places_rows_in_expert_order(ep, E, k, skew):
    H, El = 16, E // ep
    ranks, counts = _routing(ep, E, k, 11, H, seed=ep * 10 + k, skew=skew)
    cap = max(d["plan"].max_recv for d in ranks)
    assert len({d["plan"].max_recv for d in ranks}) == 1
    bufs = [torch.full((cap, H), float("nan")) for _ in range(ep)]
    for d in ranks:
        EF.dispatch_reference(d["x"], d["plan"], bufs)
    for r, d in enumerate(ranks):
        p = d["plan"]
        assert p.n_recv == int(counts[:, r * El:(r + 1) * El].sum()) and sum(p.per_expert) == p.n_recv
        assert not torch.isnan(bufs[r][: p.n_recv]).any()          # every receive row written exactly by someone
        # rows are grouped by local expert, and inside an expert by source rank
        off = 0
        for e in range(El):
            for s, ds in enumerate(ranks):
                sel = ds["flat_e"][ds["order"]] == r * El + e
                want = ds["x"][ds["plan"].token_of.long()][sel]
                n = want.shape[0]
                assert torch.equal(bufs[r][off:off + n], want)
                off += n
    # experts run on the buffers in place; combine returns the weighted sum per token
    outs = [b.clone() for b in bufs]
    for r, d in enumerate(ranks):
        off = 0
        for e, n in enumerate(d["plan"].per_expert):
            outs[r][off:off + n] = _expert_fn(r * El + e, bufs[r][off:off + n])
            off += n
    for d in ranks:
        w = d["topw"].reshape(-1)[d["order"]]
        got, ys = EF.combine_reference(outs, d["plan"], w=w, save=True)
        torch.testing.assert_close(got, _dense_expected(d, E, k), rtol=1e-5, atol=1e-5)
        assert ys.shape == (d["plan"].drank.numel(), H)


def test_reference_backward_identities():
    """dispatch backward == combine with unit weights; combine backward == scaled dispatch + dot."""
    ep, E, k, H = 2, 4, 2, 8
    ranks, _ = _routing(ep, E, k, 7, H, seed=3)
    cap = ranks[0]["plan"].max_recv
    d = ranks[0]
    # gradient of sum(got * G) w.r.t. x, with G per receive row, via autograd on the dense gather
    G = [torch.randn(cap, H) for _ in range(ep)]
    x = d["x"].clone().requires_grad_(True)
    rows = x[d["plan"].token_of.long()]
    loss = sum((rows[d["plan"].drank == r] * G[r][d["plan"].drow[d["plan"].drank == r].long()]).sum() for r in range(ep))
    loss.backward()
    dx, _ = EF.combine_reference(G, d["plan"])
    torch.testing.assert_close(dx, x.grad, rtol=1e-5, atol=1e-5)
    # combine backward
    ys = torch.randn(d["plan"].drank.numel(), H)
    w = torch.rand(d["plan"].drank.numel(), requires_grad=True)
    ysg = ys.clone().requires_grad_(True)
    out = (ysg * w.unsqueeze(-1))[d["plan"].inv.long()].view(d["plan"].n_tokens, k, H).sum(1)
    dout = torch.randn_like(out)
    out.backward(dout)
    bufs = [torch.zeros(cap, H) for _ in range(ep)]
    dw = EF.dispatch_reference(dout, d["plan"], bufs, scale=w.detach(), ys=ys)
    torch.testing.assert_close(dw, w.grad, rtol=1e-4, atol=1e-5)
    back, _ = None, None
    got = torch.zeros_like(ys)
    for r in range(ep):
        sel = d["plan"].drank == r
        got[sel] = bufs[r][d["plan"].drow[sel].long()]
    torch.testing.assert_close(got, ysg.grad, rtol=1e-5, atol=1e-5)


@pytest.mark.gpu
@pytest.mark.parametrize("ep,E,k,H,T", [(2, 8, 2, 256, 300), (4, 16, 8, 2048, 1024), (1, 4, 2, 72, 50)])
def test_kernels_match_reference_on_emulated_ranks(ep, E, k, H, T):
    from areal_b200.ops import lib as oplib
    from areal_b200.parallel.symm import ptr_array

    dev = torch.device("cuda:0")
    ranks, _ = _routing(ep, E, k, T, H, seed=7, device=dev, dtype=torch.bfloat16, skew=True)
    cap = ranks[0]["plan"].max_recv + 5
    comm = types.SimpleNamespace(world=ep, hidden=H, capacity=cap, device=dev)
    bufs = [torch.zeros(cap, H, dtype=torch.bfloat16, device=dev) for _ in range(ep)]
    ref = [torch.zeros(cap, H, dtype=torch.bfloat16, device=dev) for _ in range(ep)]
    slab = (None, None, ptr_array([b.data_ptr() for b in bufs]))
    for d in ranks:
        EF._dispatch(comm, d["x"], d["plan"], slab)
        EF.dispatch_reference(d["x"], d["plan"], ref)
    for a, b in zip(bufs, ref):
        assert torch.equal(a, b)
    for d in ranks:
        w = d["topw"].reshape(-1)[d["order"]].float()
        out, ys = EF._combine(comm, d["plan"], slab, w=w, save=True)
        want, ys_ref = EF.combine_reference(ref, d["plan"], w=w, save=True)
        assert torch.equal(ys, ys_ref)
        torch.testing.assert_close(out.float(), want.float(), rtol=2e-2, atol=2e-2)
        # the scaled dispatch of the combine backward, with the gate-weight gradients
        dout = torch.randn(d["plan"].n_tokens, H, device=dev, dtype=torch.bfloat16)
        for b in bufs + ref:
            b.zero_()
        dw = EF._dispatch(comm, dout, d["plan"], slab, scale=w, ys=ys)
        dw_ref = EF.dispatch_reference(dout, d["plan"], ref, scale=w, ys=ys)
        torch.testing.assert_close(dw, dw_ref, rtol=1e-3, atol=1e-2)
        for a, b in zip(bufs, ref):
            torch.testing.assert_close(a.float(), b.float(), rtol=1e-2, atol=1e-2)
        # unit-weight combine (dispatch backward)
        dx, _ = EF._combine(comm, d["plan"], slab)
        dx_ref, _ = EF.combine_reference(ref, d["plan"])
        torch.testing.assert_close(dx.float(), dx_ref.float(), rtol=2e-2, atol=2e-2)
    assert oplib.kernel_error() == 0
