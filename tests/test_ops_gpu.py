"""Numerics of the sm_100a kernels against plain PyTorch fp32 references."""
import math

import pytest
import torch

from areal_b200.ops import functional as OF
from areal_b200.ops import lib as oplib

pytestmark = pytest.mark.gpu


def _no_kernel_error():
    assert oplib.kernel_error() == 0


def _rel_err(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (300, 200, 136), (1024, 4096, 1024), (64, 6144, 4096)])
def test_gemm_layouts(a_mn, b_mn, M, N, K):
    if (a_mn and M % 8) or (b_mn and N % 8):
        pytest.skip("MN-major operands need the contiguous dim to be a multiple of 8")
    torch.manual_seed(0)
    dev = "cuda"
    A = torch.randn(M, K, device=dev).bfloat16()
    B = torch.randn(N, K, device=dev).bfloat16()
    a = A.t().contiguous() if a_mn else A
    b = B.t().contiguous() if b_mn else B
    ref = A.float() @ B.float().t()
    out = OF.gemm(a, b, a_mn=a_mn, b_mn=b_mn)
    _no_kernel_error()
    assert _rel_err(out, ref) < 1e-2
    out32 = OF.gemm(a, b, a_mn=a_mn, b_mn=b_mn, epi=OF.EPI_F32)
    assert _rel_err(out32, ref) < 2e-3
    acc = torch.ones(M, N, device=dev)
    OF.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out=acc, epi=OF.EPI_F32_ACC)
    assert _rel_err(acc, ref + 1) < 2e-3
    R = torch.randn(M, N, device=dev).bfloat16()
    outr = OF.gemm(a, b, a_mn=a_mn, b_mn=b_mn, epi=OF.EPI_BF16_RESID, resid=R)
    assert _rel_err(outr, ref + R.float()) < 1e-2
    _no_kernel_error()


@pytest.mark.parametrize("bn", [32, 64, 128, 256])
def test_gemm_tile_widths(bn):
    torch.manual_seed(1)
    A = torch.randn(384, 512, device="cuda").bfloat16()
    B = torch.randn(640, 512, device="cuda").bfloat16()
    out = OF.gemm(A, B, bn=bn)
    _no_kernel_error()
    assert _rel_err(out, A.float() @ B.float().t()) < 1e-2


@pytest.mark.parametrize("M,N,K,split", [(1, 256, 64, 1), (7, 4096, 4096, 0), (33, 6144, 4096, 0), (128, 4096, 12288, 0),
                                          (200, 1000, 520, 4), (256, 24576, 4096, 0), (64, 151936, 1024, 0), (16, 384, 4096, 16)])
def test_gemm_skinny_matches_fp32(M, N, K, split):
    """Decode-shaped GEMM (swap-AB, split-K reduced in L2) against an fp32 matmul; two calls in a
    row check that the workspace and tile counters are left zeroed."""
    torch.manual_seed(3)
    x = torch.randn(M, K, device="cuda").bfloat16()
    w = (torch.randn(N, K, device="cuda") / K ** 0.5).bfloat16()
    r = torch.randn(M, N, device="cuda").bfloat16()
    ref = x.float() @ w.float().t()
    for _ in range(2):
        y = OF.gemm_skinny(x, w, split_k=split)
        assert _rel_err(y, ref) < 1e-2
    y32 = OF.gemm_skinny(x, w, out_dtype=torch.float32, split_k=split)
    assert _rel_err(y32, ref) < 2e-3
    yr = OF.gemm_skinny(x, w, resid=r, split_k=split)
    assert _rel_err(yr, ref + r.float()) < 1e-2
    with torch.no_grad():
        assert _rel_err(OF.linear(x, w, r), ref + r.float()) < 1e-2      # inference-shaped linear may take this path
    _no_kernel_error()


def test_linear_autograd():
    torch.manual_seed(2)
    x = torch.randn(512, 256, device="cuda").bfloat16().requires_grad_()
    w = torch.randn(384, 256, device="cuda").bfloat16().requires_grad_()
    y = OF.linear(x, w)
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().float().requires_grad_()
    wr = w.detach().float().requires_grad_()
    (xr @ wr.t()).backward(g.float())
    assert _rel_err(x.grad, xr.grad) < 1e-2
    assert _rel_err(w.grad, wr.grad) < 1e-2
    _no_kernel_error()


@pytest.mark.parametrize("H", [128, 1536, 4096, 8192])
def test_rmsnorm(H):
    torch.manual_seed(3)
    x = torch.randn(300, H, device="cuda").bfloat16().requires_grad_()
    r = torch.randn(300, H, device="cuda").bfloat16().requires_grad_()
    w = (1 + 0.1 * torch.randn(H, device="cuda")).bfloat16().requires_grad_()
    y, res = OF.rmsnorm(x, w, 1e-6, r)
    gy, gr = torch.randn_like(y), torch.randn_like(res)
    (y.float() * gy.float()).sum().add((res.float() * gr.float()).sum()).backward()
    xr, rr, wr = (t.detach().float().requires_grad_() for t in (x, r, w))
    s = (xr + rr).bfloat16().float().detach() + (xr + rr - (xr + rr).detach())  # bf16-rounded stream, fp32 grads
    yr = s * torch.rsqrt(s.pow(2).mean(-1, keepdim=True) + 1e-6) * wr
    ((yr * gy.float()).sum() + (s * gr.float()).sum()).backward()
    assert _rel_err(y, yr) < 1e-2
    assert _rel_err(x.grad, xr.grad) < 2e-2
    assert _rel_err(r.grad, rr.grad) < 2e-2
    assert _rel_err(w.grad, wr.grad) < 2e-2


def test_rope_roundtrip_and_ref():
    torch.manual_seed(4)
    T, h, D = 257, 6, 128
    x = torch.randn(T, h, D, device="cuda").bfloat16()
    pos = torch.randint(0, 1000, (T,), device="cuda", dtype=torch.int32)
    cos, sin = OF.rope_tables(1024, D, 1e6, "cuda")
    y = OF.rope(x, pos, cos, sin)
    assert _rel_err(y, OF.rope_ref(x, pos.long(), cos, sin)) < 1e-2
    xg = x.clone().requires_grad_()
    OF.rope(xg, pos, cos, sin).backward(y)
    assert _rel_err(xg.grad, x) < 2e-2  # inverse rotation recovers the input


def test_swiglu():
    torch.manual_seed(5)
    gu = torch.randn(333, 2 * 688, device="cuda").bfloat16().requires_grad_()
    o = OF.swiglu(gu)
    g = torch.randn_like(o)
    o.backward(g)
    gr = gu.detach().float().requires_grad_()
    I = 688
    orf = torch.nn.functional.silu(gr[:, :I]) * gr[:, I:]
    orf.backward(g.float())
    assert _rel_err(o, orf) < 1e-2
    assert _rel_err(gu.grad, gr.grad) < 1e-2


def test_embedding():
    torch.manual_seed(6)
    W = torch.randn(1000, 256, device="cuda").bfloat16().requires_grad_()
    ids = torch.randint(0, 1000, (777,), device="cuda")
    o = OF.embedding(ids, W)
    assert torch.equal(o, W.detach()[ids])
    g = torch.randn_like(o)
    o.backward(g)
    ref = torch.zeros(1000, 256, device="cuda").index_add_(0, ids, g.float())
    assert _rel_err(W.grad, ref) < 1e-2


def test_adamw_and_clip():
    torch.manual_seed(7)
    n = 100003
    p = torch.randn(n, device="cuda")
    g = torch.randn(n, device="cuda") * 3
    m = torch.zeros(n, device="cuda")
    v = torch.zeros(n, device="cuda")
    pb = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    pr = p.clone().requires_grad_()
    opt = torch.optim.AdamW([pr], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    state = torch.zeros(4, device="cuda")
    for step in range(1, 4):
        state.zero_()
        OF.sqnorm_accumulate_(g, state)
        OF.clip_coef_(state, 1.0)
        OF.adamw_step_(p, m, v, g, pb, state, 1e-2, 0.9, 0.95, 1e-8, 0.1, step)
        pr.grad = g.clone()
        torch.nn.utils.clip_grad_norm_([pr], 1.0)
        opt.step()
    assert abs(state[3].item() - g.norm().item()) / g.norm().item() < 1e-4
    assert _rel_err(p, pr.detach()) < 1e-5
    assert _rel_err(pb, pr.detach()) < 1e-2


@pytest.mark.parametrize("V", [1024, 151936, 1001])
def test_logprob_entropy(V):
    torch.manual_seed(8)
    T = 37
    logits = torch.randn(T, V, device="cuda") * 3
    labels = torch.randint(0, V, (T,), device="cuda")
    if V % 4:
        pytest.skip("row stride must be a multiple of 4 floats")
    lp, ent, lse = OF.logprob_entropy_from_logits(logits, labels, 0.7)
    lpr, entr = OF.logprob_entropy_ref(logits, labels, 0.7)
    assert (lp - lpr).abs().max().item() < 1e-3
    assert (ent - entr).abs().max().item() < 1e-3


def test_lm_head_logprob_autograd():
    torch.manual_seed(9)
    T, H, V = 300, 256, 1024
    h = (torch.randn(T, H, device="cuda") * 0.5).bfloat16().requires_grad_()
    W = (torch.randn(V, H, device="cuda") * 0.1).bfloat16().requires_grad_()
    labels = torch.randint(0, V, (T,), device="cuda")
    lp, ent = OF.lm_head_logprob(h, W, labels, 1.0, chunk=128)
    gl, ge = torch.randn(T, device="cuda"), torch.randn(T, device="cuda") * 0.1
    ((lp * gl).sum() + (ent * ge).sum()).backward()
    hr, Wr = h.detach().float().requires_grad_(), W.detach().float().requires_grad_()
    lpr, entr = OF.logprob_entropy_ref(hr @ Wr.t(), labels, 1.0)
    ((lpr * gl).sum() + (entr * ge).sum()).backward()
    assert (lp - lpr).abs().max().item() < 2e-2
    assert (ent - entr).abs().max().item() < 2e-2
    assert _rel_err(h.grad, hr.grad) < 3e-2
    assert _rel_err(W.grad, Wr.grad) < 3e-2
    _no_kernel_error()


@pytest.mark.parametrize("D", [128, 64])
@pytest.mark.parametrize("causal", [True, False])
def test_attention_fwd(D, causal):
    torch.manual_seed(10)
    lens = [1, 130, 257, 128, 515, 64]
    T = sum(lens)
    Hq, Hkv = 4, 2
    qkv = torch.randn(T, (Hq + 2 * Hkv) * D, device="cuda").bfloat16()
    q = qkv[:, : Hq * D].view(T, Hq, D)
    k = qkv[:, Hq * D: (Hq + Hkv) * D].view(T, Hkv, D)
    v = qkv[:, (Hq + Hkv) * D:].view(T, Hkv, D)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), device="cuda", dtype=torch.int32)
    o, lse = OF.attention_fwd(q, k, v, cu, causal)
    _no_kernel_error()
    orf, lser = OF.attention_ref(q, k, v, cu, causal)
    assert _rel_err(o, orf) < 2e-2
    assert (lse - lser).abs().max().item() < 2e-2


@pytest.mark.parametrize("D", [128, 64])
@pytest.mark.parametrize("causal", [True, False])
def test_attention_bwd(D, causal):
    torch.manual_seed(11)
    lens = [1, 130, 257, 128, 515, 64]
    T = sum(lens)
    Hq, Hkv = 4, 2
    qkv = (torch.randn(T, (Hq + 2 * Hkv) * D, device="cuda") * 0.7).bfloat16()
    q = qkv[:, : Hq * D].view(T, Hq, D)
    k = qkv[:, Hq * D: (Hq + Hkv) * D].view(T, Hkv, D)
    v = qkv[:, (Hq + Hkv) * D:].view(T, Hkv, D)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), device="cuda", dtype=torch.int32)
    o, lse = OF.attention_fwd(q, k, v, cu, causal)
    do = torch.randn_like(o)
    scale = D ** -0.5
    dq, dk, dv = OF.attention_bwd(q, k, v, o, lse, do, cu, causal, scale)
    _no_kernel_error()
    orf, lser = OF.attention_ref(q, k, v, cu, causal)
    dqr, dkr, dvr = OF.attention_bwd_ref(q, k, v, orf, lser, do, cu, causal, scale)
    assert _rel_err(dq, dqr) < 3e-2
    assert _rel_err(dk, dkr) < 3e-2
    assert _rel_err(dv, dvr) < 3e-2


def test_attention_autograd_matches_reference_path():
    torch.manual_seed(12)
    T, Hq, Hkv, D = 700, 8, 2, 128
    q = torch.randn(T, Hq, D, device="cuda").bfloat16().requires_grad_()
    k = torch.randn(T, Hkv, D, device="cuda").bfloat16().requires_grad_()
    v = torch.randn(T, Hkv, D, device="cuda").bfloat16().requires_grad_()
    cu = torch.tensor([0, 300, 700], device="cuda", dtype=torch.int32)
    g = torch.randn(T, Hq, D, device="cuda").bfloat16()
    OF.attention(q, k, v, cu, True).backward(g)
    got = [t.grad.clone() for t in (q, k, v)]
    for t in (q, k, v):
        t.grad = None
    saved = OF._ATTN_BWD_IMPL
    OF._ATTN_BWD_IMPL = None
    try:
        OF.attention(q, k, v, cu, True).backward(g)
    finally:
        OF._ATTN_BWD_IMPL = saved
    for a, t in zip(got, (q, k, v)):
        assert _rel_err(a, t.grad) < 3e-2
    _no_kernel_error()


@pytest.mark.parametrize("D,nq,nkv,norm", [(128, 8, 2, True), (128, 4, 4, False), (64, 6, 2, True)])
def test_fused_qknorm_rope_attention_matches_fp32(D, nq, nkv, norm):
    """Fused QK-norm + RoPE + attention block (forward, dqkv, norm-weight grads) against plain
    PyTorch fp32 math with autograd."""
    import math

    torch.manual_seed(5)
    dev = "cuda"
    lens = [130, 257, 64, 61]
    T = sum(lens)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), device=dev, dtype=torch.int32)
    pos = torch.cat([torch.arange(n) for n in lens]).to(dev).int()
    W = (nq + 2 * nkv) * D
    qkv = torch.randn(T, W, device=dev).bfloat16().requires_grad_()
    wq = (1 + 0.1 * torch.randn(D, device=dev)).bfloat16().requires_grad_() if norm else None
    wk = (1 + 0.1 * torch.randn(D, device=dev)).bfloat16().requires_grad_() if norm else None
    cos, sin = OF.rope_tables(512, D, 1e4, dev)
    eps = 1e-6
    o = OF.qknorm_rope_attention(qkv, wq, wk, pos, cos, sin, cu, nq, nkv, D, eps)
    g = torch.randn_like(o)
    o.backward(g)
    _no_kernel_error()

    # ---- fp32 oracle
    x = qkv.detach().float().requires_grad_()
    wq32 = wq.detach().float().requires_grad_() if norm else None
    wk32 = wk.detach().float().requires_grad_() if norm else None
    q = x[:, : nq * D].view(T, nq, D)
    k = x[:, nq * D:(nq + nkv) * D].view(T, nkv, D)
    v = x[:, (nq + nkv) * D:].view(T, nkv, D)

    def nrm(t, w):
        return t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + eps) * w

    def rot(t):
        c, s_ = cos[pos.long()][:, None, :], sin[pos.long()][:, None, :]
        a, b = t[..., : D // 2], t[..., D // 2:]
        return torch.cat([a * c - b * s_, b * c + a * s_], -1)
    if norm:
        q, k = nrm(q, wq32), nrm(k, wk32)
    q, k = rot(q), rot(k)
    outs = []
    rep = nq // nkv
    b = 0
    for n in lens:
        qi = q[b:b + n].transpose(0, 1)
        ki = k[b:b + n].transpose(0, 1).repeat_interleave(rep, 0)
        vi = v[b:b + n].transpose(0, 1).repeat_interleave(rep, 0)
        sc = (qi @ ki.transpose(1, 2)) / math.sqrt(D)
        sc = sc.masked_fill(~torch.tril(torch.ones(n, n, device=dev, dtype=torch.bool)), float("-inf"))
        outs.append((torch.softmax(sc, -1) @ vi).transpose(0, 1))
        b += n
    ref = torch.cat(outs, 0)
    ref.backward(g.float())
    assert _rel_err(o, ref) < 2e-2
    assert _rel_err(qkv.grad, x.grad) < 3e-2
    if norm:
        assert _rel_err(wq.grad, wq32.grad) < 3e-2 and _rel_err(wk.grad, wk32.grad) < 3e-2


@pytest.mark.parametrize("counts", [[130, 0, 77, 256, 1], [5, 5, 5, 5], [0, 0, 300]])
def test_grouped_gemm_matches_fp32(counts):
    """Grouped expert GEMM (variable row groups, 3-D tensor map over the expert stack) forward,
    input gradient and weight gradient against per-expert fp32 matmuls."""
    torch.manual_seed(6)
    E, K, N = len(counts), 256, 384
    R = sum(counts)
    x = torch.randn(R, K, device="cuda").bfloat16().requires_grad_()
    w = (torch.randn(E, N, K, device="cuda") / K ** 0.5).bfloat16().requires_grad_()
    y = OF.grouped_linear(x, w, counts)
    g = torch.randn_like(y)
    y.backward(g)
    _no_kernel_error()
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    outs, off = [], 0
    for e, n in enumerate(counts):
        if n:
            outs.append(xr[off:off + n] @ wr[e].t())
        off += n
    ref = torch.cat(outs, 0)
    ref.backward(g.float())
    assert _rel_err(y, ref) < 1e-2 and _rel_err(x.grad, xr.grad) < 1e-2 and _rel_err(w.grad, wr.grad) < 1e-2


@pytest.mark.parametrize("T,E,k,sigmoid,bias", [(3000, 128, 8, False, False), (517, 64, 6, True, True), (40, 32, 1, False, False),
                                                (5000, 96, 4, False, True)])
def test_moe_route_kernels_match_pytorch(T, E, k, sigmoid, bias):
    """Device-side routing (scores, top-k, stable sort by expert, group sizes, GEMM tile list) against
    softmax / topk / argsort / bincount in PyTorch, and the same bits when run twice."""
    g = torch.Generator(device="cuda").manual_seed(T + E)
    logits = torch.randn(T, E, device="cuda", generator=g) * 2.0
    b = torch.randn(E, device="cuda", generator=g) * 0.05 if bias else None
    r = OF.moe_route(logits, k, bias=b, sigmoid=sigmoid, norm=True, scale=1.5)
    torch.cuda.synchronize()
    _no_kernel_error()
    ref = OF.moe_route_ref(logits, k, bias=b, sigmoid=sigmoid, norm=True, scale=1.5)
    assert torch.allclose(r.probs, ref.probs, atol=1e-6, rtol=1e-5)
    # random fp32 scores have no ties: the chosen sets and their order agree
    assert torch.equal(r.tope, ref.tope) and torch.allclose(r.topw, ref.topw, atol=1e-6, rtol=1e-5)
    assert torch.equal(r.counts, ref.counts) and torch.equal(r.offs, ref.offs)
    assert torch.equal(r.order, ref.order) and torch.equal(r.token_of, ref.token_of) and torch.equal(r.inv, ref.inv)
    n = int(r.num_row_tiles.item())
    assert n == ref.row_tiles.shape[0] and torch.equal(r.row_tiles[:n], ref.row_tiles)
    assert r.host_counts() == ref.counts.tolist()
    r2 = OF.moe_route(logits, k, bias=b, sigmoid=sigmoid, norm=True, scale=1.5)
    assert torch.equal(r2.order, r.order) and torch.equal(r2.topw, r.topw)
    # a choice made elsewhere: only the sort and the tables are produced
    r3 = OF.moe_route(logits, k, tope=ref.tope)
    assert torch.equal(r3.order, ref.order) and torch.equal(r3.counts, ref.counts) and r3.topw is None


def test_grouped_linear_with_device_routing_matches_host_tile_table():
    """The grouped GEMM fed by the device-made tile list (grid sized for an upper bound of the tiles) gives the
    bits of the host-built table, forward and backward; the MoE layer on top of it matches fp32."""
    torch.manual_seed(8)
    T, E, k, K, N = 1500, 16, 4, 256, 384
    logits = torch.randn(T, E, device="cuda")
    logits[:, 3] = -30.0                                    # one expert without tokens
    r = OF.moe_route(logits, k)
    counts = r.host_counts()
    assert counts[3] == 0 and sum(counts) == T * k
    x = torch.randn(T, K, device="cuda").bfloat16()
    w = (torch.randn(E, N, K, device="cuda") / K ** 0.5).bfloat16()
    xs = x.index_select(0, r.token_of)
    xa, wa = xs.clone().requires_grad_(), w.clone().requires_grad_()
    xb, wb = xs.clone().requires_grad_(), w.clone().requires_grad_()
    ya, yb = OF.grouped_linear(xa, wa, r), OF.grouped_linear(xb, wb, counts)
    gy = torch.randn_like(ya)
    ya.backward(gy)
    yb.backward(gy)
    _no_kernel_error()
    assert torch.equal(ya, yb) and torch.equal(xa.grad, xb.grad) and torch.equal(wa.grad, wb.grad)

    from areal_b200.models.config import ModelConfig
    from areal_b200.models.decoder import MoEMLP

    cfg = ModelConfig(hidden_size=256, num_experts=16, num_experts_per_tok=4, moe_intermediate_size=128, norm_topk_prob=True)
    m = MoEMLP(cfg, torch.bfloat16, "cuda")
    for p_ in m.parameters():
        torch.nn.init.normal_(p_, std=0.05)
    xin = torch.randn(700, 256, device="cuda").bfloat16().requires_grad_()
    out = m(xin)
    out.float().pow(2).sum().backward()
    m32 = MoEMLP(cfg, torch.float32, "cpu")                 # the oracle runs on the host in fp32
    m32.load_state_dict({k_: v.float().cpu() for k_, v in m.state_dict().items()})
    x32 = xin.detach().float().cpu().requires_grad_()
    o32 = m32(x32)
    o32.pow(2).sum().backward()
    assert _rel_err(out.cpu(), o32) < 2e-2 and _rel_err(xin.grad.cpu(), x32.grad) < 3e-2
    assert _rel_err(m.w_down.grad.cpu(), m32.w_down.grad) < 3e-2 and _rel_err(m.router.grad.cpu(), m32.router.grad) < 5e-2


@pytest.mark.parametrize("D,Hq,Hkv,page_size,splits", [(128, 32, 8, 64, 4), (128, 8, 1, 16, 3), (128, 12, 2, 64, 1), (64, 4, 2, 16, 4),
                                                       (64, 16, 2, 32, 2)])
def test_paged_decode_attention_matches_fp32(D, Hq, Hkv, page_size, splits):
    """Split-KV paged decode attention (K/V chunks staged in shared memory) against fp32 softmax
    attention over each row's gathered cache; rows of length 0 (idle slots) and 1 included."""
    g = torch.Generator(device="cuda").manual_seed(D + Hq + page_size)
    B, max_len = 9, 700
    lens = torch.randint(2, max_len + 1, (B,), device="cuda", generator=g).int()
    lens[0], lens[1], lens[2] = 0, 1, max_len
    max_pages = (max_len + page_size - 1) // page_size
    n_pages = B * max_pages + 5
    kc = torch.randn(n_pages * page_size, Hkv, D, device="cuda", generator=g).bfloat16()
    vc = torch.randn(n_pages * page_size, Hkv, D, device="cuda", generator=g).bfloat16()
    q = torch.randn(B, Hq, D, device="cuda", generator=g).bfloat16()
    pt = torch.randperm(n_pages, device="cuda", generator=g)[: B * max_pages].int().view(B, max_pages).contiguous()
    po = torch.empty(B * Hq * splits * D, device="cuda")
    pml = torch.empty(B * Hq * splits * 2, device="cuda")
    out = torch.full_like(q, float("nan"))
    rc = oplib.get_lib().ab2_paged_decode(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), pt.data_ptr(), lens.data_ptr(), po.data_ptr(),
                                          pml.data_ptr(), out.data_ptr(), B, Hq, Hkv, D, page_size, max_pages, splits, D ** -0.5,
                                          oplib.stream_ptr())
    assert rc == 0
    torch.cuda.synchronize()
    assert oplib.kernel_error() == 0
    G = Hq // Hkv
    for b in range(B):
        n = int(lens[b])
        if n == 0:
            assert (out[b].float() == 0).all()
            continue
        t = torch.arange(n, device="cuda")
        slots = pt[b, t // page_size].long() * page_size + t % page_size
        k = kc[slots].float().repeat_interleave(G, dim=1)          # [n, Hq, D]
        v = vc[slots].float().repeat_interleave(G, dim=1)
        s = torch.einsum("hd,nhd->hn", q[b].float(), k) * D ** -0.5
        ref = torch.einsum("hn,nhd->hd", torch.softmax(s, -1), v)
        err = ((out[b].float() - ref).norm() / ref.norm()).item()
        assert err < 1e-2, f"row {b} (len {n}): relative error {err}"


@pytest.mark.parametrize("mode", [OF.FP8_ROW, OF.FP8_BLOCK_1x128, OF.FP8_BLOCK_128x128])
@pytest.mark.parametrize("pow2", [False, True])
def test_fp8_quantisation_kernels(mode, pow2):
    """Scales equal the PyTorch statement; de-quantised values are within one e4m3 step."""
    torch.manual_seed(mode)
    x = (torch.randn(300, 576, device="cuda") * torch.rand(300, 1, device="cuda") * 3).bfloat16()
    q, s = OF.quant_fp8(x, mode, pow2)
    qr, sr = OF.quant_fp8_ref(x, mode, pow2)
    assert s.shape == sr.shape and torch.allclose(s, sr, rtol=1e-6, atol=0)
    d, dr = OF.dequant_fp8(q, s, mode), OF.dequant_fp8(qr, sr, mode)
    assert (d - x.float()).abs().max() <= 0.0626 * x.float().abs().max()
    # the kernel multiplies by the reciprocal scale, the statement divides: the two differ by an fp32 ulp, which
    # moves a value across an e4m3 rounding boundary for about one element in a thousand (never by more than one step)
    assert (q.view(torch.uint8) != qr.view(torch.uint8)).float().mean().item() < 5e-3
    assert (d - dr).abs().max() <= 0.0626 * x.float().abs().max()
    assert oplib.kernel_error() == 0


@pytest.mark.parametrize("M,N,K", [(256, 256, 512), (300, 384, 576), (4096, 1024, 2048), (64, 6144, 4096)])
@pytest.mark.parametrize("block", [False, True])
def test_fp8_gemm_matches_fp32_on_the_same_operands(M, N, K, block):
    """tcgen05 kind::f8f6f4 GEMM with row-wise / block-wise scales against an fp32 matmul of the
    de-quantised operands (so only the accumulation order differs)."""
    torch.manual_seed(M + N)
    a = torch.randn(M, K, device="cuda").bfloat16()
    b = (torch.randn(N, K, device="cuda") * 0.05).bfloat16()
    am, bm = (OF.FP8_BLOCK_1x128, OF.FP8_BLOCK_128x128) if block else (OF.FP8_ROW, OF.FP8_ROW)
    aq, sa = OF.quant_fp8(a, am)
    bq, sb = OF.quant_fp8(b, bm)
    ref = OF.dequant_fp8(aq, sa, am) @ OF.dequant_fp8(bq, sb, bm).t()
    for dt, tol in ((torch.float32, 2e-4), (torch.bfloat16, 6e-3)):
        c = OF.gemm_fp8(aq, sa, bq, sb, block, dt)
        torch.cuda.synchronize()
        assert oplib.kernel_error() == 0
        err = ((c.float() - ref).norm() / ref.norm()).item()
        assert err < tol, f"{dt}: relative error {err}"
    # and the quantised product is close to the bf16 one
    full = a.float() @ b.float().t()
    assert ((ref - full).norm() / full.norm()).item() < 0.06


def test_fp8_linear_gradients_close_to_bf16():
    torch.manual_seed(0)
    x = torch.randn(512, 1024, device="cuda").bfloat16().requires_grad_(True)
    w = (torch.randn(768, 1024, device="cuda") * 0.03).bfloat16().requires_grad_(True)
    dy = torch.randn(512, 768, device="cuda").bfloat16()
    y = OF.fp8_linear(x, w)
    y.backward(dy)
    yr = x.detach().float() @ w.detach().float().t()
    assert ((y.float() - yr).norm() / yr.norm()).item() < 0.06
    dxr = dy.float() @ w.detach().float()
    dwr = dy.float().t() @ x.detach().float()
    assert ((x.grad.float() - dxr).norm() / dxr.norm()).item() < 0.06
    assert ((w.grad.float() - dwr).norm() / dwr.norm()).item() < 1e-2


def test_bounded_peer_wait_reports_instead_of_hanging():
    """A flag that nothing sets: the device-side barrier gives up after its (short) limit, records
    the failed wait in the error word and returns; the context stays usable. When the peer's flag
    is there, the same barrier passes."""
    import time

    from areal_b200.parallel.symm import CHANNELS, MAX_PEERS, ptr_array

    L = oplib.get_lib()
    mine = torch.zeros(CHANNELS * MAX_PEERS, dtype=torch.int32, device="cuda")
    absent_peer = torch.zeros(CHANNELS * MAX_PEERS, dtype=torch.int32, device="cuda")    # plays rank 1's pad; nobody runs rank 1
    pads = ptr_array([mine.data_ptr(), absent_peer.data_ptr()])
    assert oplib.kernel_error() == 0
    t0 = time.perf_counter()
    rc = L.ab2_signal_barrier(pads, 0, 2, 0, 1, 50, oplib.stream_ptr())                  # 50 ms limit
    assert rc == 0
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 5.0
    assert oplib.kernel_error() != 0                                                     # the wait that gave up was recorded
    assert oplib.kernel_error() == 0                                                     # ... and reading cleared it
    assert int(absent_peer[0]) == 1                                                      # this rank's own arrival was published
    assert float((torch.ones(8, device="cuda") * 2).sum()) == 16.0                       # the context still works
    mine[1] = 2                                                                           # "rank 1" arrived for epoch 2
    rc = L.ab2_signal_barrier(pads, 0, 2, 0, 2, 50, oplib.stream_ptr())
    torch.cuda.synchronize()
    assert rc == 0 and oplib.kernel_error() == 0 and int(absent_peer[0]) == 2


@pytest.mark.parametrize("M,N,K", [(64, 6144, 4096), (64, 4096, 12288), (7, 4096, 4096), (128, 2048, 1024), (64, 24576, 4096)])
@pytest.mark.parametrize("with_resid", [False, True])
def test_decode_splitk_gemm_matches_fp32(M, N, K, with_resid):
    """Decode-shaped product with K split over CTAs (fp32 pieces + reduce kernel) against an fp32 matmul."""
    torch.manual_seed(M + N)
    x = torch.randn(M, K, device="cuda").bfloat16()
    w = (torch.randn(N, K, device="cuda") * 0.05).bfloat16()
    r = torch.randn(M, N, device="cuda").bfloat16() if with_resid else None
    y = OF.gemm_decode(x, w, r)
    torch.cuda.synchronize()
    assert oplib.kernel_error() == 0
    ref = x.float() @ w.float().t() + (r.float() if with_resid else 0)
    assert ((y.float() - ref).norm() / ref.norm()).item() < 4e-3
    y2 = OF.gemm_decode(x, w, r)                                    # the workspace is reusable without clearing
    assert torch.equal(y, y2)


# --------------------------------------------------------------------------- RL losses
@pytest.mark.parametrize("rs", [None, ("mask", "ratio", None, 5.0), ("clamp", "ratio", 0.5, 2.0), ("mask", "kl_k3", None, 0.05),
                                ("mask", "binary_kl", None, 0.02), ("mask", "kl_k2", None, 0.02)])
@pytest.mark.parametrize("c_clip,hi", [(None, None), (3.0, 0.28)])
def test_fused_ppo_token_loss_matches_eager_statement(rs, c_clip, hi):
    """Loss value, gradient with respect to the new log-probs and every logged per-token statistic
    of the one-kernel loss against the eager PyTorch statement of the same math (fp32)."""
    from areal_b200.algo import functional as AF
    from areal_b200.api.cli_args import RejectionSamplingConfig

    torch.manual_seed(3)
    n = 5000
    old = (-torch.rand(n, device="cuda") * 6).requires_grad_(False)
    prox = old + 0.3 * torch.randn(n, device="cuda")
    logp0 = prox + 0.25 * torch.randn(n, device="cuda")
    adv = torch.randn(n, device="cuda")
    adv[::7] = 0.0
    mask = torch.rand(n, device="cuda") < 0.8
    cfg = None
    if rs is not None:
        cfg = RejectionSamplingConfig(level="token", action=rs[0], metric=rs[1], lower=rs[2], upper=rs[3])
    outs = []
    for fused in (False, True):
        AF._FUSED_LOSS = fused
        lp = logp0.clone().requires_grad_(True)
        loss, stat = AF.ppo_actor_loss_fn(lp, prox, old, adv, 0.2, mask, hi, c_clip, cfg, "token", None)
        loss.backward()
        outs.append((loss.detach(), lp.grad.clone(), stat))
    AF._FUSED_LOSS = True
    (l0, g0, s0), (l1, g1, s1) = outs
    assert torch.allclose(l0, l1, rtol=1e-5, atol=1e-7), (float(l0), float(l1))
    assert torch.allclose(g0, g1, rtol=1e-4, atol=1e-9)
    assert torch.equal(s0["clip_mask"], s1["clip_mask"]) and torch.equal(s0["dual_clip_mask"], s1["dual_clip_mask"])
    assert torch.allclose(s0["importance_weight"], s1["importance_weight"], rtol=1e-5)
    assert torch.allclose(torch.where(mask, s0["loss"], torch.zeros_like(s0["loss"])), torch.where(mask, s1["loss"], torch.zeros_like(s1["loss"])),
                          rtol=1e-4, atol=1e-7)
    if rs is not None:
        assert torch.equal(s0["behave_mask"], s1["behave_mask"])
        assert torch.allclose(s0["behave_imp_weight"], s1["behave_imp_weight"], rtol=1e-5)
        assert abs(float(s0["filtered_fraction"]) - float(s1["filtered_fraction"])) < 1e-6
    assert float(s1["n_valid_tokens"]) == float(mask.sum())


@pytest.mark.parametrize("lam", [0.95, "per_sequence"])
def test_gae_scan_kernel_matches_the_loop(lam):
    from areal_b200.algo.advantages import token_level_gae

    torch.manual_seed(4)
    B, L = 37, 301
    rewards = torch.randn(B, L, device="cuda") * 0.1
    values = torch.randn(B, L, device="cuda")
    lm = (torch.rand(B, L, device="cuda") < 0.7).int()
    lm[:, :20] = 0
    no_eos = torch.rand(B, device="cuda") < 0.3
    gl = 0.95 if lam == 0.95 else torch.rand(B, device="cuda") * 0.2 + 0.8
    want_adv, want_ret = token_level_gae(rewards.cpu(), values.cpu(), lm.cpu(), no_eos.cpu(), 0.99, gl if lam == 0.95 else gl.cpu())
    adv, ret = OF.gae_scan(rewards, values, lm, no_eos, 0.99, gl)
    assert torch.allclose(adv.cpu(), want_adv, rtol=1e-4, atol=1e-5)
    assert torch.allclose(ret.cpu(), want_ret, rtol=1e-4, atol=1e-5)
    got_adv, _ = token_level_gae(rewards, values, lm, no_eos, 0.99, gl)      # CUDA inputs take the kernel
    assert torch.allclose(got_adv, adv)


@pytest.mark.parametrize("M,N,K", [(1024, 512, 256), (2048, 1024, 512), (1096, 776, 328), (4096, 4096, 1024)])
@pytest.mark.parametrize("layout", ["nt", "nn", "tn", "tt"])
def test_gemm_2sm_pair_kernel_matches_fp32(M, N, K, layout):
    """256 x 256 tiles on CTA pairs (tcgen05 cta_group::2): all operand layouts, ragged edges, every
    epilogue, against fp32 matmul; and bit-identical to the one-CTA kernel (same accumulation order)."""
    torch.manual_seed(M + N + K)
    A = torch.randn(M, K, device="cuda").bfloat16()
    B = (torch.randn(N, K, device="cuda") * 0.05).bfloat16()
    a_mn, b_mn = layout[0] == "t", layout[1] == "n"
    Aop = A.t().contiguous() if a_mn else A
    Bop = B.t().contiguous() if b_mn else B
    ref = A.float() @ B.float().t()
    old = OF.GEMM_2SM
    try:
        OF.GEMM_2SM = False
        base = OF.gemm(Aop, Bop, a_mn=a_mn, b_mn=b_mn)
        OF.GEMM_2SM = True
        out = OF.gemm(Aop, Bop, a_mn=a_mn, b_mn=b_mn)
        assert oplib.kernel_error() == 0
        assert _rel_err(out, ref) < 4e-3
        assert torch.equal(out, base)
        acc = torch.ones(M, N, device="cuda")
        OF.gemm(Aop, Bop, a_mn=a_mn, b_mn=b_mn, out=acc, epi=OF.EPI_F32_ACC)
        assert _rel_err(acc, ref + 1.0) < 1e-4
        resid = torch.randn(M, N, device="cuda").bfloat16()
        y = OF.gemm(Aop, Bop, a_mn=a_mn, b_mn=b_mn, epi=OF.EPI_BF16_RESID, resid=resid)
        assert _rel_err(y, ref + resid.float()) < 4e-3
        assert oplib.kernel_error() == 0
    finally:
        OF.GEMM_2SM = old


@pytest.mark.parametrize("cp,D,Hq,Hkv", [(2, 128, 8, 2), (4, 64, 4, 4)])
def test_context_parallel_blockwise_attention_on_flash_kernels(cp, D, Hq, Hkv):
    """Zig-zag context parallelism with emulated ranks on one device: every rank's chunk-pair calls of the flash
    kernels, merged through their log-sum-exp, give causal attention over the whole sequences; the per-rank
    gradient contributions add up to the gradients of the unsplit attention."""
    from areal_b200.parallel import cp as CP

    torch.manual_seed(cp + D)
    lens = [700, 1130, 64, 333]
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    T = int(cu[-1])
    q = torch.randn(T, Hq, D, device="cuda").bfloat16()
    k = torch.randn(T, Hkv, D, device="cuda").bfloat16()
    v = torch.randn(T, Hkv, D, device="cuda").bfloat16()
    do = torch.randn(T, Hq, D, device="cuda").bfloat16()
    scale = D ** -0.5
    o_ref, lse_ref = OF.attention_ref(q, k, v, cu.cuda(), True, scale)
    dq_ref, dk_ref, dv_ref = OF.attention_bwd_ref(q, k, v, o_ref, lse_ref, do, cu.cuda(), True, scale)
    parts = [[CP.zigzag_split(t, cu, cp, r) for r in range(cp)] for t in (q, k, v, do)]
    k_all, v_all = torch.stack(parts[1]), torch.stack(parts[2])
    dk_sum, dv_sum = torch.zeros_like(k_all, dtype=torch.float32), torch.zeros_like(v_all, dtype=torch.float32)
    for r in range(cp):
        src, _, local_lens = CP.zigzag_indices(cu, cp, r)
        valid = (src >= 0).cuda()
        o, lse = CP.cp_block_forward(parts[0][r], k_all, v_all, local_lens, r, scale)
        want = CP.zigzag_split(o_ref, cu, cp, r)
        assert _rel_err(o[valid], want[valid]) < 1e-2
        dq, dk_c, dv_c = CP.cp_block_backward(parts[0][r], k_all, v_all, o, lse, parts[3][r], local_lens, r, scale)
        assert _rel_err(dq[valid], CP.zigzag_split(dq_ref, cu, cp, r)[valid]) < 2e-2
        dk_sum += dk_c
        dv_sum += dv_c
    _no_kernel_error()
    for r in range(cp):
        src, _, _ = CP.zigzag_indices(cu, cp, r)
        valid = (src >= 0).cuda()
        assert _rel_err(dk_sum[r][valid], CP.zigzag_split(dk_ref, cu, cp, r)[valid]) < 2e-2
        assert _rel_err(dv_sum[r][valid], CP.zigzag_split(dv_ref, cu, cp, r)[valid]) < 2e-2


def test_embedding_reports_an_out_of_range_token_id():
    """A token id outside the vocabulary is clamped (no stray read) and sets the device error word with the bounds
    code, which the engines turn into an exception at their next poll; in-range ids leave the word alone."""
    W = torch.randn(100, 64, device="cuda").bfloat16()
    ok = OF.embedding(torch.tensor([0, 5, 99], device="cuda", dtype=torch.int32), W)
    torch.cuda.synchronize()
    assert oplib.kernel_error() == 0 and torch.equal(ok, W[[0, 5, 99]])
    bad = OF.embedding(torch.tensor([3, 100, -1], device="cuda", dtype=torch.int32), W)
    torch.cuda.synchronize()
    assert oplib.kernel_error() == 6                              # ERR_BOUNDS; reading clears the word
    assert torch.equal(bad, W[[3, 99, 0]]) and oplib.kernel_error() == 0


def test_forward_and_decode_are_bitwise_reproducible_and_training_is_close():
    """Run-twice check: the forward pass (log-probs of a packed batch) and greedy decoding give the same bits when
    repeated; a training step uses float atomics (attention dQ, embedding rows), so two runs from one state agree to
    rounding, not to the bit."""
    from areal_b200.models.config import preset
    from areal_b200.models.decoder import build_model

    cfg = preset("tiny-qwen3")
    model = build_model(cfg, dtype=torch.bfloat16, device="cuda", seed=3)
    ids = torch.randint(0, cfg.vocab_size, (900,), device="cuda", dtype=torch.int32)
    cu = torch.tensor([0, 300, 420, 900], dtype=torch.int32, device="cuda")
    labels = torch.roll(ids, -1).long()
    outs = []
    for _ in range(2):
        with torch.no_grad():
            h = model(ids, cu, max_seqlen=480)
            outs.append(model.logprobs_entropy(h, labels))
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
    grads = []
    for _ in range(2):
        model.zero_grad()
        h = model(ids, cu, max_seqlen=480)
        lp, _ = model.logprobs_entropy(h, labels)
        (-lp.mean()).backward()
        grads.append(torch.cat([p.grad.float().flatten() for p in model.parameters() if p.grad is not None]))
    assert _rel_err(grads[0], grads[1]) < 1e-3
    _no_kernel_error()
