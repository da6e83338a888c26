"""The fused compute + communication kernels on ONE GPU with emulated ranks: every "peer" buffer
is a tensor of the same device and the ranks' kernels are launched one after another on one
stream. That is a valid schedule for these kernels because none of them waits for another
launch: the gathers copy and consume inside one kernel, the scatters / reductions / pushes only
store, and the tensor-parallel partial-sum exchange is driven with all producers first and the
consumers after them. Each result is compared with plain fp32 PyTorch on the gathered operands.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from areal_b200.ops import lib as oplib
    from areal_b200.parallel import fused_zero, symm, tp_fused  # noqa: F401  (declare the symbols)

    return oplib.get_lib(), oplib


def _ptrs(tensors):
    from areal_b200.parallel.symm import ptr_array

    return ptr_array([t.data_ptr() for t in tensors])


def _rel(a, b):
    return float((a.float() - b.float()).norm() / b.float().norm().clamp(min=1e-12))


def _rand(*shape, seed=0, scale=1.0, dtype=torch.bfloat16):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, generator=g, device="cuda") * scale).to(dtype)


@pytest.mark.parametrize("P,copy_once", [(2, True), (4, True), (2, False)])
def test_allgather_gemm_emulated(P, copy_once):
    """y_r = concat_ranks(x) @ w_r^T for every emulated rank r (column-parallel product)."""
    L, oplib = _lib()
    rows, K, N = 256, 512, 384
    xs = [_rand(rows, K, seed=10 + r) for r in range(P)]
    ws = [_rand(N, K, seed=20 + r, scale=0.05) for r in range(P)]
    full = torch.cat(xs).float()
    for r in range(P):
        y = torch.empty(rows * P, N, dtype=torch.bfloat16, device="cuda")
        gathered = torch.empty(rows * P * K, dtype=torch.bfloat16, device="cuda")
        flags = torch.zeros(rows * P // 128 + 1, dtype=torch.int32, device="cuda")
        rc = L.ab2_allgather_gemm(_ptrs(xs), ws[r].data_ptr(), y.data_ptr(), rows * P, N, K, K, K, N, 0, r, P,
                                  gathered.data_ptr() if copy_once else None, flags.data_ptr() if copy_once else None, 1,
                                  oplib.stream_ptr())
        assert rc == 0
        assert _rel(y, full @ ws[r].float().t()) < 1e-2, (P, r)
    assert oplib.kernel_error() == 0


@pytest.mark.parametrize("P,half", [(2, False), (4, False), (2, True)])
def test_gemm_reduce_scatter_emulated(P, half):
    """out_r = rows r of sum_ranks(x_q @ w_q^T): every rank's epilogue adds into the owners' buffers."""
    L, oplib = _lib()
    rows, Kl, N = 128, 256, 512
    M = rows * P
    xs = [_rand(M, Kl, seed=30 + r) for r in range(P)]
    ws = [_rand(N, Kl, seed=40 + r, scale=0.05) for r in range(P)]
    outs = [torch.zeros(rows, N, dtype=torch.bfloat16 if half else torch.float32, device="cuda") for _ in range(P)]
    for r in range(P):
        rc = L.ab2_gemm_reduce_scatter(xs[r].data_ptr(), ws[r].data_ptr(), _ptrs(outs), M, N, Kl, Kl, Kl, N, 0, r, P, int(half),
                                       oplib.stream_ptr())
        assert rc == 0
    want = sum(x.float() @ w.float().t() for x, w in zip(xs, ws))
    for r in range(P):
        assert _rel(outs[r], want[r * rows:(r + 1) * rows]) < (3e-2 if half else 1e-2), (P, r)
    assert oplib.kernel_error() == 0


@pytest.mark.parametrize("P", [2, 4])
def test_ulysses_projection_exchanges_emulated(P):
    """QKV projection + seq->heads (columns scattered to their owners from the epilogue) and
    heads->seq + output projection (copy CTAs pull this rank's rows of every panel)."""
    L, oplib = _lib()
    M, K, N = 256, 512, 128 * P                     # M rows per rank, N output columns over P ranks
    xs = [_rand(M, K, seed=50 + r) for r in range(P)]
    w = _rand(N, K, seed=60, scale=0.05)
    bufs = [torch.zeros(P * M, N // P, dtype=torch.bfloat16, device="cuda") for _ in range(P)]
    for r in range(P):
        rc = L.ab2_gemm_scatter_cols(xs[r].data_ptr(), w.data_ptr(), _ptrs(bufs), M, N, K, K, K, N // P, 0, r, P, oplib.stream_ptr())
        assert rc == 0
    full = torch.cat(xs).float() @ w.float().t()                          # [P*M, N]
    for r in range(P):
        assert _rel(bufs[r], full[:, r * (N // P):(r + 1) * (N // P)]) < 1e-2, ("scatter", P, r)
    # heads -> seq: rank r owns columns r of a [P*M, Kt] matrix; every rank wants its M rows of all columns
    Kt, N2 = 64 * P * 2, 384
    panels = [_rand(P * M, Kt // P, seed=70 + r) for r in range(P)]
    w2 = _rand(N2, Kt, seed=80, scale=0.05)
    a_full = torch.cat(panels, dim=1).float()                              # [P*M, Kt]
    for r in range(P):
        y = torch.empty(M, N2, dtype=torch.bfloat16, device="cuda")
        gathered = torch.empty(M * Kt, dtype=torch.bfloat16, device="cuda")
        flags = torch.zeros((M // 128 + 1) * P, dtype=torch.int32, device="cuda")
        rc = L.ab2_gather_cols_gemm(_ptrs(panels), w2.data_ptr(), y.data_ptr(), M, N2, Kt, Kt // P, Kt, N2, 0, r, P,
                                    gathered.data_ptr(), flags.data_ptr(), 1, oplib.stream_ptr())
        assert rc == 0
        assert _rel(y, a_full[r * M:(r + 1) * M] @ w2.float().t()) < 1e-2, ("gather", P, r)
    assert oplib.kernel_error() == 0


@pytest.mark.parametrize("P", [2, 4])
def test_reduce_scatter_sumsq_and_adamw_push_emulated(P):
    """Gradient reduce-scatter by peer loads with the squared-norm partial, then the sharded AdamW
    whose bf16 result lands in every destination buffer, against torch.optim.AdamW in fp32."""
    L, oplib = _lib()
    n_shard = 4096 * 3
    n = n_shard * P
    grads = [_rand(n, seed=90 + r, dtype=torch.float32) for r in range(P)]
    p0 = _rand(n, seed=99, dtype=torch.float32)
    want_g = sum(grads)
    lr, b1, b2, eps, wd = 1e-2, 0.9, 0.95, 1e-8, 0.1
    ref = torch.nn.Parameter(p0.clone())
    opt = torch.optim.AdamW([ref], lr=lr, betas=(b1, b2), eps=eps, weight_decay=wd)
    ref.grad = want_g.clone()
    opt.step()
    dst = [torch.zeros(n, dtype=torch.bfloat16, device="cuda") for _ in range(P + 1)]     # P trainers + one rollout replica
    total_sq = 0.0
    for r in range(P):
        lo = r * n_shard
        out = torch.empty(n_shard, dtype=torch.float32, device="cuda")
        state = torch.zeros(4, dtype=torch.float32, device="cuda")
        assert L.ab2_rs_sumsq(_ptrs(grads), P, lo, n_shard, out.data_ptr(), state.data_ptr(), ctypes.c_float(1.0), oplib.stream_ptr()) == 0
        assert torch.allclose(out, want_g[lo:lo + n_shard], rtol=1e-6, atol=1e-6)
        total_sq += float(state[0])
        state[1], state[2] = 1.0, 1.0                                      # clip coefficient 1, step allowed
        master, m, v = p0[lo:lo + n_shard].clone(), torch.zeros(n_shard, device="cuda"), torch.zeros(n_shard, device="cuda")
        rc = L.ab2_adamw_push(master.data_ptr(), m.data_ptr(), v.data_ptr(), out.data_ptr(), _ptrs(dst), len(dst), lo, state.data_ptr(),
                              n_shard, ctypes.c_float(lr), ctypes.c_float(b1), ctypes.c_float(b2), ctypes.c_float(eps), ctypes.c_float(wd), 1,
                              oplib.stream_ptr())
        assert rc == 0
        assert torch.allclose(master, ref.data[lo:lo + n_shard], rtol=1e-5, atol=1e-6), r
    assert abs(total_sq - float(want_g.double().pow(2).sum())) / total_sq < 1e-4
    for d in dst:
        assert torch.equal(d, dst[0])                                       # every destination received the same bits
    # master weights agree to 1e-5; a value on a bf16 rounding boundary may land on either side
    assert (dst[0] != ref.data.to(torch.bfloat16)).float().mean().item() < 1e-3
    assert torch.allclose(dst[0].float(), ref.data, rtol=1e-2, atol=1e-3)


@pytest.mark.parametrize("tp,n_rep", [(2, 1), (2, 2), (4, 1)])
def test_push_plan_reshards_every_tp_slice_emulated(tp, n_rep):
    """The whole FSDP-shard -> tensor-parallel re-shard plan in one launch per trainer shard: every
    TP rank of every replica ends up with exactly ``TP.shard_tensor`` of every parameter."""
    from areal_b200.engine.flat_params import FlatParamStore
    from areal_b200.models.config import preset
    from areal_b200.models.decoder import build_model
    from areal_b200.parallel import tp as TP
    from areal_b200.parallel.weight_push import TPPushPlan

    cfg = preset("tiny-qwen3", num_heads=4, num_kv_heads=4, intermediate_size=256)
    world = 3                                                                 # trainer shards
    model = build_model(cfg, dtype=torch.bfloat16, device="cuda", seed=3)
    stores = [FlatParamStore(model if r == 0 else build_model(cfg, dtype=torch.bfloat16, device="cuda", seed=3), world, r, with_grads=False)
              for r in range(world)]
    local_cfg = TP.local_config(cfg, tp)
    dst_models = [[build_model(local_cfg, dtype=torch.bfloat16, device="cuda", seed=100 + k * tp + j) for j in range(tp)] for k in range(n_rep)]
    dst_stores = [[FlatParamStore(m, 1, 0, with_grads=False) for m in row] for row in dst_models]
    dst_ptrs = [s.flat_param.data_ptr() for row in dst_stores for s in row]
    for r in range(world):
        plan = TPPushPlan.build(cfg, stores[r], tp, [dict(zip(s.names, s.offsets)) for s in dst_stores[0]], device="cuda")
        plan.run(stores[r].flat_param, dst_ptrs, n_rep)
    torch.cuda.synchronize()
    full = dict(stores[0].named_views())
    for k in range(n_rep):
        for j in range(tp):
            for name, p in dst_models[k][j].named_parameters():
                assert torch.equal(p.data, TP.shard_tensor(cfg, name, full[name].data, tp, j)), (k, j, name)


def test_push_plan_fp8_block_cast_emulated():
    """The same plan with the in-kernel 1 x 128 block-scaled e4m3 cast: values and scales equal the
    quantisation of the re-sharded bf16 tensors."""
    from areal_b200.ops import functional as OF
    from areal_b200.parallel.weight_push import CopyOp, TPPushPlan

    rows, cols = 96, 512
    src = _rand(rows * cols + 256, seed=7)
    ops = [CopyOp(src_off=256, dst_tp=0, dst_off=0, rows=rows, cols=256, ld_src=cols, ld_dst=256),
           CopyOp(src_off=256 + 256, dst_tp=1, dst_off=0, rows=rows, cols=256, ld_src=cols, ld_dst=256)]
    plan = TPPushPlan(ops, tp=2, device="cuda")
    q = [torch.zeros(rows * 256, dtype=torch.uint8, device="cuda") for _ in range(2)]
    s = [torch.zeros(rows * 256 // 128, dtype=torch.float32, device="cuda") for _ in range(2)]
    plan.run(src, [t.data_ptr() for t in q], 1, scale_ptrs=[t.data_ptr() for t in s], pow2=False)
    torch.cuda.synchronize()
    mat = src[256:256 + rows * cols].view(rows, cols)
    for j in range(2):
        want_q, want_s = OF.quant_fp8_ref(mat[:, j * 256:(j + 1) * 256].contiguous(), OF.FP8_BLOCK_1x128)   # scales [kb, rows]
        assert torch.allclose(s[j].view(rows, 2), want_s.t().contiguous(), rtol=1e-6)     # here: one scale per 128 elements, row-major
        got = q[j].view(rows, 256)
        # multiply-by-reciprocal against divide: an fp32 ulp moves about one value in a thousand over an e4m3 boundary
        assert (got != want_q.view(torch.uint8).view(rows, 256)).float().mean().item() < 5e-3
        deq = got.view(torch.float8_e4m3fn).float() * s[j].view(rows, 2).repeat_interleave(128, dim=1)
        assert (deq - mat[:, j * 256:(j + 1) * 256].float()).abs().max() <= 0.0626 * mat.float().abs().max()


@pytest.mark.parametrize("P", [2, 4])
def test_tp_partial_sum_exchange_emulated(P):
    """Row-parallel product handed to every rank from the GEMM epilogue, then sum over ranks +
    residual + RMSNorm in one kernel; several rounds so both buffer sets and the growing counters
    are exercised. Producers of all ranks run before any consumer (one GPU)."""
    from areal_b200.ops import lib as oplib
    from areal_b200.parallel.tp_decode import TPDecodeExchange

    H, Kl, max_rows = 512, 256, 256
    exs = TPDecodeExchange.emulated(P, "cuda", H, max_rows)
    wn = _rand(H, seed=5).abs() + 0.5
    for rnd, M in enumerate([64, 200, 1, 256, 64]):
        xs = [_rand(M, Kl, seed=100 + 10 * rnd + r) for r in range(P)]
        ws = [_rand(H, Kl, seed=200 + 10 * rnd + r, scale=0.05) for r in range(P)]
        resid = _rand(M, H, seed=300 + rnd)
        pend = [exs[r].linear_bcast(xs[r], ws[r]) for r in range(P)]
        outs = [exs[r].reduce_rmsnorm(pend[r], wn, 1e-6, resid) for r in range(P)]
        parts = [(x.float() @ w.float().t()).to(torch.bfloat16).float() for x, w in zip(xs, ws)]
        tot = (sum(parts).to(torch.bfloat16).float() + resid.float()).to(torch.bfloat16).float()
        want = tot * torch.rsqrt(tot.pow(2).mean(-1, keepdim=True) + 1e-6) * wn.float()
        for r in range(P):
            x, new_resid = outs[r]
            assert _rel(new_resid, tot) < 1e-2 and _rel(x, want) < 1e-2, (P, rnd, r)
            assert torch.equal(x, outs[0][0]) and torch.equal(new_resid, outs[0][1])      # every rank holds the same bits
    assert oplib.kernel_error() == 0


def test_tp_partial_sum_consumer_gives_up_when_a_peer_never_produces():
    """A consumer whose peer never produced returns after its (short) limit with the error word
    set; the context stays usable and the next complete round is correct again."""
    from areal_b200.ops import lib as oplib
    from areal_b200.parallel.tp_decode import TPDecodeExchange

    H, Kl, M = 256, 128, 32
    exs = TPDecodeExchange.emulated(2, "cuda", H, 64, timeout_ms=50)
    wn = torch.ones(H, dtype=torch.bfloat16, device="cuda")
    x, w = _rand(M, Kl, seed=1), _rand(H, Kl, seed=2, scale=0.05)
    resid = _rand(M, H, seed=3)
    p0 = exs[0].linear_bcast(x, w)                     # rank 1 stays silent
    exs[0].reduce_rmsnorm(p0, wn, 1e-6, resid)
    assert oplib.kernel_error() == 5                   # ERR_WAIT_PEER_FLAG, recorded not trapped
    assert oplib.kernel_error() == 0                   # cleared by the read
    exs[1]._calls += 1                                 # rank 1 skipped that product entirely
    exs[1].counters.copy_(exs[0].counters)             # and both ranks agree on what has been counted
    exs[1].state.copy_(exs[0].state)
    pend = [exs[r].linear_bcast(x, w) for r in range(2)]
    outs = [exs[r].reduce_rmsnorm(pend[r], wn, 1e-6, resid) for r in range(2)]
    part = (x.float() @ w.float().t()).to(torch.bfloat16).float()
    tot = ((2 * part).to(torch.bfloat16).float() + resid.float()).to(torch.bfloat16).float()
    assert oplib.kernel_error() == 0
    assert _rel(outs[0][1], tot) < 1e-2 and torch.equal(outs[0][1], outs[1][1])
