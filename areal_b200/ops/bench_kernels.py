"""Micro-benchmarks of the individual sm_100a kernels (CUDA-event timing, L2 flushed between
iterations) with achieved throughput and the fraction of the measured device peaks.

    python -m areal_b200.ops.bench_kernels gemm --m 8192 --n 8192 --k 8192
    python -m areal_b200.ops.bench_kernels attn_fwd --seqlen 4096 --batch 4
    python -m areal_b200.ops.bench_kernels attn_bwd --seqlen 4096 --batch 4
    python -m areal_b200.ops.bench_kernels decode --batch 128 --ctx 1024
    python -m areal_b200.ops.bench_kernels rmsnorm | swiglu | adamw | logprob

The same entry points are what the profiler summaries under ``profiles/`` were captured from
(small cases: one kernel, a few launches).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

from . import functional as OF
from . import lib as oplib

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def peaks() -> dict:
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


_flush_buf = None


def flush_l2():
    global _flush_buf
    if _flush_buf is None:
        _flush_buf = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")  # > 126 MB L2
    _flush_buf.zero_()


def timeit(fn, iters: int = 10, warmup: int = 3, flush: bool = True) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        if flush:
            flush_l2()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        total += a.elapsed_time(b)
    return total / iters


def report(name: str, ms: float, flops: float = 0.0, bytes_: float = 0.0, **extra) -> dict:
    pk = peaks()
    out = {"kernel": name, "ms": round(ms, 4), **extra}
    if flops:
        out["tflops"] = round(flops / ms / 1e9, 1)
        out[f"frac_of_{pk['source']}_bf16_peak"] = round(flops / ms / 1e9 / pk["bf16_tflops"], 3)
    if bytes_:
        out["gbs"] = round(bytes_ / ms / 1e6, 1)
        out[f"frac_of_{pk['source']}_hbm_peak"] = round(bytes_ / ms / 1e6 / pk["hbm_gbs"], 3)
    out["kernel_error"] = oplib.kernel_error()
    print(json.dumps(out), flush=True)
    return out


def bench_gemm(a):
    A = torch.randn(a.m, a.k, device="cuda").bfloat16()
    B = torch.randn(a.n, a.k, device="cuda").bfloat16()
    a_mn, b_mn = a.layout[0] == "t", a.layout[1] == "n"
    Aop = A.t().contiguous() if a_mn else A
    Bop = B.t().contiguous() if b_mn else B
    C = torch.empty(a.m, a.n, device="cuda", dtype=torch.float32 if a.epi in (1, 2) else torch.bfloat16)
    if a.epi == 2:
        C.zero_()
    old = OF.GEMM_2SM
    OF.GEMM_2SM = False                   # first row: the one-CTA kernel
    try:
        ms = timeit(lambda: OF.gemm(Aop, Bop, a_mn=a_mn, b_mn=b_mn, out=C, epi=a.epi, bn=a.bn), a.iters, a.warmup)
    finally:
        OF.GEMM_2SM = old
    fl = 2.0 * a.m * a.n * a.k
    by = 2.0 * (a.m * a.k + a.n * a.k) + C.element_size() * a.m * a.n
    res = report("gemm_bf16_tcgen05", ms, fl, by, m=a.m, n=a.n, k=a.k, layout=a.layout, epi=a.epi)
    if a.bn == 0:
        old = OF.GEMM_2SM
        OF.GEMM_2SM = True
        try:
            ms3 = timeit(lambda: OF.gemm(Aop, Bop, a_mn=a_mn, b_mn=b_mn, out=C, epi=a.epi), a.iters, a.warmup)
            report("gemm_bf16_tcgen05_2sm (cta_group::2, 256x256 per CTA pair)", ms3, fl, by, m=a.m, n=a.n, k=a.k, layout=a.layout, epi=a.epi)
        finally:
            OF.GEMM_2SM = old
    if a.compare:
        ref = torch.empty(a.m, a.n, device="cuda", dtype=torch.bfloat16)
        ms2 = timeit(lambda: torch.matmul(A, B.t(), out=ref), a.iters, a.warmup)
        report("cublas_bf16 (library baseline)", ms2, fl, by)
    return res


def bench_gemm_decode(a):
    """Decode-shaped ``x @ W^T``: split-K kernel pair against the general kernel (``--compare``)."""
    x = torch.randn(a.m, a.k, device="cuda").bfloat16()
    w = (torch.randn(a.n, a.k, device="cuda") * 0.05).bfloat16()
    bn, splits = OF.decode_gemm_plan(a.m, a.n, a.k)
    ms = timeit(lambda: OF.gemm_decode(x, w), a.iters, a.warmup)
    res = report("gemm_decode_splitk", ms, 2.0 * a.m * a.n * a.k, 2.0 * (a.n * a.k + a.m * a.k + a.m * a.n), m=a.m, n=a.n, k=a.k, bn=bn, splits=splits)
    if a.compare:
        ms_g = timeit(lambda: OF.gemm(x, w), a.iters, a.warmup)
        report("gemm_bf16_tcgen05 (same shape)", ms_g, 2.0 * a.m * a.n * a.k, 2.0 * (a.n * a.k + a.m * a.k + a.m * a.n), m=a.m, n=a.n, k=a.k)
    return res


def bench_gemm_fp8(a):
    """e4m3 GEMM (``--split 1``: block-wise scales, 0: row-wise), operands quantised once outside the timed region."""
    block = bool(a.split)
    x = torch.randn(a.m, a.k, device="cuda").bfloat16()
    w = (torch.randn(a.n, a.k, device="cuda") * 0.05).bfloat16()
    am, bm = (OF.FP8_BLOCK_1x128, OF.FP8_BLOCK_128x128) if block else (OF.FP8_ROW, OF.FP8_ROW)
    xq, xs = OF.quant_fp8(x, am)
    wq, ws = OF.quant_fp8(w, bm)
    ms = timeit(lambda: OF.gemm_fp8(xq, xs, wq, ws, block), a.iters, a.warmup)
    res = report("gemm_fp8_tcgen05" + ("_blockscaled" if block else "_rowscaled"), ms, 2.0 * a.m * a.n * a.k,
                 1.0 * (a.m * a.k + a.n * a.k) + 2.0 * a.m * a.n, m=a.m, n=a.n, k=a.k)
    if a.compare:
        ms_q = timeit(lambda: OF.quant_fp8(x, am), a.iters, a.warmup)
        report("quant_fp8" + ("_1x128" if block else "_row"), ms_q, 0.0, 3.0 * a.m * a.k, m=a.m, k=a.k)
    return res


def bench_gemm_skinny(a):
    """Decode-shaped product: --m tokens (<= 256) against an [--n, --k] weight; --split 0 = automatic."""
    x = torch.randn(a.m, a.k, device="cuda").bfloat16()
    w = torch.randn(a.n, a.k, device="cuda").bfloat16()
    fl = 2.0 * a.m * a.n * a.k
    by = 2.0 * (a.m * a.k + a.n * a.k + a.m * a.n)
    ms = timeit(lambda: OF.gemm_skinny(x, w, split_k=a.split), a.iters, a.warmup)
    res = report("gemm_skinny_tcgen05", ms, fl, by, m=a.m, n=a.n, k=a.k, split=a.split)
    if a.compare:
        out = torch.empty(a.m, a.n, device="cuda", dtype=torch.bfloat16)
        ms1 = timeit(lambda: OF.gemm(x, w, out=out), a.iters, a.warmup)
        report("gemm_bf16_tcgen05 (general kernel)", ms1, fl, by)
        ms2 = timeit(lambda: torch.matmul(x, w.t(), out=out), a.iters, a.warmup)
        report("cublas_bf16 (library baseline)", ms2, fl, by)
    return res


def _attn_inputs(a):
    T = a.seqlen * a.batch
    q = torch.randn(T, a.heads, a.dim, device="cuda").bfloat16()
    k = torch.randn(T, a.kv_heads, a.dim, device="cuda").bfloat16()
    v = torch.randn(T, a.kv_heads, a.dim, device="cuda").bfloat16()
    cu = torch.arange(0, T + 1, a.seqlen, device="cuda", dtype=torch.int32)
    return q, k, v, cu, OF.attn_tile_table(cu, T)


def bench_attn_fwd(a):
    q, k, v, cu, ti = _attn_inputs(a)
    ms = timeit(lambda: OF.attention_fwd(q, k, v, cu, True, None, ti), a.iters, a.warmup)
    fl = 4.0 * a.batch * a.heads * a.seqlen * a.seqlen * a.dim / 2
    return report("attn_fwd_tcgen05", ms, fl, seqlen=a.seqlen, batch=a.batch, heads=a.heads, kv_heads=a.kv_heads)


def bench_attn_bwd(a):
    q, k, v, cu, ti = _attn_inputs(a)
    o, lse = OF.attention_fwd(q, k, v, cu, True, None, ti)
    do = torch.randn_like(o)
    ms = timeit(lambda: OF.attention_bwd(q, k, v, o, lse, do, cu, True, a.dim ** -0.5, ti), a.iters, a.warmup)
    fl = 2.5 * 4.0 * a.batch * a.heads * a.seqlen * a.seqlen * a.dim / 2
    return report("attn_bwd_tcgen05 (+delta, dq cast)", ms, fl, seqlen=a.seqlen, batch=a.batch, heads=a.heads)


def bench_qknorm_rope(a):
    """Fused QK-norm + RoPE forward and backward on the layout of a fused QKV projection."""
    T = a.seqlen * a.batch
    nq, nkv, D = a.heads, a.kv_heads, a.dim
    W = (nq + 2 * nkv) * D
    qkv = torch.randn(T, W, device="cuda").bfloat16()
    wq = torch.ones(D, device="cuda").bfloat16()
    wk = torch.ones(D, device="cuda").bfloat16()
    pos = (torch.arange(T, device="cuda") % a.seqlen).int()
    cos, sin = OF.rope_tables(a.seqlen, D, 1e6, "cuda")
    ms = timeit(lambda: OF.qknorm_rope_fwd(qkv, wq, wk, pos, cos, sin, nq, nkv, D, 1e-6), a.iters, a.warmup)
    by = 2.0 * T * (nq + nkv) * D * 2
    report("qknorm_rope_fwd", ms, 0.0, by, tokens=T, heads=nq, kv_heads=nkv)
    qk, rstd = OF.qknorm_rope_fwd(qkv, wq, wk, pos, cos, sin, nq, nkv, D, 1e-6)
    dq32 = torch.randn(T, nq, D, device="cuda")
    dqkv = torch.randn(T, W, device="cuda").bfloat16()
    dwq, dwk = torch.zeros(D, device="cuda"), torch.zeros(D, device="cuda")
    L = oplib.get_lib()

    def bwd():
        oplib.check(L.ab2_qknorm_rope_bwd(qkv.data_ptr(), wq.data_ptr(), wk.data_ptr(), pos.data_ptr(), cos.data_ptr(), sin.data_ptr(),
                                          rstd.data_ptr(), dq32.data_ptr(), dqkv.data_ptr(), dwq.data_ptr(), dwk.data_ptr(), T, nq, nkv, D,
                                          W, W, oplib.stream_ptr()), "qknorm_rope_bwd")
    ms = timeit(bwd, a.iters, a.warmup)
    # reads: x (bf16), dq (fp32), dk (bf16); writes: dq/dk region (bf16)
    by = T * D * (nq * (2 + 4 + 2) + nkv * (2 + 2 + 2))
    return report("qknorm_rope_bwd", ms, 0.0, by, tokens=T, heads=nq, kv_heads=nkv)


def bench_decode(a):
    ps = 64
    pages_per = (a.ctx + ps - 1) // ps
    n_pages = a.batch * pages_per
    kc = torch.randn(n_pages * ps, a.kv_heads, a.dim, device="cuda").bfloat16()
    vc = torch.randn(n_pages * ps, a.kv_heads, a.dim, device="cuda").bfloat16()
    q = torch.randn(a.batch, a.heads, a.dim, device="cuda").bfloat16()
    pt = torch.randperm(n_pages, device="cuda").int().view(a.batch, pages_per).contiguous()
    lens = torch.full((a.batch,), a.ctx, device="cuda", dtype=torch.int32)
    splits = a.splits
    po = torch.empty(a.batch * a.heads * splits * a.dim, device="cuda")
    pml = torch.empty(a.batch * a.heads * splits * 2, device="cuda")
    out = torch.empty_like(q)
    L = oplib.get_lib()

    def run():
        oplib.check(L.ab2_paged_decode(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), pt.data_ptr(), lens.data_ptr(),
                                       po.data_ptr(), pml.data_ptr(), out.data_ptr(), a.batch, a.heads, a.kv_heads, a.dim,
                                       ps, pages_per, splits, a.dim ** -0.5, oplib.stream_ptr()), "decode")
    ms = timeit(run, a.iters, a.warmup)
    by = 2.0 * 2 * a.batch * a.ctx * a.kv_heads * a.dim
    return report("paged_decode_attention", ms, 0.0, by, batch=a.batch, ctx=a.ctx)


def bench_rmsnorm(a):
    x = torch.randn(a.rows, a.hidden, device="cuda").bfloat16()
    r = torch.randn_like(x)
    w = torch.ones(a.hidden, device="cuda").bfloat16()
    ms = timeit(lambda: OF.rmsnorm(x, w, 1e-6, r), a.iters, a.warmup)
    return report("rmsnorm_fwd(+residual)", ms, 0.0, 2.0 * 4 * a.rows * a.hidden, rows=a.rows, hidden=a.hidden)


def bench_swiglu(a):
    gu = torch.randn(a.rows, 2 * a.inter, device="cuda").bfloat16()
    ms = timeit(lambda: OF.swiglu(gu), a.iters, a.warmup)
    return report("swiglu_fwd", ms, 0.0, 2.0 * 3 * a.rows * a.inter, rows=a.rows, inter=a.inter)


def bench_adamw(a):
    n = a.numel
    p, m, v, g = (torch.randn(n, device="cuda") for _ in range(4))
    v.abs_()
    pb = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    st = torch.tensor([1.0, 1.0, 1.0, 1.0], device="cuda")
    ms = timeit(lambda: OF.adamw_step_(p, m, v, g, pb, st, 1e-5, 0.9, 0.95, 1e-8, 0.01, 3), a.iters, a.warmup)
    return report("adamw_fused(+bf16 copy)", ms, 0.0, n * (4 * 4 + 3 * 4 + 2), numel=n)


def bench_logprob(a):
    logits = torch.randn(a.rows, a.vocab, device="cuda")
    labels = torch.randint(0, a.vocab, (a.rows,), device="cuda")
    ms = timeit(lambda: OF.logprob_entropy_from_logits(logits, labels, 1.0), a.iters, a.warmup)
    return report("logprob_entropy_fwd", ms, 0.0, 4.0 * a.rows * a.vocab, rows=a.rows, vocab=a.vocab)


def bench_engine_decode(a):
    """Decode throughput of the rollout engine itself (continuous batching, CUDA graphs):
    ``--batch`` concurrent requests of ``--ctx`` prompt tokens generating ``--new`` tokens."""
    import asyncio
    import time

    from ..api.cli_args import GenerationHyperparameters, InferenceEngineConfig, NativeInferConfig
    from ..api.io_struct import ModelRequest
    from ..engine.infer_engine import NativeInferenceEngine
    from ..models.config import preset

    mc = preset(a.model) if not a.layers else preset(a.model, num_layers=a.layers)
    eng = NativeInferenceEngine(InferenceEngineConfig(), NativeInferConfig(max_running_requests=a.batch, context_length=a.ctx + a.new + 64,
                                                                           mem_fraction_static=0.5), model_config=mc)
    eng.initialize(start_executor=False)
    g = GenerationHyperparameters(max_new_tokens=a.new, max_tokens=a.ctx + a.new + 8, ignore_eos=True)
    gen = torch.Generator().manual_seed(0)

    async def run():
        reqs = [ModelRequest(input_ids=torch.randint(0, mc.vocab_size, (a.ctx,), generator=gen).tolist(), gconfig=g) for _ in range(a.batch)]
        return await asyncio.gather(*[eng.agenerate(r) for r in reqs])
    asyncio.run(run())          # warm-up: captures the graphs
    torch.cuda.synchronize()
    s0 = dict(eng.stats)
    t0 = time.perf_counter()
    out = asyncio.run(run())
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    steps = eng.stats["decode_steps"] - s0.get("decode_steps", 0)
    ntok = sum(r.output_len for r in out)
    wbytes = 2.0 * mc.num_params()
    res = {"kernel": "engine_decode (end to end, host included)", "model": a.model, "layers": mc.num_layers, "batch": a.batch, "ctx": a.ctx,
           "new": a.new, "seconds": round(dt, 3), "decode_steps": int(steps), "tokens_per_s": round(ntok / dt, 1),
           "ms_per_step_incl_prefill": round(1e3 * dt / max(1, steps), 3),
           "weight_stream_frac_of_hbm_peak": round(wbytes * steps / dt / 1e9 / peaks()["hbm_gbs"], 3), "kernel_error": oplib.kernel_error()}
    print(json.dumps(res), flush=True)
    eng.destroy()
    return res


def bench_ep(a):
    """Expert-parallel dispatch and combine kernels on ONE GPU: the ranks' receive buffers are separate local
    tensors (the kernels never wait on each other), so this measures the kernels against local HBM; over NVLink
    the same launches are bound by the 770 GB/s peer path for the remote share of the rows."""
    import types

    from ..parallel import ep_fused as EF
    from ..parallel.symm import ptr_array

    dev = torch.device("cuda")
    T, H, k, E, ep = a.rows, a.hidden, 8, 64, 2
    g = torch.Generator(device=dev).manual_seed(1)
    x = torch.randn(T, H, device=dev, generator=g).bfloat16()
    scores = torch.rand(T, E, device=dev, generator=g)
    topw, tope = scores.topk(k, dim=-1)
    flat_e = tope.reshape(-1)
    order = torch.argsort(flat_e, stable=True)
    mine = torch.bincount(flat_e, minlength=E)
    counts = torch.stack([mine, mine])                          # the other emulated rank routes the same way
    plan = EF.build_plan(counts, order, flat_e[order], 0, k)
    cap = plan.max_recv + 8
    bufs = [torch.zeros(cap, H, dtype=torch.bfloat16, device=dev) for _ in range(ep)]
    comm = types.SimpleNamespace(world=ep, hidden=H, capacity=cap, device=dev)
    slab = (None, None, ptr_array([b.data_ptr() for b in bufs]))
    w = topw.reshape(-1)[order].float().contiguous()
    N = T * k
    ms = timeit(lambda: EF._dispatch(comm, x, plan, slab), a.iters, a.warmup)
    report("ep_dispatch", ms, bytes_=N * H * 2 + T * H * 2, rows=N, hidden=H, note="reads T rows (k-fold reuse from L2), writes T*k rows")
    ms = timeit(lambda: EF._combine(comm, plan, slab, w=w), a.iters, a.warmup)
    report("ep_combine", ms, bytes_=N * H * 2 + T * H * 2, rows=N, hidden=H, note="reads T*k rows, writes T rows")
    ms = timeit(lambda: EF._combine(comm, plan, slab, w=w, save=True), a.iters, a.warmup)
    report("ep_combine_save", ms, bytes_=2 * N * H * 2 + T * H * 2, rows=N, hidden=H, note="also keeps the pulled rows for the backward")
    ys = torch.randn(N, H, device=dev, generator=g).bfloat16()
    ms = timeit(lambda: EF._dispatch(comm, x, plan, slab, scale=w, ys=ys), a.iters, a.warmup)
    return report("ep_dispatch_bwd", ms, bytes_=2 * N * H * 2 + T * H * 2, rows=N, hidden=H, note="scaled rows out + gate-weight gradients (reads the saved rows)")


def bench_moe_route(a):
    """Device-side routing (scores, top-k, stable sort by expert, group sizes, GEMM tile list; four small launches, no
    host read) against the eager statement of the same step (softmax, topk, argsort, bincount and the host copy of
    the counts that the tile table needs). ``--rows`` tokens, ``--experts`` experts, ``--topk`` choices."""
    T, E, k = a.rows, a.experts, a.topk
    logits = torch.randn(T, E, device="cuda") * 2.0

    def eager():
        probs = torch.softmax(logits, -1)
        tope = torch.topk(probs, k, -1).indices
        w = probs.gather(1, tope)
        w = w / w.sum(-1, keepdim=True)
        flat = tope.reshape(-1)
        order = torch.argsort(flat, stable=True)
        counts = torch.bincount(flat, minlength=E).tolist()          # the host needs them to build the tile table
        return order, w, counts
    ms = timeit(lambda: OF.moe_route(logits, k, want_probs=False), a.iters, a.warmup)
    by = 4.0 * T * E + 4.0 * T * k * 5
    res = report("moe_route (topk + stable sort + counts + tile list, 4 launches)", ms, 0.0, by, tokens=T, experts=E, topk=k)
    ms2 = timeit(eager, a.iters, a.warmup)
    report("eager routing (softmax, topk, argsort, bincount, counts to host)", ms2, 0.0, by, tokens=T, experts=E, topk=k)
    return res


def bench_push_plan(a):
    """The one-launch re-shard of ONE trainer shard (1 of ``--shards`` FSDP ranks) of ``--model`` into the
    tensor-parallel layout (``--tp``) of ``--replicas`` rollout replicas. On one GPU the "replicas" are local
    buffers, so this times the kernel against HBM (read the shard once, write it ``replicas`` times); over
    NVLink the same launch is timed inside ``bench.py`` (``weight_sync_device_ms``)."""
    from ..engine.flat_params import flat_layout
    from ..models.config import preset
    from ..models.decoder import build_model
    from ..parallel import tp as TP
    from ..parallel.weight_push import TPPushPlan, build_push_plan, tp_dst_layout

    cfg = preset(a.model)
    meta = build_model(cfg, dtype=torch.bfloat16, device="meta")
    names = [n for n, _ in meta.named_parameters()]
    shapes = [tuple(p.shape) for _, p in meta.named_parameters()]
    offs, padded = flat_layout([p.numel() for _, p in meta.named_parameters()], a.shards)
    lo = padded // a.shards * (a.shards - 1)                     # the last shard (has the LM head and the last layers)
    layout = tp_dst_layout(cfg, a.tp)
    ops = build_push_plan(cfg, names, offs, shapes, (lo, lo + padded // a.shards), a.tp, layout)
    plan = TPPushPlan(ops, a.tp, "cuda")
    src = torch.randn(padded // a.shards, device="cuda").bfloat16()
    for op in plan.ops:                                          # the source buffer here holds the shard only
        op.src_off -= lo
    plan = TPPushPlan(plan.ops, a.tp, "cuda")
    local = build_model(TP.local_config(cfg, a.tp), dtype=torch.bfloat16, device="meta")
    _, n_local = flat_layout([p.numel() for _, p in local.named_parameters()], 1)
    dst = [torch.empty(n_local, dtype=torch.bfloat16, device="cuda") for _ in range(a.replicas * a.tp)]
    ptrs = [t.data_ptr() for t in dst]
    ms = timeit(lambda: plan.run(src, ptrs, a.replicas), a.iters, a.warmup)
    return report("push_plan (FSDP shard -> TP layout, one launch)", ms, bytes_=plan.bytes * (1 + a.replicas), ops=len(plan.ops), tp=a.tp,
                  replicas=a.replicas, shard_gb=round(plan.bytes / 1e9, 2), note="local destinations: HBM-bound form of the NVLink push")


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("kernel", choices=["gemm", "gemm_decode", "gemm_fp8", "gemm_skinny", "qknorm_rope", "attn_fwd", "attn_bwd", "decode", "rmsnorm", "swiglu", "adamw", "logprob",
                                           "engine_decode", "ep", "push_plan", "moe_route"])
    ap.add_argument("--experts", type=int, default=128); ap.add_argument("--topk", type=int, default=8)
    ap.add_argument("--shards", type=int, default=4); ap.add_argument("--tp", type=int, default=2); ap.add_argument("--replicas", type=int, default=2)
    ap.add_argument("--model", type=str, default="qwen3-8b"); ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--new", type=int, default=128)
    ap.add_argument("--m", type=int, default=8192); ap.add_argument("--n", type=int, default=8192); ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--layout", type=str, default="nt", help="A major n|t, B major t|n: nt = x@W^T, nn = dy@W, tn = dy^T@x")
    ap.add_argument("--epi", type=int, default=0); ap.add_argument("--bn", type=int, default=0)
    ap.add_argument("--compare", action="store_true"); ap.add_argument("--split", type=int, default=0)
    ap.add_argument("--seqlen", type=int, default=4096); ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--heads", type=int, default=32); ap.add_argument("--kv-heads", type=int, default=8); ap.add_argument("--dim", type=int, default=128)
    ap.add_argument("--ctx", type=int, default=1024); ap.add_argument("--splits", type=int, default=4)
    ap.add_argument("--rows", type=int, default=32768); ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--inter", type=int, default=12288); ap.add_argument("--numel", type=int, default=1 << 28)
    ap.add_argument("--vocab", type=int, default=151936)
    ap.add_argument("--iters", type=int, default=10); ap.add_argument("--warmup", type=int, default=3)
    a = ap.parse_args(argv)
    if a.kernel == "logprob" and a.rows > 4096:
        a.rows = 2048
    return {"gemm": bench_gemm, "gemm_decode": bench_gemm_decode, "gemm_fp8": bench_gemm_fp8, "gemm_skinny": bench_gemm_skinny, "qknorm_rope": bench_qknorm_rope, "attn_fwd": bench_attn_fwd, "attn_bwd": bench_attn_bwd, "decode": bench_decode,
            "rmsnorm": bench_rmsnorm, "swiglu": bench_swiglu, "adamw": bench_adamw, "logprob": bench_logprob,
            "engine_decode": bench_engine_decode, "ep": bench_ep, "push_plan": bench_push_plan, "moe_route": bench_moe_route}[a.kernel](a)


if __name__ == "__main__":
    main()
