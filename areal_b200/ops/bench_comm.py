"""Multi-rank microbenchmarks of the fused communication paths, one process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \\
        -m areal_b200.ops.bench_comm zero_step --numel 2000000000

``zero_step``: the optimizer step of ZeRO data parallelism over ``N`` ranks on a flat buffer of ``--numel``
parameters: fp32 gradient reduce-scatter + global norm + clipping + AdamW on the shard + bf16 parameter write-back
to every rank. Fused form: ``rs_sumsq`` (peer loads) -> ``norm_allreduce`` (peer stores) -> ``clip_coef`` ->
``adamw_push`` (peer stores) with two flag barriers. Library form: NCCL ``reduce_scatter_tensor`` -> squared norm
+ ``all_reduce`` -> ``clip_coef`` -> AdamW kernel -> NCCL ``all_gather_into_tensor``. Times are CUDA events on
the launching stream, the maximum over ranks; every rank prints nothing, rank 0 prints one JSON line per form.
"""
from __future__ import annotations

import argparse
import json
import os
import types

import torch
import torch.distributed as dist


def _timed(fn, iters: int, warmup: int) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(iters)]
    for a, b in ev:
        a.record()
        fn()
        b.record()
    torch.cuda.synchronize()
    ms = sum(a.elapsed_time(b) for a, b in ev) / iters
    t = torch.tensor([ms], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t[0])


def bench_zero_step(a) -> None:
    from ..api.cli_args import OptimizerConfig
    from ..ops import functional as OF
    from ..ops import lib as oplib
    from ..parallel.fused_zero import FusedGradReducer
    from ..parallel.symm import symm_empty

    rank, world = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cuda", torch.cuda.current_device())
    unit = 128 * world
    n = (int(a.numel) + unit - 1) // unit * unit
    shard = n // world
    grad, gh = symm_empty(n, torch.float32, dev, dist.group.WORLD)
    param, ph = symm_empty(n, torch.bfloat16, dev, dist.group.WORLD)
    grad.normal_(0, 1e-3)
    param.normal_(0, 0.02)
    store = types.SimpleNamespace(device=dev, shard_numel=shard, shard_range=(rank * shard, (rank + 1) * shard),
                                  param_shard=param[rank * shard:(rank + 1) * shard], numel=n)
    cfg = OptimizerConfig(lr=1e-5, weight_decay=0.01, gradient_clipping=1.0)
    opt = types.SimpleNamespace(cfg=cfg, master=param[rank * shard:(rank + 1) * shard].float(), exp_avg=torch.zeros(shard, device=dev),
                                exp_avg_sq=torch.zeros(shard, device=dev), step_count=0, state=torch.zeros(4, device=dev))
    red = FusedGradReducer(store, dist.group.WORLD, list(gh.buffer_ptrs), list(ph.buffer_ptrs))

    def fused():
        red.reduce_scatter(opt.state)
        OF.clip_coef_(opt.state, 1.0, 1.0)
        opt.step_count += 1
        red.adamw_and_all_gather(opt, opt.state, 1e-5)

    gshard = torch.empty(shard, device=dev)
    pfull = torch.empty(n, dtype=torch.bfloat16, device=dev)

    def library():
        dist.reduce_scatter_tensor(gshard, grad)
        opt.state.zero_()
        OF.sqnorm_accumulate_(gshard, opt.state)
        dist.all_reduce(opt.state[0:1])
        OF.clip_coef_(opt.state, 1.0, 1.0)
        opt.step_count += 1
        OF.adamw_step_(opt.master, opt.exp_avg, opt.exp_avg_sq, gshard, store.param_shard, opt.state, 1e-5, cfg.beta1, cfg.beta2, cfg.eps,
                       cfg.weight_decay, opt.step_count)
        dist.all_gather_into_tensor(pfull, store.param_shard)

    ms_f = _timed(fused, a.iters, a.warmup)
    err = oplib.kernel_error()
    ms_l = _timed(library, a.iters, a.warmup)
    # bytes that must cross NVLink per GPU and direction: (world - 1) / world of the fp32 gradient shard's peers
    # inbound, the same share of the bf16 parameters outbound (the two phases do not overlap)
    link_bytes = (world - 1) * shard * 4.0 + (world - 1) * shard * 2.0
    hbm_bytes = shard * (4.0 * world + 4.0 + 4 * 3 * 2 + 2.0 * world)       # local reads of every peer's slice + state read/write + writes
    if rank == 0:
        for name, ms in (("zero_step fused (rs_sumsq + norm exchange + adamw_push, peer memory)", ms_f),
                         ("zero_step library (NCCL reduce-scatter / all-reduce / all-gather + AdamW kernel)", ms_l)):
            print(json.dumps({"kernel": name, "ms": round(ms, 3), "world": world, "numel": n, "nvlink_gbs_per_gpu_direction": round(link_bytes / ms / 1e6, 1),
                              "frac_of_770_gbs_peer_copy": round(link_bytes / ms / 1e6 / 770.0, 3), "kernel_error": err,
                              "nvls": os.environ.get("NCCL_NVLS_ENABLE", "default")}), flush=True)


def main(argv=None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("kernel", choices=["zero_step"])
    ap.add_argument("--numel", type=float, default=2.0e9)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    a = ap.parse_args(argv)
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    dist.init_process_group("nccl")
    try:
        {"zero_step": bench_zero_step}[a.kernel](a)
        dist.barrier()
    finally:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
