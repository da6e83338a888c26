"""2+ GPU check of the fused all-gather->GEMM and GEMM->reduce-scatter kernels against plain
PyTorch fp32 math on gathered operands, plus device-event timings against the NCCL pair.
Launched by tests/test_multi_gpu.py under torchrun. Prints TP_FUSED_OK per rank."""
import faulthandler
import json
import os
import sys

faulthandler.dump_traceback_later(150, exit=True)
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import torch
import torch.distributed as dist

from areal_b200.ops import lib as oplib
from areal_b200.parallel.tp_fused import FusedTPLinear


def rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def timed(fn, iters=10):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl")
    big = os.environ.get("TP_FUSED_BENCH", "0") == "1"
    rows, K, N = (4096, 4096, 6144) if big else (256, 512, 768)
    tp = FusedTPLinear(dist.group.WORLD, dev, max_rows_per_rank=rows, max_k=max(K, N), max_n=max(K, N))
    g = torch.Generator(device=dev).manual_seed(7 + rank)
    # ---- all-gather -> GEMM (column parallel forward): x rows differ per rank, w is this rank's slice
    x_loc = torch.randn(rows, K, device=dev, generator=g).bfloat16()
    w_col = (torch.randn(N // world, K, device=dev, generator=g) / K ** 0.5).bfloat16()
    xs = [torch.empty_like(x_loc) for _ in range(world)]
    dist.all_gather(xs, x_loc)
    x_full = torch.cat(xs, 0)
    for b_mn in (False, True):
        w = w_col.t().contiguous() if b_mn else w_col
        ref = x_full.float() @ w_col.float().t()
        for copy_once in (True, False, True):
            y = tp.allgather_gemm(x_loc, w, b_mn=b_mn, copy_once=copy_once)
            assert rel(y, ref) < 1e-2, ("ag_gemm", b_mn, copy_once, rel(y, ref))
        assert rel(tp.baseline_allgather_gemm(x_loc, w, b_mn=b_mn), ref) < 1e-2
    # ---- GEMM -> reduce-scatter (row parallel forward): full rows, K split over ranks
    x_row = torch.randn(rows * world, K // world, device=dev, generator=g).bfloat16()
    w_row = (torch.randn(N, K // world, device=dev, generator=g) / K ** 0.5).bfloat16()
    part = x_row.float() @ w_row.float().t()
    dist.all_reduce(part)
    mine = part[rank * rows:(rank + 1) * rows]
    for b_mn in (False, True):
        w = w_row.t().contiguous() if b_mn else w_row
        for _ in range(2):                                  # twice: the target buffer is reused
            o = tp.gemm_reduce_scatter(x_row, w, b_mn=b_mn, out_dtype=torch.float32)
            assert rel(o, mine) < 1e-2, ("gemm_rs", b_mn, rel(o, mine))
            o = tp.gemm_reduce_scatter(x_row, w, b_mn=b_mn, out_dtype=torch.float32, reduce_dtype=torch.bfloat16)
            assert rel(o, mine) < 2e-2, ("gemm_rs_bf16", b_mn, rel(o, mine))
        assert rel(tp.baseline_gemm_reduce_scatter(x_row, w, b_mn=b_mn, out_dtype=torch.float32), mine) < 1e-2
    torch.cuda.synchronize()
    assert oplib.kernel_error() == 0, oplib.kernel_error()
    if big:
        res = {
            "shape": {"rows_per_rank": rows, "K": K, "N": N, "world": world},
            "allgather_gemm_copy_once_ms": timed(lambda: tp.allgather_gemm(x_loc, w_col)),
            "allgather_gemm_remote_tma_ms": timed(lambda: tp.allgather_gemm(x_loc, w_col, copy_once=False)),
            "nccl_allgather_then_gemm_ms": timed(lambda: tp.baseline_allgather_gemm(x_loc, w_col)),
            "gemm_reduce_scatter_ms": timed(lambda: tp.gemm_reduce_scatter(x_row, w_row)),
            "gemm_reduce_scatter_bf16_ms": timed(lambda: tp.gemm_reduce_scatter(x_row, w_row, reduce_dtype=torch.bfloat16)),
            "gemm_only_ms": timed(lambda: tp.baseline_gemm_only(x_loc, w_col)),
            "gemm_then_nccl_reduce_scatter_ms": timed(lambda: tp.baseline_gemm_reduce_scatter(x_row, w_row)),
        }
        if rank == 0:
            print("TP_FUSED_BENCH " + json.dumps(res), flush=True)
    print("TP_FUSED_OK", flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
