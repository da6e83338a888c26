"""2+ GPU check of the projection kernels that carry the Ulysses all-to-alls (GEMM -> scatter
by head owner, gather of column panels -> GEMM) against fp32 math on gathered operands, with
timings against projection + NCCL all_to_all_single. Prints ULYSSES_FUSED_OK per rank."""
import faulthandler
import json
import os
import sys

faulthandler.dump_traceback_later(150, exit=True)
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import torch
import torch.distributed as dist

from areal_b200.ops import lib as oplib
from areal_b200.parallel.tp_fused import FusedUlyssesLinear


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
    big = os.environ.get("ULYSSES_FUSED_BENCH", "0") == "1"
    M, H, NQKV = (4096, 4096, 6144) if big else (256, 512, 768)     # tokens per rank, hidden, q+k+v columns
    ul = FusedUlyssesLinear(dist.group.WORLD, dev, max_rows_per_rank=M, max_cols=max(H, NQKV))
    g = torch.Generator(device=dev).manual_seed(11 + rank)
    # ---- QKV projection + seq->heads
    x_loc = torch.randn(M, H, device=dev, generator=g).bfloat16()
    gw = torch.Generator(device=dev).manual_seed(3)                 # weights identical on every rank
    w_qkv = (torch.randn(NQKV, H, device=dev, generator=gw) / H ** 0.5).bfloat16()
    xs = [torch.empty_like(x_loc) for _ in range(world)]
    dist.all_gather(xs, x_loc)
    ref_full = torch.cat(xs, 0).float() @ w_qkv.float().t()          # [P*M, NQKV]
    cpr = NQKV // world
    ref_mine = ref_full[:, rank * cpr:(rank + 1) * cpr]
    for _ in range(2):
        y = ul.project_scatter(x_loc, w_qkv)
        assert y.shape == (world * M, cpr) and rel(y, ref_mine) < 1e-2, ("project_scatter", rel(y, ref_mine))
    assert rel(ul.baseline_project_scatter(x_loc, w_qkv), ref_mine) < 1e-2
    # ---- heads->seq + output projection
    o_full = torch.randn(world * M, H // world, device=dev, generator=g).bfloat16()   # all tokens, local heads' outputs
    w_o = (torch.randn(H, H, device=dev, generator=gw) / H ** 0.5).bfloat16()
    os_ = [torch.empty_like(o_full) for _ in range(world)]
    dist.all_gather(os_, o_full)
    a_mine = torch.cat([o[rank * M:(rank + 1) * M] for o in os_], dim=1)               # [M, H]
    ref_o = a_mine.float() @ w_o.float().t()
    for _ in range(2):
        y = ul.gather_project(o_full, w_o)
        assert rel(y, ref_o) < 1e-2, ("gather_project", rel(y, ref_o))
    assert rel(ul.baseline_gather_project(o_full, w_o), ref_o) < 1e-2
    torch.cuda.synchronize()
    assert oplib.kernel_error() == 0, oplib.kernel_error()
    if big:
        res = {"shape": {"tokens_per_rank": M, "hidden": H, "qkv_cols": NQKV, "world": world},
               "project_scatter_ms": timed(lambda: ul.project_scatter(x_loc, w_qkv)),
               "project_then_nccl_a2a_ms": timed(lambda: ul.baseline_project_scatter(x_loc, w_qkv)),
               "gather_project_ms": timed(lambda: ul.gather_project(o_full, w_o)),
               "nccl_a2a_then_project_ms": timed(lambda: ul.baseline_gather_project(o_full, w_o))}
        if rank == 0:
            print("ULYSSES_FUSED_BENCH " + json.dumps(res), flush=True)
    print("ULYSSES_FUSED_OK", flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
