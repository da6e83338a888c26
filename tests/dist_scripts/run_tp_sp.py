"""Sequence-parallel TP linear pair (column then row) against the unsplit MLP-like chain on
gloo ranks. Prints TP_SP_OK per rank."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from areal_b200.parallel.tp import column_parallel_sp, row_parallel_sp  # noqa: E402


def main():
    dist.init_process_group("gloo")
    rank, P = dist.get_rank(), dist.get_world_size()
    g = torch.Generator().manual_seed(0)
    T, H, I = 8 * P, 16, 24 * P
    x = torch.randn(T, H, generator=g)
    w1 = torch.randn(I, H, generator=g) * 0.2
    w2 = torch.randn(H, I, generator=g) * 0.2
    gy = torch.randn(T, H, generator=g)
    # reference
    xr, w1r, w2r = x.clone().requires_grad_(), w1.clone().requires_grad_(), w2.clone().requires_grad_()
    yr = torch.tanh(xr @ w1r.t()) @ w2r.t()
    yr.backward(gy)
    # sharded: rows of x / y per rank, w1 by output features, w2 by input features
    rows = slice(rank * T // P, (rank + 1) * T // P)
    cols = slice(rank * I // P, (rank + 1) * I // P)
    xs = x[rows].clone().requires_grad_()
    w1s, w2s = w1[cols].clone().requires_grad_(), w2[:, cols].clone().requires_grad_()
    ys = row_parallel_sp(torch.tanh(column_parallel_sp(xs, w1s, dist.group.WORLD)), w2s, dist.group.WORLD)
    ys.backward(gy[rows])
    assert torch.allclose(ys, yr[rows], atol=1e-5)
    assert torch.allclose(xs.grad, xr.grad[rows], atol=1e-5)
    assert torch.allclose(w1s.grad, w1r.grad[cols], atol=1e-5) and torch.allclose(w2s.grad, w2r.grad[:, cols], atol=1e-5)
    print("TP_SP_OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
