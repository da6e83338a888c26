"""Zig-zag context parallelism on gloo ranks: split / gather round trip, attention of the local
queries against gathered keys / values (forward and gradients) against single-process causal
attention. Prints CP_OK per rank."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
os.environ["AREAL_FORCE_CPU"] = "1"

from areal_b200.ops import functional as OF  # noqa: E402
from areal_b200.parallel import cp as CP  # noqa: E402


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    g = torch.Generator().manual_seed(0)
    lens = [13, 32, 7, 21]
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    T, Hq, Hkv, D = int(cu[-1]), 4, 2, 16
    q = torch.randn(T, Hq, D, generator=g, dtype=torch.float64)
    k = torch.randn(T, Hkv, D, generator=g, dtype=torch.float64)
    v = torch.randn(T, Hkv, D, generator=g, dtype=torch.float64)
    do = torch.randn(T, Hq, D, generator=g, dtype=torch.float64)
    # layout: every rank holds chunks r and 2cp-1-r; local loads are equal
    src, pos, local_lens = CP.zigzag_indices(cu, world, rank)
    assert sum(local_lens) == src.numel() and all(n % 2 == 0 for n in local_lens)
    x = torch.arange(T, dtype=torch.float64)[:, None].repeat(1, 3)
    xl = CP.zigzag_split(x, cu, world, rank, pad_value=-1)
    back = CP.gather_sequence(xl, cu, world, dist.group.WORLD)
    assert torch.equal(back, x)
    # attention
    ql = CP.zigzag_split(q, cu, world, rank).requires_grad_(True)
    kl = CP.zigzag_split(k, cu, world, rank).requires_grad_(True)
    vl = CP.zigzag_split(v, cu, world, rank).requires_grad_(True)
    ol = CP.cp_attention(ql, kl, vl, cu, world, rank, dist.group.WORLD)
    dol = CP.zigzag_split(do, cu, world, rank)
    valid = (src >= 0)
    (ol * dol)[valid].sum().backward()
    qr, kr, vr = (t.clone().requires_grad_(True) for t in (q, k, v))
    oref, _ = OF.attention_ref(qr.float(), kr.float(), vr.float(), cu, True)
    # float64 reference for tight tolerances
    import math
    outs = []
    for a, b in zip(cu[:-1].tolist(), cu[1:].tolist()):
        s = torch.einsum("qhd,khd->hqk", qr[a:b], kr[a:b].repeat_interleave(2, 1)) / math.sqrt(D)
        s = s.masked_fill(~torch.ones(b - a, b - a, dtype=torch.bool).tril(), float("-inf"))
        outs.append(torch.einsum("hqk,khd->qhd", torch.softmax(s, -1), vr[a:b].repeat_interleave(2, 1)))
    oref = torch.cat(outs, 0)
    (oref * do).sum().backward()
    assert torch.allclose(ol[valid], CP.zigzag_split(oref.detach(), cu, world, rank)[valid], atol=1e-9)
    assert torch.allclose(ql.grad[valid], CP.zigzag_split(qr.grad, cu, world, rank)[valid], atol=1e-9)
    # dK / dV: each rank's local gradient is the reduce-scattered total
    assert torch.allclose(kl.grad[valid], CP.zigzag_split(kr.grad, cu, world, rank)[valid], atol=1e-9)
    assert torch.allclose(vl.grad[valid], CP.zigzag_split(vr.grad, cu, world, rank)[valid], atol=1e-9)
    print("CP_OK", flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
