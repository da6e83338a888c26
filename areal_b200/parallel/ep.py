"""Expert parallelism for the MoE MLP.

Experts are partitioned over the EP group (rank r owns experts ``[r*E/ep, (r+1)*E/ep)``);
the router is replicated. Per layer: count exchange -> token dispatch all-to-all (variable
splits) -> local regroup by expert -> expert GEMMs -> inverse regroup -> combine all-to-all.
Both all-to-alls are differentiable (the backward of a dispatch is a combine with the splits
swapped). This is the library path (and the CPU path); on GPUs ``parallel/ep_fused.py`` replaces both
directions with one peer-memory kernel each. Reference:
``areal/experimental/models/archon/expert_parallel.py`` (count exchange :131, dispatch :163,
combine :207).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist
import torch.nn as nn


class _AllToAll(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, send_splits: list[int], recv_splits: list[int], group):
        ctx.group, ctx.send_splits, ctx.recv_splits = group, send_splits, recv_splits
        out = x.new_empty((sum(recv_splits),) + tuple(x.shape[1:]))
        dist.all_to_all_single(out, x.contiguous(), output_split_sizes=recv_splits, input_split_sizes=send_splits, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        out = g.new_empty((sum(ctx.send_splits),) + tuple(g.shape[1:]))
        dist.all_to_all_single(out, g.contiguous(), output_split_sizes=ctx.send_splits, input_split_sizes=ctx.recv_splits,
                               group=ctx.group)
        return out, None, None, None


def all_to_all_tokens(x: torch.Tensor, send_splits: list[int], recv_splits: list[int], group) -> torch.Tensor:
    if dist.get_backend(group) == "gloo" and not hasattr(dist, "_gloo_a2a_ok"):
        # gloo has no all_to_all_single with uneven splits on every build: emulate with p2p
        return _P2PAllToAll.apply(x, send_splits, recv_splits, group)
    return _AllToAll.apply(x, send_splits, recv_splits, group)


def _p2p_a2a(x, send_splits, recv_splits, group):
    ranks = dist.get_process_group_ranks(group)
    me = dist.get_rank(group)
    out = x.new_empty((sum(recv_splits),) + tuple(x.shape[1:]))
    ins = list(torch.split(x.contiguous(), send_splits))
    outs = list(torch.split(out, recv_splits))
    ops = []
    for r in range(len(ranks)):
        if r == me:
            outs[r].copy_(ins[r])
            continue
        if send_splits[r] > 0:
            ops.append(dist.P2POp(dist.isend, ins[r].contiguous(), ranks[r], group))
        if recv_splits[r] > 0:
            ops.append(dist.P2POp(dist.irecv, outs[r], ranks[r], group))
    if ops:
        for w in dist.batch_isend_irecv(ops):
            w.wait()
    return out


class _P2PAllToAll(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, send_splits, recv_splits, group):
        ctx.group, ctx.send_splits, ctx.recv_splits = group, send_splits, recv_splits
        return _p2p_a2a(x, send_splits, recv_splits, group)

    @staticmethod
    def backward(ctx, g):
        return _p2p_a2a(g, ctx.recv_splits, ctx.send_splits, ctx.group), None, None, None


class ExpertParallelDispatcher:
    """Callable installed as ``MoEMLP.ep_dispatcher``."""

    def __init__(self, group, ep_rank: int, ep_size: int):
        self.group, self.ep_rank, self.ep_size = group, ep_rank, ep_size
        self.last_recv_tokens = 0

    def __call__(self, mlp, xs: torch.Tensor, sorted_experts: torch.Tensor) -> torch.Tensor:
        """``xs``: [N, H] tokens sorted by global expert id ``sorted_experts`` [N]. Returns the
        expert outputs in the same order."""
        E, ep = mlp.cfg.num_experts, self.ep_size
        El = E // ep
        counts = torch.bincount(sorted_experts, minlength=E).view(ep, El)
        recv_counts = torch.empty_like(counts)
        if dist.get_backend(self.group) == "gloo":
            gathered = [torch.empty_like(counts) for _ in range(ep)]
            dist.all_gather(gathered, counts.contiguous(), group=self.group)
            recv_counts = torch.stack([gathered[src][self.ep_rank] for src in range(ep)])
        else:
            dist.all_to_all_single(recv_counts, counts.contiguous(), group=self.group)
        send_splits = counts.sum(1).tolist()                 # host sync: split sizes drive the transfer
        recv_mat = recv_counts.tolist()                      # [src][local expert]
        recv_splits = [sum(r) for r in recv_mat]
        got = all_to_all_tokens(xs, send_splits, recv_splits, self.group)
        self.last_recv_tokens = got.shape[0]
        # received order: (source rank, local expert); regroup to (local expert, source rank)
        expert_of = torch.cat([torch.repeat_interleave(torch.arange(El, device=xs.device), torch.tensor(r, device=xs.device))
                               for r in recv_mat]) if got.shape[0] else torch.zeros(0, dtype=torch.long, device=xs.device)
        perm = torch.argsort(expert_of, stable=True)
        per_expert = [sum(recv_mat[src][e] for src in range(ep)) for e in range(El)]
        ys_local = mlp.experts_forward(got[perm], per_expert, first_expert=0)
        back = torch.empty_like(ys_local)
        back[perm] = ys_local
        return all_to_all_tokens(back, recv_splits, send_splits, self.group)


def shard_experts(model, ep_rank: int, ep_size: int, group, fused: bool = False, device=None) -> list[str]:
    """Keeps only this rank's experts in every MoE layer and installs the dispatcher. Returns
    the names of the expert parameters (they are NOT replicated over the EP group: their
    gradients are reduced over the expert-data-parallel replicas only). ``fused`` wraps the
    dispatchers with the peer-memory dispatch / combine kernels (CUDA only); the communicator
    is kept as ``model.ep_fused_comm``."""
    expert_params = []
    for lname, layer in model.layers.named_children():
        mlp = layer.mlp
        if not hasattr(mlp, "w_gate_up"):
            continue
        E = mlp.cfg.num_experts
        if E % ep_size:
            raise ValueError(f"{E} experts are not divisible by ep={ep_size}")
        El = E // ep_size
        sl = slice(ep_rank * El, (ep_rank + 1) * El)
        mlp.w_gate_up = nn.Parameter(mlp.w_gate_up.detach()[sl].clone())
        mlp.w_down = nn.Parameter(mlp.w_down.detach()[sl].clone())
        mlp.ep_dispatcher = ExpertParallelDispatcher(group, ep_rank, ep_size)
        mlp.first_local_expert, mlp.num_local_experts = ep_rank * El, El
        expert_params += [f"layers.{lname}.mlp.w_gate_up", f"layers.{lname}.mlp.w_down"]
    if fused and expert_params:
        from .ep_fused import install_fused_dispatch

        model.ep_fused_comm = install_fused_dispatch(model, group, ep_rank, ep_size, device)
    return expert_params


def unshard_expert_tensor(parts: list[torch.Tensor]) -> torch.Tensor:
    return torch.cat(parts, dim=0)
