"""Flat parameter / gradient / optimizer-state storage for ZeRO-style data parallelism.

All parameters of a model are re-homed into one contiguous compute-dtype buffer
(``flat_param``); every parameter also gets ``main_grad``, a view into one contiguous fp32
gradient buffer (``flat_grad``) that the weight-gradient GEMMs accumulate into directly.
Each data-parallel rank owns one contiguous shard of the flat space: fp32 master weights and
Adam moments exist only for that shard.

B200 sizing rule: compute-dtype parameters stay replicated on every rank (a 8B model is
16 GB of 180 GB), so forward/backward need no parameter all-gather at all; gradients are
reduce-scattered once per step and the updated bf16 shard is written back to every peer.
The reference reaches the same state with FSDP2 ``fully_shard``
(``areal/engine/fsdp_utils/parallel.py:388-396``) at the cost of per-layer all-gathers.
"""
from __future__ import annotations

import math
from typing import Callable, Optional

import torch
import torch.nn as nn

ALIGN = 256  # elements; keeps every shard 16-byte aligned for vector / TMA access
TENSOR_ALIGN = 128  # elements: every tensor starts on a 128-element boundary, so 1 x 128 scaling blocks of a
                    # row never straddle a shard boundary (in-kernel fp8 cast of the weight push) and all
                    # vector / TMA accesses are 16-byte aligned


def flat_layout(numels: list[int], world_size: int = 1) -> tuple[list[int], int]:
    """(element offset of every tensor, padded total) of a flat buffer over tensors of ``numels``
    elements, sharded over ``world_size`` ranks. Pure arithmetic: used to plan against a layout
    that lives in another process."""
    offs, total = [], 0
    for n in numels:
        offs.append(total)
        total += (n + TENSOR_ALIGN - 1) // TENSOR_ALIGN * TENSOR_ALIGN
    unit = ALIGN * world_size
    return offs, (total + unit - 1) // unit * unit


class FlatParamStore:
    def __init__(self, model: nn.Module, world_size: int = 1, rank: int = 0, grad_dtype=torch.float32,
                 alloc_param: Optional[Callable[[int, torch.dtype, torch.device], torch.Tensor]] = None,
                 alloc_grad: Optional[Callable[[int, torch.dtype, torch.device], torch.Tensor]] = None,
                 with_grads: bool = True, only_trainable: bool = False, include: Optional[Callable[[str], bool]] = None):
        params = [(n, p) for n, p in model.named_parameters()
                  if (p.requires_grad or not only_trainable) and (include is None or include(n))]
        if not params:
            raise ValueError("model has no parameters")
        self.names = [n for n, _ in params]
        self.params = [p for _, p in params]
        dev, dtype = self.params[0].device, self.params[0].dtype
        self.device, self.dtype = dev, dtype
        self.world_size, self.rank = world_size, rank
        offs, self.padded = flat_layout([p.numel() for p in self.params], world_size)
        self.numel = (offs[-1] + self.params[-1].numel()) if offs else 0
        self.offsets = offs
        self.shard_numel = self.padded // world_size
        alloc_param = alloc_param or (lambda n, dt, d: torch.zeros(n, dtype=dt, device=d))
        alloc_grad = alloc_grad or (lambda n, dt, d: torch.zeros(n, dtype=dt, device=d))
        self.flat_param = alloc_param(self.padded, dtype, dev)
        with torch.no_grad():
            for p, off in zip(self.params, offs):
                self.flat_param[off:off + p.numel()].copy_(p.data.reshape(-1))
                p.data = self.flat_param[off:off + p.numel()].view(p.shape)
        self.flat_grad = None
        if with_grads:
            self.flat_grad = alloc_grad(self.padded, grad_dtype, dev)
            for p, off in zip(self.params, offs):
                p.main_grad = self.flat_grad[off:off + p.numel()].view(p.shape)
        lo = rank * self.shard_numel
        self.shard_range = (lo, lo + self.shard_numel)

    # ------------------------------------------------------------------ views
    @property
    def param_shard(self) -> torch.Tensor:
        return self.flat_param[self.shard_range[0]:self.shard_range[1]]

    @property
    def grad_shard(self) -> torch.Tensor:
        return self.flat_grad[self.shard_range[0]:self.shard_range[1]]

    def zero_grad(self) -> None:
        if self.flat_grad is not None:
            self.flat_grad.zero_()
        for p in self.params:
            p.grad = None

    @torch.no_grad()
    def fold_autograd_grads(self) -> None:
        """Adds gradients that autograd produced in ``.grad`` (ops without a fused fp32
        accumulation path) into ``main_grad`` and drops them."""
        for p in self.params:
            if p.grad is not None:
                p.main_grad.add_(p.grad.to(p.main_grad.dtype))
                p.grad = None

    def named_views(self):
        return zip(self.names, self.params)

    def locate(self, name: str) -> tuple[int, int]:
        i = self.names.index(name)
        return self.offsets[i], self.params[i].numel()

    def memory_bytes(self) -> int:
        b = self.flat_param.numel() * self.flat_param.element_size()
        if self.flat_grad is not None:
            b += self.flat_grad.numel() * self.flat_grad.element_size()
        return b
