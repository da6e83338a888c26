"""Parameter sharding (ZeRO-3): no rank keeps a full copy of the weights.

:class:`FlatParamStore` replicates the compute-dtype parameters and the fp32 gradient buffer on every rank and
shards only the optimizer state: right for an 8B model on 180 GB GPUs, not for a model whose bf16 weights plus
fp32 gradients do not fit beside the activations. :class:`ShardedParamStore` keeps the same flat element space and
the same contiguous shard per rank (so :class:`~areal_b200.engine.optimizer.ShardedAdamW` and the sharded checkpoint
work unchanged) but holds only

* ``param_shard``  this rank's slice of the compute-dtype weights,
* ``grad_shard``   this rank's slice of the fp32 gradients (already summed over the group),

and materialises the weights one *unit* at a time: unit 0 is everything outside the decoder layers (embedding, final
norm, heads), unit ``i + 1`` is decoder layer ``i``. A unit's elements are contiguous in the flat space, so it is
owned by one to three neighbouring ranks; materialising it is one broadcast per owner into a transient buffer that the
unit's parameters are pointed at, releasing it points them at a placeholder again.

During a training micro-batch the model's layer loop calls :meth:`enter` / :meth:`leave` around every layer:

=============  =====================================================================================
forward        ``enter``: wait for the unit (prefetched one layer ahead), start fetching the next;
               ``leave``: release the unit
backward       the gradient of ``leave`` re-materialises the unit (and starts fetching the previous
               one); the gradient of ``enter`` runs after every gradient of the layer exists: the
               unit's fp32 gradients are reduced to their owners with asynchronous collectives that
               overlap the backward of the layers below, and the unit is released
=============  =====================================================================================

Role of FSDP2 ``fully_shard`` with ``reshard_after_forward`` in the reference
(``areal/engine/fsdp_utils/parallel.py:388-396``, ``areal/engine/fsdp_utils/__init__.py:62``,
``areal/engine/fsdp_engine.py:696-727``). Collectives here are the library's (NCCL on GPUs, gloo on CPU).
"""
from __future__ import annotations

import re
from typing import Iterator, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from .flat_params import TENSOR_ALIGN, flat_layout

_LAYER = re.compile(r"^layers\.(\d+)\.")


def unit_of(name: str) -> int:
    """0 for parameters outside the decoder layers, ``i + 1`` for ``layers.<i>.*``."""
    m = _LAYER.match(name)
    return int(m.group(1)) + 1 if m else 0


class _Enter(torch.autograd.Function):
    @staticmethod
    def forward(ctx, store, unit, *tensors):
        ctx.store, ctx.unit = store, unit
        store._fwd_enter(unit)
        return tensors

    @staticmethod
    def backward(ctx, *grads):
        ctx.store._bwd_leave(ctx.unit)
        return (None, None) + grads


class _Leave(torch.autograd.Function):
    @staticmethod
    def forward(ctx, store, unit, *tensors):
        ctx.store, ctx.unit = store, unit
        store._fwd_leave(unit)
        return tensors

    @staticmethod
    def backward(ctx, *grads):
        ctx.store._bwd_enter(ctx.unit)
        return (None, None) + grads


class ShardedParamStore:
    def __init__(self, model: nn.Module, world_size: int = 1, rank: int = 0, group=None, group_ranks: Optional[list[int]] = None,
                 grad_dtype=torch.float32, with_grads: bool = True, prefetch: bool = True, device=None):
        named = [(n, p) for n, p in model.named_parameters()]
        if not named:
            raise ValueError("model has no parameters")
        order = sorted(range(len(named)), key=lambda i: (unit_of(named[i][0]), i))
        self.names = [named[i][0] for i in order]
        self.params = [named[i][1] for i in order]
        self.units_of = [unit_of(n) for n in self.names]
        self.n_units = max(self.units_of) + 1
        # ``device``: where the shards and the transient units live; the model itself may have been built on the host
        # so that no device ever sees the whole of it
        dev, dtype = torch.device(device) if device is not None else self.params[0].device, self.params[0].dtype
        self.device, self.dtype, self.grad_dtype = dev, dtype, grad_dtype
        self.world_size, self.rank, self.group = world_size, rank, group
        self.group_ranks = list(group_ranks) if group_ranks is not None else list(range(world_size))
        self.prefetch = bool(prefetch) and world_size > 1
        self.offsets, self.padded = flat_layout([p.numel() for p in self.params], world_size)
        self.numel = self.offsets[-1] + self.params[-1].numel()
        self.shard_numel = self.padded // world_size
        lo = rank * self.shard_numel
        self.shard_range = (lo, lo + self.shard_numel)
        # element range of every unit (whole aligned slots of its parameters)
        self.unit_range: list[tuple[int, int]] = []
        self.unit_members: list[list[int]] = [[] for _ in range(self.n_units)]
        for i, u in enumerate(self.units_of):
            self.unit_members[u].append(i)
        for u in range(self.n_units):
            idx = self.unit_members[u]
            if not idx:
                self.unit_range.append((0, 0))
                continue
            a = self.offsets[idx[0]]
            last = idx[-1]
            b = self.offsets[last] + (self.params[last].numel() + TENSOR_ALIGN - 1) // TENSOR_ALIGN * TENSOR_ALIGN
            self.unit_range.append((a, b))
        self.param_shard = torch.zeros(self.shard_numel, dtype=dtype, device=dev)
        with torch.no_grad():
            for p, off in zip(self.params, self.offsets):
                self._write_flat(off, p.data.reshape(-1))
        self.grad_shard = torch.zeros(self.shard_numel, dtype=grad_dtype, device=dev) if with_grads else None
        self.flat_param = None          # never exists as a whole
        self.flat_grad = None
        self._nan = torch.full((1,), float("nan"), dtype=dtype, device=dev)
        self._live: dict[int, tuple] = {}            # unit -> (buffer, pending works)
        self._gbuf: dict[int, torch.Tensor] = {}     # unit -> fp32 gradient buffer of a unit that is in its backward
        self._reducing: list[tuple] = []             # (works, buffer, pieces, unit start) of reductions in flight
        self._root_users = 0
        self.peak_live_numel = 0
        # called with (names, parameters) of a unit after its gradients were folded into ``main_grad`` and before they are
        # reduced: the place for sums over another parallel dimension (tensor-parallel partial gradients)
        self.grad_hook = None
        for u in range(self.n_units):
            self._point_at_placeholder(u)
        for b in model.buffers():
            if b.device != dev:
                b.data = b.data.to(dev)

    # ------------------------------------------------------------------ arithmetic
    def _pieces(self, a: int, b: int) -> list[tuple[int, int, int]]:
        """(owner, lo, hi) for every rank whose shard meets [a, b)."""
        S = self.shard_numel
        out = []
        for o in range(a // S, min(self.world_size - 1, (b - 1) // S) + 1 if b > a else 0):
            lo, hi = max(a, o * S), min(b, (o + 1) * S)
            if lo < hi:
                out.append((o, lo, hi))
        return out

    def _write_flat(self, off: int, flat: torch.Tensor) -> None:
        """Copies ``flat`` (elements [off, off + n) of the flat space) into this rank's shard where they meet."""
        lo, hi = self.shard_range
        a, b = max(off, lo), min(off + flat.numel(), hi)
        if a < b:
            self.param_shard[a - lo:b - lo].copy_(flat[a - off:b - off].to(self.dtype))

    def locate(self, name: str) -> tuple[int, int]:
        i = self.names.index(name)
        return self.offsets[i], self.params[i].numel()

    def named_views(self):
        return zip(self.names, self.params)

    def memory_bytes(self) -> int:
        b = self.param_shard.numel() * self.param_shard.element_size()
        if self.grad_shard is not None:
            b += self.grad_shard.numel() * self.grad_shard.element_size()
        return b

    # ------------------------------------------------------------------ units
    def _point_at_placeholder(self, u: int) -> None:
        for i in self.unit_members[u]:
            p = self.params[i]
            p.data = self._nan.expand(p.shape)          # keeps the shape, owns no memory; a stray read shows as NaN
            if hasattr(p, "main_grad"):
                del p.main_grad

    def materialise(self, u: int, wait: bool = True) -> None:
        """Brings unit ``u`` into a transient buffer (one broadcast per owning rank). ``wait=False`` only starts it."""
        if u not in self._live:
            a, b = self.unit_range[u]
            buf = torch.empty(b - a, dtype=self.dtype, device=self.device)
            works = []
            lo0 = self.shard_range[0]
            for o, lo, hi in self._pieces(a, b):
                view = buf[lo - a:hi - a]
                if o == self.rank:
                    view.copy_(self.param_shard[lo - lo0:hi - lo0])
                if self.world_size > 1:
                    works.append(dist.broadcast(view, src=self.group_ranks[o], group=self.group, async_op=True))
            self._live[u] = (buf, works, False)
            self.peak_live_numel = max(self.peak_live_numel, sum(v[0].numel() for v in self._live.values()))
        if wait:
            buf, works, bound = self._live[u]
            for w in works:
                w.wait()
            if not bound:
                a = self.unit_range[u][0]
                for i in self.unit_members[u]:
                    p = self.params[i]
                    off = self.offsets[i] - a
                    p.data = buf[off:off + p.numel()].view(p.shape)
                self._live[u] = (buf, [], True)

    def release(self, u: int) -> None:
        if u in self._live:
            buf, works, _ = self._live.pop(u)
            for w in works:           # a prefetch nobody used: finish it before the buffer goes away
                w.wait()
            self._point_at_placeholder(u)

    def _open_grads(self, u: int) -> None:
        """fp32 gradient buffer of a unit whose backward is about to run; ``main_grad`` views for the kernels that
        accumulate weight gradients in place."""
        if self.grad_shard is None or u in self._gbuf:
            return
        a, b = self.unit_range[u]
        g = torch.zeros(b - a, dtype=self.grad_dtype, device=self.device)
        self._gbuf[u] = g
        for i in self.unit_members[u]:
            p = self.params[i]
            off = self.offsets[i] - a
            p.main_grad = g[off:off + p.numel()].view(p.shape)

    @torch.no_grad()
    def reduce_unit_grads(self, u: int) -> None:
        """Sums the unit's gradients over the group into their owners' ``grad_shard``. The collectives are started
        here and finished by :meth:`drain` (at the latest before the optimizer step), so they overlap what follows."""
        g = self._gbuf.pop(u, None)
        if g is None:
            return
        a, b = self.unit_range[u]
        for i in self.unit_members[u]:
            p = self.params[i]
            if p.grad is not None:
                p.main_grad.add_(p.grad.to(self.grad_dtype))
                p.grad = None
        if self.grad_hook is not None:
            self.grad_hook([self.names[i] for i in self.unit_members[u]], [self.params[i] for i in self.unit_members[u]])
        for i in self.unit_members[u]:
            p = self.params[i]
            if hasattr(p, "main_grad"):
                del p.main_grad
        self.drain(keep=1)                                 # at most two units' gradient buffers alive
        pieces = self._pieces(a, b)
        works = []
        if self.world_size > 1:
            for o, lo, hi in pieces:
                works.append(dist.reduce(g[lo - a:hi - a], dst=self.group_ranks[o], group=self.group, async_op=True))
        self._reducing.append((works, g, pieces, a))

    @torch.no_grad()
    def drain(self, keep: int = 0) -> None:
        """Finishes reductions in flight (all but the newest ``keep``) and adds this rank's pieces to ``grad_shard``."""
        lo0 = self.shard_range[0]
        while len(self._reducing) > keep:
            works, g, pieces, a = self._reducing.pop(0)
            for w in works:
                w.wait()
            for o, lo, hi in pieces:
                if o == self.rank:
                    self.grad_shard[lo - lo0:hi - lo0].add_(g[lo - a:hi - a])

    # ------------------------------------------------------------------ protocol of a micro-batch
    def begin(self, train: bool) -> None:
        """Before the forward of a micro-batch: the root unit (embedding, final norm, heads) stays for all of it."""
        self._root_users += 1
        self.materialise(0)
        if train:
            self._open_grads(0)
        if self.prefetch and self.n_units > 1:
            self.materialise(1, wait=False)

    def end(self, train: bool) -> None:
        """After the backward (or the forward of a forward-only pass) of a micro-batch."""
        self._root_users -= 1
        if train:
            self.reduce_unit_grads(0)
        if self._root_users <= 0:
            for u in list(self._live):
                self.release(u)
            for u in list(self._gbuf):        # a unit whose backward never ran (unused layer): nothing to reduce
                self.reduce_unit_grads(u)
            self._root_users = 0

    def enter(self, layer: int, *tensors):
        """Called by the model in front of decoder layer ``layer`` with the tensors that flow into it."""
        live = tuple(t for t in tensors if t is not None)
        if torch.is_grad_enabled() and any(t.requires_grad for t in live):
            out = iter(_Enter.apply(self, layer + 1, *live))
            return tuple(next(out) if t is not None else None for t in tensors)
        self._fwd_enter(layer + 1)
        return tensors

    def leave(self, layer: int, *tensors):
        live = tuple(t for t in tensors if t is not None)
        if torch.is_grad_enabled() and any(t.requires_grad for t in live):
            out = iter(_Leave.apply(self, layer + 1, *live))
            return tuple(next(out) if t is not None else None for t in tensors)
        self._fwd_leave(layer + 1)
        return tensors

    def _fwd_enter(self, u: int) -> None:
        self.materialise(u)
        if self.prefetch and u + 1 < self.n_units:
            self.materialise(u + 1, wait=False)

    def _fwd_leave(self, u: int) -> None:
        self.release(u)

    def _bwd_enter(self, u: int) -> None:
        self.materialise(u)
        self._open_grads(u)
        if self.prefetch and u - 1 >= 1:
            self.materialise(u - 1, wait=False)

    def _bwd_leave(self, u: int) -> None:
        self.reduce_unit_grads(u)
        self.release(u)

    # ------------------------------------------------------------------ optimizer-facing
    def zero_grad(self) -> None:
        self.drain()
        if self.grad_shard is not None:
            self.grad_shard.zero_()
        for p in self.params:
            p.grad = None

    def fold_autograd_grads(self) -> None:
        """Gradients are folded unit by unit as the backward leaves a unit; only reductions in flight remain."""
        self.drain()

    # ------------------------------------------------------------------ whole tensors in and out
    @torch.no_grad()
    def full_tensors(self, to_cpu: bool = False) -> Iterator[tuple[str, torch.Tensor]]:
        """(name, full tensor) of every parameter, one unit in memory at a time. A collective of the group."""
        for u in range(self.n_units):
            held = u in self._live
            self.materialise(u)
            for i in self.unit_members[u]:
                t = self.params[i].detach()
                yield self.names[i], (t.to("cpu", copy=True) if to_cpu else t.clone())
            if not held:
                self.release(u)

    @torch.no_grad()
    def write_piece(self, name: str, expert: Optional[int], rows: Optional[tuple[int, int]], tensor: torch.Tensor) -> None:
        """Stores part of a parameter: expert ``expert`` of a stacked tensor and / or rows ``rows`` of it (the pieces a
        checkpoint in another naming keeps as separate tensors). Every rank keeps what falls into its shard."""
        i = self.names.index(name)
        shape = tuple(self.params[i].shape)
        off = self.offsets[i]
        if expert is not None:
            per = 1
            for d in shape[1:]:
                per *= d
            off += expert * per
            shape = shape[1:]
        row = 1
        for d in shape[1:]:
            row *= d
        want = shape
        if rows is not None:
            off += rows[0] * row
            want = (rows[1] - rows[0],) + tuple(shape[1:])
        if tuple(tensor.shape) != tuple(want):
            raise ValueError(f"shape mismatch for {name}: checkpoint {tuple(tensor.shape)} vs model {tuple(want)}")
        self._write_flat(off, tensor.reshape(-1).to(self.device))

    @torch.no_grad()
    def write_full(self, name: str, tensor: torch.Tensor) -> None:
        """Stores a full tensor: every rank keeps the part that falls into its shard."""
        i = self.names.index(name)
        if tensor.numel() != self.params[i].numel():
            raise ValueError(f"{name}: expected {self.params[i].numel()} elements, got {tensor.numel()}")
        self._write_flat(self.offsets[i], tensor.reshape(-1).to(self.device))
