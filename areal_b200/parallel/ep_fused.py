"""Expert parallelism with the dispatch and the combine fused into one peer-memory kernel each.

The NCCL dispatcher of ``parallel/ep.py`` runs, per MoE layer and direction, a row gather, a
variable-split all-to-all and a regroup by local expert (and the mirror image on the way back,
followed by the gate weighting and a scatter-add). Here every rank first learns the full
``[ep, E]`` count matrix (one small all-gather, the only library collective left), derives for
each of its routed rows the owning rank and the row's final position in that rank's
expert-sorted receive buffer, and then

* ``ab2_ep_dispatch`` reads ``x[token_of[i]]`` and stores it over NVLink straight into that
  position (gather + transfer + regroup in one pass);
* the expert GEMMs run on the receive buffer as it is (rows grouped by local expert);
* ``ab2_ep_combine`` pulls the ``k`` expert outputs of each token from the owning ranks, weights
  them with the gate values and sums them in fp32 (transfer + inverse regroup + weighting +
  scatter-add in one pass).

The backward of a dispatch is a combine with unit weights; the backward of a combine is a
dispatch scaled by the gate weights that also yields the gate-weight gradients. Ordering between
ranks comes from the bounded device barrier of :class:`SymmComm` between the writes and the reads
of a phase; buffers alternate between two symmetric slabs by phase so that a rank that is one
phase ahead never overwrites rows a slower peer is still reading.

Reference behaviour: ``areal/experimental/models/archon/expert_parallel.py`` (token dispatcher
:131-240) and the DeepEP option of ``areal/api/cli_args.py`` (``moe_enable_deepep``).
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist

from ..ops import lib as oplib

c_void_p, c_int, c_ll = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
oplib.declare("ab2_ep_dispatch", [c_void_p, c_ll] + [c_void_p] * 7 + [c_int, c_ll, c_int, c_int, c_ll, c_void_p])
oplib.declare("ab2_ep_combine", [c_void_p, c_int, c_ll] + [c_void_p] * 5 + [c_ll, c_void_p, c_int, c_int, c_int, c_ll, c_void_p])


@dataclass
class DispatchPlan:
    """Row maps of one MoE layer call on one rank (device tensors are int32)."""

    token_of: torch.Tensor      # [N] source token of sorted row i
    inv: torch.Tensor           # [T*k] sorted row of slot (t, j)
    drank: torch.Tensor         # [N] owning rank of sorted row i
    drow: torch.Tensor          # [N] row in the owner's receive buffer
    n_tokens: int
    top_k: int
    n_recv: int                 # rows this rank receives
    per_expert: list            # rows per local expert (all sources)
    max_recv: int               # largest n_recv over the group (the same on every rank)


def build_plan(counts_all: torch.Tensor, order: torch.Tensor, sorted_experts: torch.Tensor, me: int, top_k: int,
               counts_host: Optional[list] = None) -> DispatchPlan:
    """``counts_all`` [ep, E]: routed rows per (source rank, global expert); ``order`` [N]: the
    stable argsort of this rank's flat expert choices; ``sorted_experts`` = choices[order].

    The owner of expert g is rank g // El. Its receive buffer is ordered by (local expert,
    source rank), so rows of expert g coming from rank s start at
    ``sum_{g' < g, same owner} tot[g'] + sum_{s' < s} counts_all[s', g]``."""
    ep, E = counts_all.shape
    El = E // ep
    N = order.numel()
    dev = order.device
    tot = counts_all.sum(0)                                            # [E]
    tot_r = tot.view(ep, El)
    base_e = (tot_r.cumsum(1) - tot_r).reshape(E)                      # start of expert g in its owner's buffer
    pre = counts_all.cumsum(0) - counts_all                            # [ep, E] rows of g from lower ranks
    dst_base = base_e + pre[me]
    mine = counts_all[me]
    start = mine.cumsum(0) - mine                                      # start of expert g in my sorted list
    se = sorted_experts.long()
    drow = (dst_base[se] + torch.arange(N, device=dev) - start[se]).to(torch.int32)
    drank = (se // El).to(torch.int32)
    inv = torch.empty(N, dtype=torch.int32, device=dev)
    inv[order] = torch.arange(N, dtype=torch.int32, device=dev)
    host = counts_host if counts_host is not None else counts_all.tolist()
    per_rank_recv = [sum(host[s][r * El + e] for s in range(ep) for e in range(El)) for r in range(ep)]
    per_expert = [sum(host[s][me * El + e] for s in range(ep)) for e in range(El)]
    return DispatchPlan(token_of=(order // top_k).to(torch.int32), inv=inv, drank=drank, drow=drow, n_tokens=N // top_k,
                        top_k=top_k, n_recv=per_rank_recv[me], per_expert=per_expert, max_recv=max(per_rank_recv))


# ---------------------------------------------------------------- plain-torch statements of the two kernels
def dispatch_reference(src, plan: DispatchPlan, bufs: list, scale=None, ys=None):
    """What ``ab2_ep_dispatch`` does, on a list of per-rank buffers [rows, H] in one process."""
    rows = src[plan.token_of.long()].float()
    dw = (rows * ys.float()).sum(-1) if ys is not None else None
    if scale is not None:
        rows = (rows.to(src.dtype).float() * scale.float().unsqueeze(-1))
    rows = rows.to(src.dtype)
    for r, buf in enumerate(bufs):
        sel = plan.drank == r
        buf[plan.drow[sel].long()] = rows[sel]
    return dw


def combine_reference(bufs: list, plan: DispatchPlan, w=None, save=False):
    """What ``ab2_ep_combine`` does, on a list of per-rank buffers in one process."""
    N = plan.drank.numel()
    H = bufs[0].shape[1]
    ys = torch.zeros(N, H, dtype=bufs[0].dtype, device=bufs[0].device)
    for r, buf in enumerate(bufs):
        sel = plan.drank == r
        ys[sel] = buf[plan.drow[sel].long()]
    wt = w.float() if w is not None else torch.ones(N, device=ys.device)
    per_slot = (ys.float() * wt.unsqueeze(-1))[plan.inv.long()]        # [T*k, H] in slot order
    out = per_slot.view(plan.n_tokens, plan.top_k, H).sum(1).to(ys.dtype)
    return (out, ys) if save else (out, None)


# ---------------------------------------------------------------- symmetric buffers
class FusedEPComm:
    """Two symmetric slabs of ``capacity_rows x hidden`` bf16 per rank, the signal pads and the
    phase counter. One instance serves every MoE layer of a model."""

    HEADROOM = 1.25
    MAX_BYTES = 16 << 30       # per slab; beyond this the caller falls back to the library all-to-all

    def __init__(self, group, device, hidden: int, capacity_rows: int = 0):
        from .symm import SymmComm

        self.group, self.device, self.hidden = group, device, hidden
        self.comm = SymmComm(group, device)
        self.world, self.rank = self.comm.world, self.comm.rank
        self.capacity = 0
        self.slabs: list = []
        self.phase = 0
        if capacity_rows:
            self.reserve(capacity_rows)

    def fits(self, rows: int) -> bool:
        return int(rows * self.HEADROOM) * self.hidden * 2 <= self.MAX_BYTES

    def reserve(self, rows: int) -> None:
        """Collective over the group: every rank calls it with the same ``rows``."""
        if rows <= self.capacity:
            return
        from .symm import ptr_array, symm_empty

        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)                  # nobody still reads the old slabs
        cap = max(1024, int(rows * self.HEADROOM))
        self.slabs = []
        for _ in range(2):
            t, hdl = symm_empty(cap * self.hidden, torch.bfloat16, self.device, self.group)
            self.slabs.append((t, hdl, ptr_array(list(hdl.buffer_ptrs))))
        self.capacity = cap

    def next_slab(self):
        self.phase += 1
        return self.slabs[self.phase & 1]

    def barrier(self) -> None:
        self.comm.barrier(channel=1)


def _dispatch(comm: FusedEPComm, src, plan: DispatchPlan, slab, scale=None, ys=None):
    dw = torch.empty(plan.drank.numel(), dtype=torch.float32, device=src.device) if ys is not None else None
    rc = oplib.get_lib().ab2_ep_dispatch(src.data_ptr(), src.stride(0), plan.token_of.data_ptr(), plan.drank.data_ptr(),
                                         plan.drow.data_ptr(), oplib.ptr(scale), oplib.ptr(ys), oplib.ptr(dw), slab[2],
                                         comm.world, 0, plan.drank.numel(), comm.hidden, comm.capacity, oplib.stream_ptr())
    oplib.check(rc, "ab2_ep_dispatch")
    return dw


def _combine(comm: FusedEPComm, plan: DispatchPlan, slab, w=None, save=False, dtype=torch.bfloat16):
    out = torch.empty(plan.n_tokens, comm.hidden, dtype=dtype, device=comm.device)
    ys = torch.empty(plan.drank.numel(), comm.hidden, dtype=dtype, device=comm.device) if save else None
    rc = oplib.get_lib().ab2_ep_combine(slab[2], comm.world, 0, plan.inv.data_ptr(), plan.drank.data_ptr(), plan.drow.data_ptr(),
                                        oplib.ptr(w), out.data_ptr(), out.stride(0), oplib.ptr(ys), plan.n_tokens, plan.top_k,
                                        comm.hidden, comm.capacity, oplib.stream_ptr())
    oplib.check(rc, "ab2_ep_combine")
    return out, ys


class _FusedDispatch(torch.autograd.Function):
    """x [T, H] -> this rank's received rows [n_recv, H], grouped by local expert."""

    @staticmethod
    def forward(ctx, x, comm: FusedEPComm, plan: DispatchPlan, keep: bool):
        ctx.comm, ctx.plan = comm, plan
        x = x if x.stride(1) == 1 else x.contiguous()
        slab = comm.next_slab()
        _dispatch(comm, x, plan, slab)
        comm.barrier()
        got = slab[0][: plan.n_recv * comm.hidden].view(plan.n_recv, comm.hidden)
        # the slab is rewritten two phases later; what autograd keeps for the weight gradients must be private
        return got.clone() if keep else got

    @staticmethod
    def backward(ctx, g):
        comm, plan = ctx.comm, ctx.plan
        slab = comm.next_slab()
        if plan.n_recv:
            slab[0][: plan.n_recv * comm.hidden].view(plan.n_recv, comm.hidden).copy_(g)
        comm.barrier()
        dx, _ = _combine(comm, plan, slab, dtype=g.dtype)
        return dx, None, None, None


class _FusedCombine(torch.autograd.Function):
    """expert outputs [n_recv, H] (+ gate weights per sorted row) -> combined tokens [T, H]."""

    @staticmethod
    def forward(ctx, ys_local, w, comm: FusedEPComm, plan: DispatchPlan):
        slab = comm.next_slab()
        if plan.n_recv:
            slab[0][: plan.n_recv * comm.hidden].view(plan.n_recv, comm.hidden).copy_(ys_local)
        comm.barrier()
        need = ctx.needs_input_grad[0] or ctx.needs_input_grad[1]
        out, ys = _combine(comm, plan, slab, w=w, save=need, dtype=ys_local.dtype)
        ctx.comm, ctx.plan = comm, plan
        if need:
            ctx.save_for_backward(w, ys)
        return out

    @staticmethod
    def backward(ctx, dout):
        comm, plan = ctx.comm, ctx.plan
        w, ys = ctx.saved_tensors
        dout = dout if dout.stride(1) == 1 else dout.contiguous()
        slab = comm.next_slab()
        dw = _dispatch(comm, dout, plan, slab, scale=w, ys=ys)
        comm.barrier()
        # consumed by the expert GEMM backward before this slab's turn comes again (two phases on)
        g = slab[0][: plan.n_recv * comm.hidden].view(plan.n_recv, comm.hidden)
        return g, dw, None, None


class FusedExpertDispatcher:
    """Installed as ``MoEMLP.ep_dispatcher`` in place of the NCCL dispatcher; ``fused_forward``
    takes the routing result and returns the combined expert output of every token."""

    def __init__(self, group, ep_rank: int, ep_size: int, comm: FusedEPComm, fallback):
        self.group, self.ep_rank, self.ep_size, self.comm, self.fallback = group, ep_rank, ep_size, comm, fallback
        self.last_recv_tokens = 0
        self.fused_calls = 0

    def __call__(self, mlp, xs, sorted_experts):
        return self.fallback(mlp, xs, sorted_experts)

    def fused_forward(self, mlp, x, order, flat_e, topw) -> Optional[torch.Tensor]:
        """Returns None when this call has to take the library path (receive buffers would not
        fit); the decision depends only on the gathered counts, so every rank takes the same one."""
        E, ep, k = mlp.cfg.num_experts, self.ep_size, mlp.cfg.num_experts_per_tok
        counts = torch.bincount(flat_e, minlength=E)
        gathered = torch.empty(ep, E, dtype=counts.dtype, device=counts.device)
        dist.all_gather_into_tensor(gathered, counts, group=self.group)
        host = gathered.tolist()                                  # host sync: the expert GEMMs need the group sizes
        plan = build_plan(gathered, order, flat_e[order], self.ep_rank, k, counts_host=host)
        if not self.comm.fits(plan.max_recv):
            return None
        self.comm.reserve(plan.max_recv)
        self.last_recv_tokens = plan.n_recv
        self.fused_calls += 1
        got = _FusedDispatch.apply(x, self.comm, plan, torch.is_grad_enabled())
        ys_local = mlp.experts_forward(got, plan.per_expert, first_expert=0)
        w = topw.reshape(-1)[order].float()
        return _FusedCombine.apply(ys_local, w, self.comm, plan)


def install_fused_dispatch(model, group, ep_rank: int, ep_size: int, device) -> Optional[FusedEPComm]:
    """Wraps the dispatcher of every expert-parallel MoE layer of ``model``. Returns the shared
    communicator (None when the hidden size does not allow 16-byte row vectors)."""
    hidden = model.cfg.hidden_size
    if hidden % 8 or model.cfg.num_experts_per_tok > 32:
        return None
    comm = FusedEPComm(group, device, hidden)
    for layer in model.layers:
        mlp = layer.mlp
        if getattr(mlp, "ep_dispatcher", None) is not None:
            mlp.ep_dispatcher = FusedExpertDispatcher(group, ep_rank, ep_size, comm, mlp.ep_dispatcher)
    return comm
