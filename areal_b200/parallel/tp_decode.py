"""Tensor-parallel inference without library collectives: the row-parallel projections of a
layer (``o_proj``, ``down_proj``) hand their partial result to every rank of the group from
inside the GEMM epilogue (peer stores over NVLink, ``ab2_gemm_bf16_bcast``), and the sum over
ranks happens in the kernel that also adds the residual stream and applies the next RMSNorm
(``ab2_tp_reduce_rmsnorm``). A decode step of a tensor-parallel replica is then a plain
sequence of kernels on one stream, so it is captured in a CUDA graph like the single-GPU step.

Buffers: two alternating sets of ``[P, max_rows, H]`` bf16 receive slots in symmetric memory
plus, per set, an arrival counter (written by all ranks) and a private consumed-count word.
Counters only grow and the consumed count lives on the device, so a graph replay needs no
host-side argument update. The protocol and why two sets are enough are described at the top
of ``ops/csrc/tp_decode.cu``.

This is the role of the tensor-parallel all-reduce inside the SGLang / vLLM servers of the
reference (``areal/engine/sglang_remote.py:255-337`` launches them with ``tp_size``).

Single-GPU emulation (``TPDecodeExchange.emulated``): the "ranks" are slices of one device's
memory and the caller runs the producers of all ranks before any consumer; used by the tests
that must run where only one GPU is visible.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from ..ops import lib as oplib
from .symm import ptr_array


class PendingSum:
    """Partial products that are on their way into every rank's receive slots: the value is
    ``sum over ranks`` and only exists once :meth:`TPDecodeExchange.reduce_rmsnorm` ran."""

    __slots__ = ("ex", "set_idx", "rows")

    def __init__(self, ex: "TPDecodeExchange", set_idx: int, rows: int):
        self.ex, self.set_idx, self.rows = ex, set_idx, rows


class TPDecodeExchange:
    def __init__(self, group, device, hidden: int, max_rows: int, timeout_ms: int = 20000):
        import torch.distributed as dist

        from .symm import symm_empty

        self.group = group
        self.P = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.H, self.max_rows, self.device = hidden, max_rows, torch.device(device)
        self.timeout_ms = timeout_ms
        if self.P > 8:
            raise ValueError("at most 8 tensor-parallel ranks")
        self.slot_stride = max_rows * hidden
        # receive slots: [set][source rank][row][H]
        self.slots, hdl = symm_empty(2 * self.P * self.slot_stride, torch.bfloat16, self.device, group)
        self.counters, chdl = symm_empty(2 * 2, torch.int64, self.device, group)     # [set] arrival counter (+ padding)
        self.state = torch.zeros(2, 2, dtype=torch.int64, device=self.device)       # [set] {consumed, CTA ticket}
        self.slots.zero_()
        self.counters.zero_()
        torch.cuda.synchronize(self.device)
        dist.barrier(group=group)
        slot_ptrs, cnt_ptrs = list(hdl.buffer_ptrs), list(chdl.buffer_ptrs)
        self._finish(slot_ptrs, cnt_ptrs)

    def _finish(self, slot_ptrs, cnt_ptrs):
        P, eb = self.P, 2
        self._dst = [ptr_array([slot_ptrs[r] + ((s * P + self.rank) * self.slot_stride) * eb for r in range(P)]) for s in range(2)]
        self._cnt = [ptr_array([cnt_ptrs[r] + s * 16 for r in range(P)]) for s in range(2)]
        self._calls = 0

    @classmethod
    def emulated(cls, n_ranks: int, device, hidden: int, max_rows: int, timeout_ms: int = 2000) -> list["TPDecodeExchange"]:
        """``n_ranks`` exchanges that live on ONE device and address each other's buffers as if
        they were peers. The caller must issue the producers of all ranks before a consumer."""
        outs = []
        slot_bufs = [torch.zeros(2 * n_ranks * max_rows * hidden, dtype=torch.bfloat16, device=device) for _ in range(n_ranks)]
        cnt_bufs = [torch.zeros(4, dtype=torch.int64, device=device) for _ in range(n_ranks)]
        for r in range(n_ranks):
            ex = cls.__new__(cls)
            ex.group, ex.P, ex.rank = None, n_ranks, r
            ex.H, ex.max_rows, ex.device, ex.timeout_ms = hidden, max_rows, torch.device(device), timeout_ms
            ex.slot_stride = max_rows * hidden
            ex.slots, ex.counters = slot_bufs[r], cnt_bufs[r]
            ex.state = torch.zeros(2, 2, dtype=torch.int64, device=device)
            ex._finish([b.data_ptr() for b in slot_bufs], [c.data_ptr() for c in cnt_bufs])
            outs.append(ex)
        return outs

    # ------------------------------------------------------------------ producer
    def linear_bcast(self, x: torch.Tensor, w: torch.Tensor) -> PendingSum:
        """``x @ w^T`` of this rank stored into slot ``rank`` of every rank's current set."""
        assert x.dim() == 2 and x.dtype == torch.bfloat16 and x.stride(1) == 1 and w.stride(1) == 1
        M, K = x.shape
        N = w.shape[0]
        if N != self.H or M > self.max_rows:
            raise ValueError(f"product of shape [{M}, {N}] does not fit the exchange ([<= {self.max_rows}, {self.H}])")
        s = self._calls & 1
        self._calls += 1
        rc = oplib.get_lib().ab2_gemm_bf16_bcast(x.data_ptr(), w.data_ptr(), self._dst[s], self._cnt[s], self.P, M, N, K,
                                                 x.stride(0), w.stride(0), N, 0, oplib.stream_ptr())
        oplib.check(rc, "ab2_gemm_bf16_bcast")
        return PendingSum(self, s, M)

    # ------------------------------------------------------------------ consumer
    def reduce_rmsnorm(self, pending: PendingSum, w: torch.Tensor, eps: float, resid: Optional[torch.Tensor]):
        """``(RMSNorm(sum + resid) * w, sum + resid)`` once all ranks' partials have arrived."""
        s, M, H = pending.set_idx, pending.rows, self.H
        x = torch.empty(M, H, dtype=torch.bfloat16, device=self.device)
        new_resid = torch.empty(M, H, dtype=torch.bfloat16, device=self.device)
        slots = self.slots.data_ptr() + s * self.P * self.slot_stride * 2
        rc = oplib.get_lib().ab2_tp_reduce_rmsnorm(slots, self.P, self.slot_stride, oplib.ptr(resid), new_resid.data_ptr(),
                                                   x.data_ptr(), w.data_ptr(), float(eps), M, H,
                                                   self.counters.data_ptr() + s * 16, self.state[s].data_ptr(),
                                                   int(self.timeout_ms), oplib.stream_ptr())
        oplib.check(rc, "ab2_tp_reduce_rmsnorm")
        return x, new_resid


def install_tp_decode(model, exchange: TPDecodeExchange) -> None:
    """Makes the row-parallel projections of every dense layer use ``exchange`` in inference."""
    for layer in model.layers:
        layer.tp_exchange = exchange
        layer.self_attn.tp_exchange = exchange
        layer.mlp.tp_exchange = exchange
    model.tp_exchange = exchange


def supports_fused_tp(model) -> bool:
    from ..models.decoder import DecoderLayer, DenseMLP

    return all(isinstance(l, DecoderLayer) and isinstance(l.mlp, DenseMLP) for l in model.layers) and \
        not getattr(model.cfg, "rms_norm_offset", False)
