"""Tensor-parallel products fused with their collective over NVLink peer memory.

``FusedTPLinear`` owns the symmetric staging buffers of one TP group and offers

* ``allgather_gemm(x_local, w)``: every rank contributes ``[T/P, K]`` rows; the result
  ``[T, N_local]`` is computed by ONE kernel whose TMA producer reads each row block from the
  GPU that owns it (``ab2_allgather_gemm``);
* ``gemm_reduce_scatter(x, w)``: ``[T, K_local] x [N, K_local]^T`` partial products are added
  tile by tile into the row owner's fp32 buffer by the GEMM epilogue (``ab2_gemm_reduce_scatter``)
  and come back as this rank's ``[T/P, N]`` rows.

Both are bracketed by the bounded device barrier of :class:`SymmComm`. The same two
primitives serve Megatron-style sequence-parallel TP in training (forward and input
gradients of column- and row-parallel layers) and TP decode on the rollout side. NCCL
equivalents (``all_gather_into_tensor`` + GEMM, GEMM + ``reduce_scatter_tensor``) are kept as
the measured baseline (``baseline_*``). Reference: ``areal/engine/fsdp_utils/parallel.py:227-385``.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch
import torch.distributed as dist

from ..ops import functional as OF
from ..ops import lib as oplib
from .symm import SymmComm, ptr_array, symm_empty

oplib.declare("ab2_allgather_gemm", [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p] + [ctypes.c_int] * 9 +
              [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p])
oplib.declare("ab2_gemm_reduce_scatter", [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p] + [ctypes.c_int] * 10 + [ctypes.c_void_p])


class FusedTPLinear:
    def __init__(self, group, device, max_rows_per_rank: int, max_k: int, max_n: int):
        self.group = group if group is not None else dist.group.WORLD
        self.device = device
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        if self.world > 8:
            raise ValueError("the fused tensor-parallel kernels address at most 8 peers")
        self.comm = SymmComm(self.group, device)
        # staging: this rank's activation rows (bf16) and its reduce-scatter target (fp32)
        self.x_buf, self.x_hdl = symm_empty(max_rows_per_rank * max_k, torch.bfloat16, device, self.group)
        self.o_buf, self.o_hdl = symm_empty(max_rows_per_rank * max_n, torch.float32, device, self.group)
        self.oh_buf, self.oh_hdl = symm_empty(max_rows_per_rank * max_n, torch.bfloat16, device, self.group)
        self.x_ptrs = list(self.x_hdl.buffer_ptrs)
        self.o_ptrs = list(self.o_hdl.buffer_ptrs)
        self.oh_ptrs = list(self.oh_hdl.buffer_ptrs)
        self.max_rows, self.max_k, self.max_n = max_rows_per_rank, max_k, max_n
        # copy-once gather: local landing buffer for the peers' rows + one ready flag per 128 rows
        self.gathered = torch.empty(max_rows_per_rank * self.world * max_k, dtype=torch.bfloat16, device=device)
        self.flags = torch.zeros(max_rows_per_rank * self.world // 128 + 1, dtype=torch.int32, device=device)
        self._epoch = 0

    # ------------------------------------------------------------------ fused
    def allgather_gemm(self, x_local: torch.Tensor, w: torch.Tensor, b_mn: bool = False, copy_once: bool = True) -> torch.Tensor:
        """``concat_ranks(x_local) @ w^T`` (``b_mn``: ``@ w``). x_local: [T/P, K] bf16 with T/P a
        multiple of 128. ``copy_once``: remote rows are brought over NVLink once by copy CTAs of
        the same kernel (default); otherwise every output tile loads them from the owner."""
        rows, K = x_local.shape
        N = w.shape[1] if b_mn else w.shape[0]
        assert rows % 128 == 0 and rows <= self.max_rows and K <= self.max_k and x_local.dtype == torch.bfloat16
        stage = self.x_buf[: rows * K].view(rows, K)
        stage.copy_(x_local)
        self.comm.barrier(0)                               # every rank's rows are in place
        M = rows * self.world
        y = torch.empty(M, N, device=self.device, dtype=torch.bfloat16)
        self._epoch += 1
        rc = oplib.get_lib().ab2_allgather_gemm(ptr_array(self.x_ptrs), w.data_ptr(), y.data_ptr(), M, N, K, K, w.stride(0),
                                                y.stride(0), int(b_mn), self.rank, self.world,
                                                self.gathered.data_ptr() if copy_once else None,
                                                self.flags.data_ptr() if copy_once else None, self._epoch, oplib.stream_ptr())
        oplib.check(rc, "ab2_allgather_gemm")
        self.comm.barrier(1)                               # peers finished reading before the stage is reused
        return y

    def gemm_reduce_scatter(self, x: torch.Tensor, w: torch.Tensor, b_mn: bool = False, out_dtype=torch.bfloat16,
                            reduce_dtype=torch.float32) -> torch.Tensor:
        """This rank's rows of ``sum_ranks(x_r @ w_r^T)``. x: [T, K_local] bf16, T/P a multiple
        of 128. Returns [T/P, N]. ``reduce_dtype=torch.bfloat16`` halves the NVLink bytes (every
        add rounds to bf16)."""
        M, K = x.shape
        N = w.shape[1] if b_mn else w.shape[0]
        rows = M // self.world
        assert M % self.world == 0 and rows % 128 == 0 and rows <= self.max_rows and N <= self.max_n
        half = reduce_dtype == torch.bfloat16
        out = (self.oh_buf if half else self.o_buf)[: rows * N].view(rows, N)
        out.zero_()
        self.comm.barrier(2)                               # every target is zeroed
        rc = oplib.get_lib().ab2_gemm_reduce_scatter(x.data_ptr(), w.data_ptr(), ptr_array(self.oh_ptrs if half else self.o_ptrs), M, N,
                                                     K, x.stride(0), w.stride(0), N, int(b_mn), self.rank, self.world, int(half),
                                                     oplib.stream_ptr())
        oplib.check(rc, "ab2_gemm_reduce_scatter")
        self.comm.barrier(3)                               # every rank's reductions have landed
        return out.to(out_dtype)

    # ------------------------------------------------------------------ NCCL baseline
    def baseline_allgather_gemm(self, x_local, w, b_mn: bool = False):
        full = torch.empty(x_local.shape[0] * self.world, x_local.shape[1], device=self.device, dtype=x_local.dtype)
        dist.all_gather_into_tensor(full, x_local.contiguous(), group=self.group)
        return OF.gemm(full, w, b_mn=b_mn)

    def baseline_gemm_only(self, x_local, w):
        """The local product alone (no communication): the floor for the fused forms."""
        full = self.gathered[: x_local.shape[0] * self.world * x_local.shape[1]].view(-1, x_local.shape[1])
        return OF.gemm(full, w)

    def baseline_gemm_reduce_scatter(self, x, w, b_mn: bool = False, out_dtype=torch.bfloat16):
        part = OF.gemm(x, w, b_mn=b_mn, epi=OF.EPI_F32)
        out = torch.empty(x.shape[0] // self.world, part.shape[1], device=self.device, dtype=torch.float32)
        dist.reduce_scatter_tensor(out, part, group=self.group)
        return out.to(out_dtype)


# --------------------------------------------------------------------------- Ulysses fused exchanges
oplib.declare("ab2_gemm_scatter_cols", [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p] + [ctypes.c_int] * 9 + [ctypes.c_void_p])
oplib.declare("ab2_gather_cols_gemm", [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p] + [ctypes.c_int] * 9 +
              [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p])


class FusedUlyssesLinear:
    """The two all-to-alls of Ulysses sequence parallelism folded into the neighbouring
    projections (one kernel each, peer memory over NVLink):

    * ``project_scatter(x_local, w)``: ``x_local[T/P, K] @ w[N, K]^T`` whose output columns
      (heads) are written by the GEMM epilogue straight into the rank that owns them; returns
      this rank's ``[T, N/P]`` block (all tokens, local heads) — QKV projection + seq->heads;
    * ``gather_project(o_full, w)``: ``o_full[T, K/P]`` (all tokens, local heads' outputs) ->
      ``[T/P, N]``: copy CTAs pull this rank's rows of every peer's panel once, the GEMM
      consumes them as they land — heads->seq + output projection.
    """

    def __init__(self, group, device, max_rows_per_rank: int, max_cols: int):
        self.group = group if group is not None else dist.group.WORLD
        self.device = device
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        if self.world > 8:
            raise ValueError("the fused kernels address at most 8 peers")
        self.comm = SymmComm(self.group, device)
        n = max_rows_per_rank * self.world * (max_cols // self.world + 64)
        # two landing buffers: projections scatter into ``s_buf``; attention outputs are staged in ``o_stage``
        self.s_buf, self.s_hdl = symm_empty(n, torch.bfloat16, device, self.group)
        self.o_stage, self.o_hdl = symm_empty(n, torch.bfloat16, device, self.group)
        self.s_ptrs, self.o_ptrs = list(self.s_hdl.buffer_ptrs), list(self.o_hdl.buffer_ptrs)
        self.gathered = torch.empty(max_rows_per_rank * max_cols, dtype=torch.bfloat16, device=device)
        self.flags = torch.zeros((max_rows_per_rank // 128 + 1) * self.world, dtype=torch.int32, device=device)
        self._epoch = 0
        self.max_rows, self.max_cols = max_rows_per_rank, max_cols

    def project_scatter(self, x_local: torch.Tensor, w: torch.Tensor, b_mn: bool = False) -> torch.Tensor:
        M, K = x_local.shape
        N = w.shape[1] if b_mn else w.shape[0]
        P = self.world
        assert N % P == 0 and (N // P) % 32 == 0 and M <= self.max_rows and N <= self.max_cols + 64 * P
        out = self.s_buf[: P * M * (N // P)].view(P * M, N // P)
        self.comm.barrier(4)                               # peers are done with the previous contents
        rc = oplib.get_lib().ab2_gemm_scatter_cols(x_local.data_ptr(), w.data_ptr(), ptr_array(self.s_ptrs), M, N, K, x_local.stride(0),
                                                   w.stride(0), N // P, int(b_mn), self.rank, P, oplib.stream_ptr())
        oplib.check(rc, "ab2_gemm_scatter_cols")
        self.comm.barrier(5)                               # every rank's tiles have landed here
        return out

    def gather_project(self, o_full: torch.Tensor, w: torch.Tensor, b_mn: bool = False) -> torch.Tensor:
        T, Kl = o_full.shape
        P = self.world
        M, K = T // P, Kl * P
        N = w.shape[1] if b_mn else w.shape[0]
        assert T % P == 0 and M % 128 == 0 and Kl % 64 == 0 and M <= self.max_rows and K <= self.max_cols
        stage = self.o_stage[: T * Kl].view(T, Kl)
        stage.copy_(o_full)
        self.comm.barrier(6)                               # every rank's panel is in place
        y = torch.empty(M, N, device=self.device, dtype=torch.bfloat16)
        self._epoch += 1
        rc = oplib.get_lib().ab2_gather_cols_gemm(ptr_array(self.o_ptrs), w.data_ptr(), y.data_ptr(), M, N, K, Kl, w.stride(0), y.stride(0),
                                                  int(b_mn), self.rank, P, self.gathered.data_ptr(), self.flags.data_ptr(), self._epoch,
                                                  oplib.stream_ptr())
        oplib.check(rc, "ab2_gather_cols_gemm")
        self.comm.barrier(7)                               # peers finished reading this rank's panel
        return y

    # NCCL baselines (projection + all_to_all_single)
    def baseline_project_scatter(self, x_local, w):
        P = self.world
        y = OF.gemm(x_local, w)                                                  # [M, N]
        M, N = y.shape
        send = y.view(M, P, N // P).permute(1, 0, 2).contiguous()               # [P(dst), M, N/P]
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=self.group)
        return recv.view(P * M, N // P)

    def baseline_gather_project(self, o_full, w):
        P = self.world
        T, Kl = o_full.shape
        M = T // P
        send = o_full.view(P, M, Kl).contiguous()                                # [P(dst rows), M, Kl]
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=self.group)                     # [P(src cols), M, Kl]
        a = recv.permute(1, 0, 2).reshape(M, P * Kl).contiguous()
        return OF.gemm(a, w)
