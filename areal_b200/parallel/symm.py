"""Symmetric (peer-addressable) device memory for the fused communication kernels.

Allocation and handle exchange ride on ``torch.distributed._symmetric_memory`` (cuMem
allocations whose handles are exchanged among the ranks of a process group and mapped into
every process); this module wraps it into what the kernels need: per-rank raw pointers as a
``ctypes`` array, a zero-initialised signal pad and float pad per communicator, and a
bounded device-side barrier (flag exchange over NVLink with an error status on time-out
instead of a trap).

Takes the place of the NCCL communicator plumbing of the reference
(``areal/engine/core/distributed.py:82`` init_custom_process_group) for the data plane.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch
import torch.distributed as dist

from ..ops import lib as oplib

MAX_PEERS = 16
CHANNELS = 8

oplib.declare("ab2_signal_barrier", [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                     ctypes.c_void_p])
oplib.declare("ab2_rs_sumsq", [ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_longlong, ctypes.c_void_p,
                               ctypes.c_void_p, ctypes.c_float, ctypes.c_void_p])
oplib.declare("ab2_rs_sumsq_multimem", [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_void_p,
                                        ctypes.c_float, ctypes.c_void_p])
oplib.declare("ab2_norm_allreduce", [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                     ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p])
oplib.declare("ab2_adamw_push", [ctypes.c_void_p] * 5 + [ctypes.c_int, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_longlong] +
              [ctypes.c_float] * 5 + [ctypes.c_int, ctypes.c_void_p])
oplib.declare("ab2_push_copy", [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_longlong,
                                ctypes.c_void_p])


def ptr_array(ptrs) -> ctypes.Array:
    arr = (ctypes.c_void_p * len(ptrs))()
    for i, p in enumerate(ptrs):
        arr[i] = p
    return arr


def symm_empty(numel: int, dtype, device, group):
    """Allocates ``numel`` elements of symmetric memory and exchanges handles over ``group``.
    Returns (local tensor, handle); ``handle.buffer_ptrs[r]`` is rank r's buffer address as
    seen from this process."""
    import torch.distributed._symmetric_memory as symm

    t = symm.empty(numel, dtype=dtype, device=device)
    hdl = symm.rendezvous(t, group if group is not None else dist.group.WORLD)
    return t, hdl


class SymmComm:
    """Signal / float pads of one communicator plus the bounded barrier."""

    def __init__(self, group, device):
        self.group = group if group is not None else dist.group.WORLD
        self.device = device
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        if self.world > MAX_PEERS:
            raise ValueError(f"at most {MAX_PEERS} peers per communicator")
        self.pad, self.pad_hdl = symm_empty(CHANNELS * MAX_PEERS, torch.int32, device, self.group)
        self.fpad, self.fpad_hdl = symm_empty(MAX_PEERS, torch.float32, device, self.group)
        self.pad.zero_()
        self.fpad.zero_()
        torch.cuda.synchronize(device)
        dist.barrier(group=self.group)
        self.pad_ptrs = ptr_array(list(self.pad_hdl.buffer_ptrs))
        self.fpad_ptrs = ptr_array(list(self.fpad_hdl.buffer_ptrs))
        self._epoch = [0] * CHANNELS
        self.timeout_ms = 20000

    def next_epoch(self, channel: int) -> int:
        self._epoch[channel] += 1
        return self._epoch[channel]

    def barrier(self, channel: int = 0) -> None:
        """Device-side barrier on the current stream: every rank's prior work on its stream is
        visible to every peer's later work. A peer that never arrives makes the wait give up
        after ``timeout_ms`` and sets the kernel error word (read with ``ops.lib.kernel_error``)."""
        rc = oplib.get_lib().ab2_signal_barrier(self.pad_ptrs, self.rank, self.world, channel, self.next_epoch(channel),
                                                self.timeout_ms, oplib.stream_ptr())
        oplib.check(rc, "ab2_signal_barrier")
