"""ZeRO data parallelism without library collectives in the step.

After backward every rank holds the full fp32 gradient of its micro-batches in a symmetric
buffer. One kernel per rank then reads its shard from every peer (NVLink loads), sums,
scales and accumulates the squared-norm partial; the partials are exchanged by peer stores;
AdamW runs on the shard and writes the refreshed bf16 parameters directly into every peer's
parameter buffer (and, during weight sync, into rollout replicas). NCCL is not involved.

Replaces FSDP2 reduce-scatter / all-gather + fused AdamW + grad-norm all-reduces of the
reference (``areal/engine/fsdp_utils/parallel.py:388-396``, ``fsdp_utils/grad.py:112-232``,
``fsdp_engine.py:696-727``).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..ops import lib as oplib
from .symm import SymmComm, ptr_array


class FusedGradReducer:
    def __init__(self, store, group, grad_peer_ptrs: list, param_peer_ptrs: list, grad_multicast_ptr: int = 0):
        """``grad_multicast_ptr``: NVLS multicast address of the gradient buffer (0: none). With it the
        reduce-scatter is one ``multimem.ld_reduce`` per 16 bytes (sum formed inside the NVLink switch)
        instead of one load per peer."""
        self.store, self.group = store, group
        self.grad_mc = int(grad_multicast_ptr or 0)
        self.comm = SymmComm(group, store.device)
        self.world, self.rank = self.comm.world, self.comm.rank
        self.grad_ptrs = ptr_array(list(grad_peer_ptrs))
        self.param_ptrs = ptr_array(list(param_peer_ptrs))
        self.param_ptr_list = list(param_peer_ptrs)
        self.gshard = torch.empty(store.shard_numel, dtype=torch.float32, device=store.device)

    def reduce_scatter(self, state: torch.Tensor = None) -> torch.Tensor:
        """Sums this rank's shard over all peers into a local fp32 buffer. If ``state`` is given
        its first element receives the *global* squared norm (partials exchanged peer to peer)."""
        L = oplib.get_lib()
        self.comm.barrier(0)  # every peer finished writing its gradients
        lo = self.store.shard_range[0]
        st = state if state is not None else torch.zeros(4, dtype=torch.float32, device=self.store.device)
        if state is not None:
            st.zero_()
        if self.grad_mc:
            rc = L.ab2_rs_sumsq_multimem(self.grad_mc, lo, self.store.shard_numel, self.gshard.data_ptr(), st.data_ptr(), 1.0,
                                         oplib.stream_ptr())
            oplib.check(rc, "ab2_rs_sumsq_multimem")
        else:
            rc = L.ab2_rs_sumsq(self.grad_ptrs, self.world, lo, self.store.shard_numel, self.gshard.data_ptr(), st.data_ptr(),
                                1.0, oplib.stream_ptr())
            oplib.check(rc, "ab2_rs_sumsq")
        if state is not None:
            rc = L.ab2_norm_allreduce(self.comm.pad_ptrs, self.comm.fpad_ptrs, self.rank, self.world, 1,
                                      self.comm.next_epoch(1), st.data_ptr(), self.comm.timeout_ms, oplib.stream_ptr())
            oplib.check(rc, "ab2_norm_allreduce")
        return self.gshard

    def adamw_and_all_gather(self, opt, state: torch.Tensor, lr: float, extra_dst: list = ()) -> None:
        """Sharded AdamW whose bf16 output is stored into every trainer peer (and any extra
        destination buffers, e.g. rollout replicas laid out like the trainer's flat buffer)."""
        cfg = opt.cfg
        dst = ptr_array(self.param_ptr_list + list(extra_dst))
        rc = oplib.get_lib().ab2_adamw_push(opt.master.data_ptr(), opt.exp_avg.data_ptr(), opt.exp_avg_sq.data_ptr(),
                                            self.gshard.data_ptr(), dst, len(dst), self.store.shard_range[0],
                                            state.data_ptr(), self.store.shard_numel, lr, cfg.beta1, cfg.beta2, cfg.eps,
                                            cfg.weight_decay, opt.step_count, oplib.stream_ptr())
        oplib.check(rc, "ab2_adamw_push")
        self.comm.barrier(2)  # all shards landed everywhere before anyone reads parameters

    def all_gather_params(self) -> None:
        """Plain write-back of the local bf16 shard to every peer (used when the optimizer ran
        through the generic path)."""
        sh = self.store.param_shard
        rc = oplib.get_lib().ab2_push_copy(sh.data_ptr(), ptr_array(self.param_ptr_list), self.world,
                                           self.store.shard_range[0], sh.numel(), oplib.stream_ptr())
        oplib.check(rc, "ab2_push_copy")
        self.comm.barrier(2)
