"""2+ rank check of the peer-memory ZeRO step against the NCCL collective path.

Launched by tests/test_multi_gpu.py under torchrun. Every rank trains the same tiny model for
two steps on rank-specific data twice: once with the fused kernels (reduce-scatter by peer
loads, peer-exchanged norm, AdamW writing into every peer) and once with
reduce_scatter_tensor / all_reduce / all_gather_into_tensor. Parameters must agree between
the two runs and be identical on all ranks.
"""
import faulthandler
import os
import sys

faulthandler.dump_traceback_later(150, exit=True)
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import torch
import torch.distributed as dist

from areal_b200.api.cli_args import MicroBatchSpec, OptimizerConfig, PPOActorConfig
from areal_b200.engine.train_engine import B200PPOActor
from areal_b200.models.config import preset
from areal_b200.ops import lib as oplib


def batch(rank, B=4, L=200, V=1024):
    g = torch.Generator().manual_seed(100 + rank)
    ids = torch.randint(0, V, (B, L), generator=g)
    am = torch.ones(B, L, dtype=torch.bool)
    lm = torch.zeros(B, L, dtype=torch.int32)
    lm[:, 50:] = 1
    return dict(input_ids=ids, attention_mask=am, loss_mask=lm, logprobs=torch.full((B, L), -6.9),
                versions=torch.zeros(B, L, dtype=torch.int32), rewards=torch.randn(B, generator=g))


def run(fused: bool, in_switch: bool = False):
    cfg = PPOActorConfig(init_from_scratch=True, dtype="bfloat16", optimizer=OptimizerConfig(lr=1e-3, gradient_clipping=0.5),
                         mb_spec=MicroBatchSpec(max_tokens_per_mb=1024), use_decoupled_loss=True, recompute_logprob=True,
                         kl_ctl=0.0, ppo_n_minibatches=1)
    cfg.fsdp.fuse_reduce_scatter_adamw = fused
    cfg.fsdp.reduce_in_switch = in_switch
    e = B200PPOActor(cfg)
    e.create_process_group()
    e.initialize(model_config=preset("tiny-qwen3"), seed=7)
    stats = []
    for step in range(2):
        data = batch(dist.get_rank() + 10 * step)
        data["prox_logp"] = e.compute_logp(data)
        e.compute_advantages(data)
        stats.append(e.ppo_update(data)[0])
    torch.cuda.synchronize()
    return e.store.flat_param.float().clone(), stats, e


def main():
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl")
    pf, sf, ef = run(True)
    assert ef._grad_reducer is not None, "fused reducer was not installed"
    pn, sn, _ = run(False)
    err = oplib.kernel_error()
    assert err == 0, f"kernel error word {err}"
    rel = ((pf - pn).norm() / pn.norm()).item()
    gn = [(a["grad_norm"], b["grad_norm"]) for a, b in zip(sf, sn)]
    # identical on all ranks
    ref = pf.clone()
    dist.broadcast(ref, src=0)
    same = bool((ref == pf).all())
    print(f"rank {dist.get_rank()} rel_diff {rel:.3e} grad_norms {gn} identical_across_ranks {same}", flush=True)
    assert rel < 2e-3, rel
    assert same
    for a, b in gn:
        assert abs(a - b) / max(b, 1e-6) < 2e-2
    if os.environ.get("AREAL_TEST_NVLS_REDUCE", "0") == "1":
        # the same step with the gradient reduce-scatter formed inside the NVLink switch (multimem.ld_reduce)
        ps, ss, es = run(True, in_switch=True)
        used = bool(es._grad_reducer.grad_mc)
        rel_s = ((ps - pf).norm() / pf.norm()).item()
        print(f"rank {dist.get_rank()} in-switch reduce used {used} rel_diff_vs_peer_loads {rel_s:.3e} "
              f"grad_norms {[(a['grad_norm'], b['grad_norm']) for a, b in zip(ss, sf)]}", flush=True)
        assert oplib.kernel_error() == 0
        assert rel_s < 2e-3, rel_s
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
