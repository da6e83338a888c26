"""GSPO (sequence-level importance ratios) under sequence parallelism over all ranks (Ulysses, or zig-zag context
parallelism with AREAL_TEST_CP_MODE=zigzag) equals the single-rank result."""
import os, sys
sys.path.insert(0, os.getcwd())
os.environ["AREAL_FORCE_CPU"] = "1"
import torch, torch.distributed as dist
from areal_b200.api.cli_args import MicroBatchSpec, OptimizerConfig, PPOActorConfig
from areal_b200.api.alloc_mode import FSDPParallelStrategy
from areal_b200.engine.train_engine import B200PPOActor
from areal_b200.models.config import preset
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
def run(sp):
    cfg = PPOActorConfig(init_from_scratch=True, dtype="float32", optimizer=OptimizerConfig(lr=1e-3, gradient_clipping=1.0),
                         mb_spec=MicroBatchSpec(max_tokens_per_mb=512), use_decoupled_loss=True, recompute_logprob=True, kl_ctl=0.0,
                         ppo_n_minibatches=1, importance_sampling_level="sequence", prox_logp_method="recompute")
    cfg.fsdp.context_parallel = os.environ.get("AREAL_TEST_CP_MODE", "ulysses")
    eng = B200PPOActor(cfg)
    if sp == 1:
        eng.set_train_ranks([rank], None)
    eng.create_process_group(FSDPParallelStrategy(data_parallel_size=1, context_parallel_size=sp) if sp > 1 else FSDPParallelStrategy())
    name = os.environ.get("AREAL_TEST_MODEL", "tiny-qwen2")
    eng.initialize(model_config=preset(name, vocab_size=64, **({"num_layers": 2} if name == "tiny-qwen2" else {})), seed=3)
    g = torch.Generator().manual_seed(0)
    B, L = 6, 40
    ids = torch.randint(0, 64, (B, L), generator=g)
    am = torch.ones(B, L, dtype=torch.bool)
    for i in range(B):
        am[i, L - 3 * i:] = False if i else True
    lm = torch.zeros(B, L, dtype=torch.int32); lm[:, 10:] = 1; lm = lm * am
    data = dict(input_ids=ids, attention_mask=am, loss_mask=lm, logprobs=torch.full((B, L), -4.0) + 0.1 * torch.randn(B, L, generator=g),
                versions=torch.zeros(B, L, dtype=torch.int32), rewards=torch.randn(B, generator=g))
    p0 = eng.store.flat_param[:eng.store.numel].clone()
    data["prox_logp"] = eng.compute_logp(data)
    eng.compute_advantages(data)
    st = eng.ppo_update(data)
    return st[0], eng.store.flat_param[:eng.store.numel].clone() - p0
s2, p2 = run(world)
s1, p1 = run(1)
assert abs(s1["grad_norm"] - s2["grad_norm"]) < 1e-4 * max(1, s1["grad_norm"]), (s1, s2)
# Adam divides by sqrt(v): elements whose gradient is numerically zero move by rounding noise, so compare the update as a whole
cos = float((p1 * p2).sum() / (p1.norm() * p2.norm()))
assert cos > 0.9999 and float((p1 - p2).abs().max()) < 2e-4, (cos, float((p1 - p2).abs().max()))
print("SP_GSPO_OK", rank, s1["grad_norm"], s2["grad_norm"], flush=True)
dist.barrier()
