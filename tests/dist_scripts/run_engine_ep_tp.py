"""Train-engine parity with expert parallelism folded into tensor parallelism (4 gloo ranks) against a single-rank
engine on the same global batch of a tiny MoE model. ``EP_TP_BACKEND`` picks the layout:

* ``native:d2t2e2`` - attention and dense parts tensor parallel, WHOLE experts spread over data x tensor ranks (each
  tensor-parallel rank routes its own share of the replica's tokens);
* ``native:(attn:d2t2|ffn:e2t2)`` - experts sliced over the tensor-parallel group as well and spread over the data ranks.

Prints ENGINE_EP_TP_OK per rank."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
os.environ["AREAL_FORCE_CPU"] = "1"

from run_engine_ep import cfg_of, loss_fn, make_batch, weight_fn  # noqa: E402

from areal_b200.api.io_struct import SaveLoadMeta  # noqa: E402
from areal_b200.engine.train_engine import B200TrainEngine  # noqa: E402
from areal_b200.models import hf_io  # noqa: E402
from areal_b200.models.config import preset  # noqa: E402
from areal_b200.models.decoder import build_model  # noqa: E402
from areal_b200.parallel import tp as TP  # noqa: E402


def main():
    dist.init_process_group("gloo")
    rank = dist.get_rank()
    backend = os.environ["EP_TP_BACKEND"]
    whole = "ffn" not in backend
    mc = preset(os.environ.get("EP_TP_MODEL", "tiny-qwen3-moe"))
    eng = B200TrainEngine(cfg_of(backend))
    eng.create_process_group()
    eng.initialize(model_config=mc, seed=5)
    assert (eng.tp_size, eng.dp_size, eng.ep_size) == (2, 2, 2) and eng.etp_size == (1 if whole else 2), (eng.tp_size, eng.dp_size, eng.ep_size, eng.etp_size)
    assert eng.tp_rank == rank % 2 and eng.dp_rank == rank // 2
    if whole:
        assert eng.ep_rank == rank % 2 and eng._n_edp == 2 and eng.model.layers[0].moe_row_share is not None
        assert eng.model.layers[0].mlp.w_gate_up.shape[1] == 2 * mc.moe_intermediate_size
    else:
        assert eng.ep_rank == rank // 2 and eng._n_edp == 1 and eng.model.layers[0].moe_row_share is None
        assert eng.model.layers[0].mlp.w_gate_up.shape[1] == mc.moe_intermediate_size
    batch = make_batch(mc.vocab_size)
    per = 8 // eng.dp_size
    mine = {k: v[eng.dp_rank * per:(eng.dp_rank + 1) * per] for k, v in batch.items()}       # tensor-parallel peers see the same rows
    stats = [eng.train_batch(mine, loss_fn, weight_fn) for _ in range(2)]
    ref = B200TrainEngine(cfg_of("d1"))
    ref.set_train_ranks([rank])
    ref.create_process_group()
    ref.initialize(model_config=mc, seed=5)
    rstats = [ref.train_batch(batch, loss_fn, weight_fn) for _ in range(2)]
    for a, b in zip(stats, rstats):
        assert abs(a["grad_norm"] - b["grad_norm"]) < 2e-3 * max(1.0, b["grad_norm"]), (a, b)
    full = {n: p.detach() for n, p in ref.model.named_parameters()}
    El = mc.num_experts // 2
    worst = 0.0
    for n, p in eng.model.named_parameters():
        want = TP.shard_tensor(mc, n, full[n], 2, eng.tp_rank, expert_tp=not whole)
        if n in eng._expert_param_names:
            want = want[eng.ep_rank * El:(eng.ep_rank + 1) * El]
        diff = (p.detach() - want).abs()
        worst = max(worst, diff.max().item())
        # (Adam turns rounding-level gradient differences into O(lr) steps: a handful of elements cannot average them out)
        assert (diff.mean().item() < 2e-5 or p.numel() < 64) and diff.max().item() < 5e-3, f"weights diverged for {n}: max {diff.max().item()}"
    path = os.environ["EP_SAVE_DIR"]
    eng.save(SaveLoadMeta(path=path, weight_format="hf", with_optim=False))
    dist.barrier()
    m = build_model(mc, dtype=torch.float32, device="cpu", seed=0)
    hf_io.load_model_hf(m, path)
    for n, p in m.named_parameters():
        assert (p.detach() - full[n]).abs().max().item() < 5e-3, n
    w = eng.export_weights()
    assert set(w) == set(full) and all(w[n].shape == full[n].shape for n in w)
    for n in w:
        assert (w[n] - full[n]).abs().max().item() < 5e-3, n
    before = {n: p.detach().clone() for n, p in eng.model.named_parameters()}
    with torch.no_grad():
        for p in eng.model.parameters():
            p.zero_()
    eng.load(SaveLoadMeta(path=path, weight_format="hf", with_optim=False))
    for n, p in eng.model.named_parameters():
        assert torch.allclose(p.detach(), before[n], atol=1e-6), n
    third = eng.train_batch(mine, loss_fn, weight_fn)
    rthird = ref.train_batch(batch, loss_fn, weight_fn)
    assert abs(third["grad_norm"] - rthird["grad_norm"]) < 3e-3 * max(1.0, rthird["grad_norm"]), (third, rthird)
    if rank == 0:
        print(f"{backend}: grad norms {[round(s['grad_norm'], 4) for s in stats]} vs {[round(s['grad_norm'], 4) for s in rstats]}; "
              f"worst weight diff {worst:.2e}", flush=True)
    print("ENGINE_EP_TP_OK", flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
