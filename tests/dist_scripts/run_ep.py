"""Expert-parallel parity (gloo ranks on CPU): each rank feeds DIFFERENT tokens through a MoE
model whose experts are split over the ranks; outputs and gradients must equal the unsplit
model's. Prints EP_OK per rank."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from areal_b200.models.config import preset  # noqa: E402
from areal_b200.models.decoder import build_model  # noqa: E402
from areal_b200.parallel import ep as EP  # noqa: E402


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    cfg = preset("tiny-qwen3-moe")
    full = build_model(cfg, dtype=torch.float32, device="cpu", seed=3)
    local = build_model(cfg, dtype=torch.float32, device="cpu", seed=3)
    names = EP.shard_experts(local, rank, world, dist.group.WORLD)
    assert names and all(dict(local.named_parameters())[n].shape[0] == cfg.num_experts // world for n in names)
    g = torch.Generator().manual_seed(100 + rank)            # every rank has its own tokens
    lens = [19 + rank * 5, 30, 11]
    T = sum(lens)
    ids = torch.randint(0, cfg.vocab_size, (T,), generator=g)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    labels = torch.roll(ids, -1)

    def run(m):
        m.train()
        h = m(ids, cu, max_seqlen=max(lens))
        lp, _ = m.logprobs_entropy(h, labels)
        loss = -lp.float().sum()
        loss.backward()
        return h.detach(), loss.detach()
    h_ref, l_ref = run(full)
    h_ep, l_ep = run(local)
    assert torch.allclose(h_ref, h_ep, atol=2e-5), (h_ref - h_ep).abs().max()
    assert abs(l_ref.item() - l_ep.item()) < 1e-3
    # replicated parameters: the local gradient equals the unsplit model's (same tokens);
    # expert parameters: the owner accumulates the contributions of EVERY rank's tokens
    ref_grads = {n: p.grad for n, p in full.named_parameters()}
    El = cfg.num_experts // world
    for n, p in local.named_parameters():
        if n in names:
            tot = ref_grads[n].clone()
            dist.all_reduce(tot)                              # sum of all ranks' unsplit-model expert grads
            want = tot[rank * El:(rank + 1) * El]
        else:
            want = ref_grads[n]
        err = (p.grad - want).abs().max().item()
        assert err < 5e-5 * max(1.0, want.abs().max().item()), f"grad of {n} off by {err}"
    print("EP_OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
