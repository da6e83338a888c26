"""Tensor-parallel forward/backward parity against the unsharded model (gloo ranks on CPU, or
NCCL ranks on GPUs when available). Prints TP_OK per rank."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from areal_b200.models.config import preset  # noqa: E402
from areal_b200.models.decoder import PackedBatch, build_model  # noqa: E402
from areal_b200.parallel import tp as TP  # noqa: E402


def main():
    use_cuda = torch.cuda.is_available() and os.environ.get("AREAL_FORCE_CPU", "0") != "1"
    dist.init_process_group("nccl" if use_cuda else "gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0))) if use_cuda else torch.device("cpu")
    if use_cuda:
        torch.cuda.set_device(dev)
    dtype = torch.bfloat16 if use_cuda else torch.float32
    for name in ("tiny-qwen3", "tiny-qwen3-moe"):
        cfg = preset(name)
        full = build_model(cfg, dtype=dtype, device=dev, seed=3)
        lcfg = TP.local_config(cfg, world)
        local = build_model(lcfg, dtype=dtype, device=dev, seed=99)
        state = {n: p.detach() for n, p in full.named_parameters()}
        TP.load_sharded_from_full(local, cfg, state, world, rank)
        TP.install_tp(local, dist.group.WORLD, world, rank)
        # round trip of the shard layout
        for n, p in local.named_parameters():
            parts = [torch.empty_like(p) for _ in range(world)]
            dist.all_gather(parts, p.detach().contiguous())
            back = TP.unshard_tensors(cfg, n, parts)
            assert back.shape == state[n].shape and torch.equal(back, state[n]), f"unshard mismatch for {n}"
        g = torch.Generator().manual_seed(0)
        lens = [37, 64, 27]
        T = sum(lens)
        ids = torch.randint(0, cfg.vocab_size, (T,), generator=g).to(dev)
        cu = torch.tensor([0, 37, 101, 128], dtype=torch.int32, device=dev)
        labels = torch.roll(ids, -1)

        def run(m):
            m.train()
            h = m(ids, cu, max_seqlen=64)
            lp, _ = m.logprobs_entropy(h, labels)
            loss = -(lp.float().mean())
            aux = m.aux_loss()
            if aux is not None:
                loss = loss + aux
            loss.backward()
            return loss.detach()
        l_full = run(full)
        l_tp = run(local)
        TP.allreduce_replicated_grads(local, dist.group.WORLD, grad_of=lambda p: p.grad)
        tol = 3e-2 if use_cuda else 2e-4
        assert abs(l_full.item() - l_tp.item()) < tol * max(1.0, abs(l_full.item())), (name, l_full.item(), l_tp.item())
        gfull = {n: p.grad for n, p in full.named_parameters()}
        worst = 0.0
        for n, p in local.named_parameters():
            ref = TP.shard_tensor(cfg, n, gfull[n], world, rank).float()
            got = p.grad.float()
            err = (got - ref).abs().max().item() / (ref.abs().max().item() + 1e-6)
            worst = max(worst, err)
            assert err < (0.08 if use_cuda else 2e-3), f"{name}: grad mismatch for {n}: {err}"
        if rank == 0:
            print(f"{name}: loss {l_full.item():.5f} vs {l_tp.item():.5f}, worst grad rel err {worst:.2e}", flush=True)
    # row shares of a tensor that every rank holds, with a row count the group does not divide (7 rows over the ranks):
    # slice -> per-share function -> gather equals the function of the whole, forward and backward
    if not use_cuda:
        torch.manual_seed(3)
        x = torch.randn(7, 5, requires_grad=True)
        w = torch.randn(5, 5)
        y = TP._GatherRows.apply(torch.tanh(TP._SliceRows.apply(x, dist.group.WORLD, world, rank) @ w), dist.group.WORLD, world, rank, 7)
        (y * torch.arange(7.0)[:, None]).sum().backward()
        x2 = x.detach().clone().requires_grad_(True)
        y2 = torch.tanh(x2 @ w)
        (y2 * torch.arange(7.0)[:, None]).sum().backward()
        assert y.shape == (7, 5) and torch.allclose(y, y2, atol=1e-6) and torch.allclose(x.grad, x2.grad, atol=1e-6)
    print("TP_OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
