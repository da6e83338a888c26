"""2+ GPU check of the fused expert-parallel dispatch / combine kernels: a MoE model whose
experts are split over the ranks runs the same tokens through the NCCL all-to-all dispatcher
and through the peer-memory kernels; hidden states, loss and every gradient must agree. With
``EP_FUSED_BENCH=1`` it also times one MoE layer (forward + backward) both ways at a
Qwen3-30B-A3B-like shape. Prints EP_FUSED_OK per rank."""
import faulthandler
import json
import os
import sys

faulthandler.dump_traceback_later(200, exit=True)
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import torch
import torch.distributed as dist

from areal_b200.models.config import preset
from areal_b200.models.decoder import build_model
from areal_b200.ops import lib as oplib
from areal_b200.parallel import ep as EP


def rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def timed(fn, iters=10):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl")
    cfg = preset("tiny-qwen3-moe")
    base = build_model(cfg, dtype=torch.bfloat16, device=dev, seed=3)
    fused = build_model(cfg, dtype=torch.bfloat16, device=dev, seed=3)
    names = EP.shard_experts(base, rank, world, dist.group.WORLD)
    EP.shard_experts(fused, rank, world, dist.group.WORLD, fused=True, device=dev)
    assert fused.ep_fused_comm is not None
    g = torch.Generator().manual_seed(100 + rank)             # every rank has its own tokens
    lens = [190 + rank * 50, 300, 110]
    T = sum(lens)
    ids = torch.randint(0, cfg.vocab_size, (T,), generator=g).to(dev)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=dev)
    labels = torch.roll(ids, -1)

    def run(m):
        m.train()
        for p in m.parameters():
            p.grad = None
        h = m(ids, cu, max_seqlen=max(lens))
        lp, _ = m.logprobs_entropy(h, labels)
        loss = -lp.float().mean()
        loss.backward()
        return h.detach(), loss.detach()

    # fp32 oracle on the CPU: the unsplit model with the same (bf16-rounded) weights on this rank's tokens.
    # Replicated parameters get exactly that gradient; an expert slice gets the sum over all ranks' tokens.
    oracle = build_model(cfg, dtype=torch.float32, device="cpu", seed=3)
    full = build_model(cfg, dtype=torch.bfloat16, device=dev, seed=3)      # same draws as the two GPU models
    with torch.no_grad():
        src = dict(full.named_parameters())
        for n, p in oracle.named_parameters():
            p.copy_(src[n].float().cpu())
    del full, src
    oracle.train()
    ho = oracle(ids.cpu(), cu.cpu(), max_seqlen=max(lens))
    lpo, _ = oracle.logprobs_entropy(ho, labels.cpu())
    (-lpo.float().mean()).backward()
    El = cfg.num_experts // world
    want = {}
    for n, p in oracle.named_parameters():
        gr = p.grad.to(dev)
        if n in names:
            dist.all_reduce(gr)
            gr = gr[rank * El:(rank + 1) * El]
        want[n] = gr

    for it in range(2):                                       # second pass reuses the slabs with advanced phases
        h0, l0 = run(base)
        h1, l1 = run(fused)
        assert rel(h1, h0) < 2e-2, ("hidden", rel(h1, h0))
        hf_, hb_ = rel(h1, ho.to(dev)), rel(h0, ho.to(dev))
        assert hf_ < max(1.5 * hb_, 5e-2), ("hidden vs fp32 (fused, library)", hf_, hb_)
        assert abs(l0.item() - l1.item()) < 2e-2 * max(1.0, abs(l0.item())), (l0.item(), l1.item())
        gb = dict(base.named_parameters())
        worst = ("", 0.0, 0.0)
        bad = []
        for n, p in fused.named_parameters():
            a, b = p.grad, gb[n].grad
            assert (a is None) == (b is None), n
            if a is None:
                continue
            # both paths against fp32 math: the fused kernels (fp32 gate weighting and top-k sums) must be at
            # least as close as the library path (bf16 products and sums), up to a small floor
            ef, eb = rel(a, want[n]), rel(b, want[n])
            if not ef < max(2.0 * eb, 5e-2):
                bad.append((n, round(ef, 4), round(eb, 4)))
            if ef > worst[1]:
                worst = (n, ef, eb)
        assert not bad, bad
    calls = sum(layer.mlp.ep_dispatcher.fused_calls for layer in fused.layers if hasattr(layer.mlp, "ep_dispatcher"))
    assert calls >= 2 * cfg.num_layers, calls                  # the fused path is what ran
    # forward-only (no_grad) path returns views of the slabs
    with torch.no_grad():
        a = base(ids, cu, max_seqlen=max(lens))
        b = fused(ids, cu, max_seqlen=max(lens))
    assert rel(b, a) < 2e-2
    assert oplib.kernel_error() == 0
    out = {"rank": rank, "hidden_rel": rel(h1, h0), "worst_grad_vs_fp32 (name, fused, library)": worst}

    if os.environ.get("EP_FUSED_BENCH", "0") == "1":
        big = preset("tiny-qwen3-moe", hidden_size=2048, num_layers=1, num_heads=16, num_kv_heads=4, head_dim=128,
                     num_experts=64, num_experts_per_tok=8, moe_intermediate_size=768)
        Tb = 8192
        res = {}
        for label, fz in (("nccl", False), ("fused", True)):
            m = build_model(big, dtype=torch.bfloat16, device=dev, seed=5)
            EP.shard_experts(m, rank, world, dist.group.WORLD, fused=fz, device=dev)
            mlp = m.layers[0].mlp
            x = torch.randn(Tb, big.hidden_size, device=dev, generator=torch.Generator(device=dev).manual_seed(rank)).bfloat16()
            x.requires_grad_(True)
            go = torch.randn(Tb, big.hidden_size, device=dev).bfloat16()

            def step():
                x.grad = None
                y = mlp(x)
                y.backward(go)
            res[label + "_fwd_bwd_ms"] = timed(step)
            with torch.no_grad():
                res[label + "_fwd_ms"] = timed(lambda: mlp(x))
            del m, mlp
            torch.cuda.empty_cache()
        res.update(tokens_per_rank=Tb, hidden=2048, experts=64, top_k=8, moe_intermediate=768, world=world,
                   remote_bytes_per_direction_per_phase=int(Tb * 8 * 2048 * 2 * (world - 1) / world))
        out["bench"] = res
        assert oplib.kernel_error() == 0
    if rank == 0:
        print(json.dumps(out), flush=True)
    print("EP_FUSED_OK", flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
