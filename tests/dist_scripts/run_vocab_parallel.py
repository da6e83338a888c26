"""Vocab-parallel LM head parity on gloo ranks (CPU) or NCCL ranks (GPU). Prints VP_OK."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from areal_b200.ops import functional as OF  # noqa: E402
from areal_b200.parallel.vocab_parallel import PartialsExchange, vocab_parallel_lm_head_logprob  # noqa: E402


def main():
    use_cuda = torch.cuda.is_available() and os.environ.get("AREAL_FORCE_CPU", "0") != "1"
    dist.init_process_group("nccl" if use_cuda else "gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0))) if use_cuda else torch.device("cpu")
    if use_cuda:
        torch.cuda.set_device(dev)
    dtype = torch.bfloat16 if use_cuda else torch.float32
    g = torch.Generator().manual_seed(0)
    T, H, V = 300, 64, 1000 if not use_cuda else 4096
    h = torch.randn(T, H, generator=g).to(dev, dtype).requires_grad_()
    W = (torch.randn(V, H, generator=g) * 0.3).to(dev, dtype)
    labels = torch.randint(0, V, (T,), generator=g).to(dev)
    Vl = V // world
    Ws = W[rank * Vl:(rank + 1) * Vl].clone().requires_grad_()
    lp, ent = vocab_parallel_lm_head_logprob(h, Ws, labels, dist.group.WORLD, temperature=0.7, chunk=128)
    gl, ge = torch.randn(T, generator=g).to(dev), torch.randn(T, generator=g).to(dev)
    (lp * gl + ent * ge).sum().backward()
    # oracle: plain fp32 math on the full matrix
    h2 = h.detach().float().requires_grad_()
    W2 = W.float().requires_grad_()
    z = (h2 @ W2.t()) / 0.7
    lsm = torch.log_softmax(z, -1)
    lp2 = lsm.gather(1, labels[:, None])[:, 0]
    ent2 = -(lsm.exp() * lsm).sum(-1)
    (lp2 * gl + ent2 * ge).sum().backward()
    tol = 3e-2 if use_cuda else 2e-4
    assert (lp.float() - lp2).abs().max() < tol and (ent.float() - ent2).abs().max() < tol
    rel = lambda a, b: ((a.float() - b.float()).norm() / (b.float().norm() + 1e-9)).item()
    assert rel(h.grad, h2.grad) < (3e-2 if use_cuda else 1e-4), rel(h.grad, h2.grad)
    assert rel(Ws.grad, W2.grad[rank * Vl:(rank + 1) * Vl]) < (3e-2 if use_cuda else 1e-4)
    if use_cuda:
        # the same with the partials exchanged through peer memory instead of an NCCL all-gather: same bits
        from areal_b200.ops import lib as oplib

        ex = PartialsExchange(dist.group.WORLD, dev, max_rows=128)
        lp3, ent3 = vocab_parallel_lm_head_logprob(h.detach(), Ws.detach(), labels, dist.group.WORLD, temperature=0.7, chunk=128, exchange=ex)
        torch.cuda.synchronize()
        assert oplib.kernel_error() == 0
        assert torch.equal(lp3, lp.detach()) and torch.equal(ent3, ent.detach())
        lp4, _ = vocab_parallel_lm_head_logprob(h.detach(), Ws.detach(), labels, dist.group.WORLD, temperature=0.7, chunk=100, exchange=ex)
        assert (lp4.float() - lp2).abs().max() < tol
        print("VP_PEER_OK", flush=True)
    print("VP_OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
