"""Prefix-sharing training: trie packing, ancestor mask, parity with per-sequence forward."""
import pytest
import torch

from areal_b200.models.config import preset
from areal_b200.models.decoder import build_model
from areal_b200.models.tree_attn import (ancestor_mask, build_tree, tree_forward_hidden, tree_hidden_for_packed_batch,
                                         tree_logprobs)


def test_trie_packing_and_mask():
    seqs = [[5, 6, 7, 1, 2], [5, 6, 7, 3], [5, 6, 9], [4, 4]]
    t = build_tree(seqs)
    assert t.num_nodes == 5 + 1 + 1 + 2 and t.n_tokens_unpacked == 14 and abs(t.saving - (1 - 9 / 14)) < 1e-9
    for s, idx in zip(seqs, t.seq_nodes):
        assert t.tokens[idx].tolist() == s and t.depth[idx].tolist() == list(range(len(s)))
        for a, b in zip(idx[:-1].tolist(), idx[1:].tolist()):
            assert int(t.parent[b]) == a
    m = ancestor_mask(t.parent)
    assert torch.equal(m, torch.tril(m))                         # DFS order: ancestors precede descendants
    last = int(t.seq_nodes[1][-1])                                # token 3 of the second sequence
    assert m[last].nonzero().flatten().tolist() == sorted(t.seq_nodes[1].tolist())


def test_tree_logprobs_match_per_sequence_forward():
    cfg = preset("tiny-qwen3")
    model = build_model(cfg, dtype=torch.float32, device="cpu", seed=4).eval()
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, cfg.vocab_size, (12,), generator=g).tolist()
    seqs = [prompt + torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (5, 9, 3, 7)]
    with torch.no_grad():
        got = tree_logprobs(model, seqs)
        for s, lp in zip(seqs, got):
            ids = torch.tensor(s)
            cu = torch.tensor([0, len(s)], dtype=torch.int32)
            h = model(ids, cu, max_seqlen=len(s))
            ref, _ = model.logprobs_entropy(h[:-1].contiguous(), ids[1:])
            assert torch.allclose(lp, ref, atol=2e-5), (lp - ref).abs().max()
    assert build_tree(seqs).saving > 0.45                         # the shared prompt is computed once


def test_flash_form_matches_masked_form_and_carries_gradients_of_shared_nodes():
    """Gather-to-sequences attention (the form the flash kernels run) against the ancestor-mask oracle on a trie
    with nested branching, forward and parameter gradients; node padding changes nothing."""
    cfg = preset("tiny-qwen3")
    model = build_model(cfg, dtype=torch.float32, device="cpu", seed=5)
    g = torch.Generator().manual_seed(1)
    r = lambda n: torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist()   # noqa: E731
    p, mid = r(9), r(4)
    seqs = [p + mid + r(5), p + mid + r(2), p + r(6), r(3)]
    tree = build_tree(seqs)
    assert tree.depth.tolist() == [int(ancestor_mask(tree.parent)[i].sum()) - 1 for i in range(tree.num_nodes)]
    outs = {}
    for form, pad in (("masked", 1), ("flash", 1), ("flash", 16)):
        model.zero_grad()
        h = tree_forward_hidden(model, tree, form, pad)
        assert h.shape[0] == tree.num_nodes
        w = torch.linspace(0.5, 1.5, h.shape[0])[:, None]
        (h * w).pow(2).sum().backward()
        outs[(form, pad)] = (h.detach(), model.layers[0].self_attn.qkv_proj.grad.clone(), model.embed_tokens.grad.clone())
    ref = outs[("masked", 1)]
    for key in (("flash", 1), ("flash", 16)):
        for a, b in zip(outs[key], ref):
            assert torch.allclose(a, b, atol=2e-4, rtol=1e-3), (key, (a - b).abs().max())


def test_packed_batch_entry_equals_plain_forward():
    cfg = preset("tiny-qwen3")
    model = build_model(cfg, dtype=torch.float32, device="cpu", seed=6).eval()
    g = torch.Generator().manual_seed(2)
    prompt = torch.randint(0, cfg.vocab_size, (10,), generator=g).tolist()
    seqs = [prompt + torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (4, 6, 3)] + [[0] * 5]
    ids = torch.tensor([t for s in seqs for t in s])
    cu = torch.tensor([0] + [len(s) for s in seqs]).cumsum(0).to(torch.int32)
    with torch.no_grad():
        h, saving = tree_hidden_for_packed_batch(model, ids, cu, pad_to=8)
        ref = model(ids, cu, max_seqlen=16)
    assert saving > 0.4 and torch.allclose(h, ref, atol=2e-5)


def test_engine_trains_the_same_with_and_without_prefix_sharing():
    """``enable_tree_training`` changes how a micro-batch is computed, not what: log-probs of a batch whose samples
    share their prompts and the parameters after one SFT-style step agree with the plain path."""
    from areal_b200.api.cli_args import MicroBatchSpec, OptimizerConfig, PPOActorConfig
    from areal_b200.engine.train_engine import B200PPOActor

    cfgm = preset("tiny-qwen3")
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(1, cfgm.vocab_size, (11,), generator=g).tolist() for _ in range(2)]
    seqs = [p + torch.randint(1, cfgm.vocab_size, (n,), generator=g).tolist() for p in prompts for n in (5, 8, 3)]
    L = max(len(s) for s in seqs)
    ids = torch.zeros(len(seqs), L, dtype=torch.long)
    am = torch.zeros(len(seqs), L, dtype=torch.long)
    for i, s in enumerate(seqs):
        ids[i, :len(s)] = torch.tensor(s)
        am[i, :len(s)] = 1
    loss_mask = am.clone()
    loss_mask[:, :11] = 0
    batch = {"input_ids": ids, "attention_mask": am, "loss_mask": loss_mask}

    def run(tree: bool):
        cfg = PPOActorConfig(init_from_scratch=True, dtype="float32", optimizer=OptimizerConfig(type="sgd", lr=1e-1, weight_decay=0.0),
                             mb_spec=MicroBatchSpec(max_tokens_per_mb=4096), enable_tree_training=tree)
        e = B200PPOActor(cfg)
        e.create_process_group()
        e.initialize(model_config=cfgm, seed=11)
        lp = e.forward_batch(dict(batch), output="logprobs")

        def loss_fn(logp, entropy, mb):
            m = torch.roll(mb["loss_mask"], -1, 0).float()
            return -(logp * m).sum() / m.sum().clamp(min=1)
        e.train_batch(dict(batch), loss_fn, lambda mb: torch.roll(mb["loss_mask"], -1, 0).float().sum())
        return lp, e.store.flat_param.clone(), getattr(e, "_tree_saving", None)

    lp0, p0, s0 = run(False)
    lp1, p1, s1 = run(True)
    assert s0 is None and s1 > 0.3
    assert torch.allclose(lp0, lp1, atol=2e-5) and torch.allclose(p0, p1, atol=2e-5)


@pytest.mark.gpu
def test_tree_training_on_the_flash_kernels_matches_the_plain_packed_forward():
    """bf16 model on the device: hidden states and parameter gradients of a batch whose groups share long prompts,
    computed over the trie (flash kernels on the gathered layout) and by the plain packed forward + backward, both
    compared with an fp32 oracle on the host: the trie path is no further from fp32 than bf16 rounding puts the
    plain path (the loss sits behind a norm, so several gradients are sums of nearly cancelling terms)."""
    cfg = preset("tiny-qwen3")
    model = build_model(cfg, dtype=torch.bfloat16, device="cuda", seed=7)
    oracle = build_model(cfg, dtype=torch.float32, device="cpu", seed=7)
    with torch.no_grad():
        for p, q in zip(model.parameters(), oracle.parameters()):
            q.copy_(p.float().cpu())
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(1, cfg.vocab_size, (n,), generator=g).tolist() for n in (300, 170)]
    seqs = [p + torch.randint(1, cfg.vocab_size, (n,), generator=g).tolist() for p in prompts for n in (90, 260, 33, 140)]
    flat = [t for s in seqs for t in s]
    cu_host = torch.tensor([0] + [len(s) for s in seqs]).cumsum(0).to(torch.int32)
    ids, cu = torch.tensor(flat, device="cuda", dtype=torch.int32), cu_host.cuda()
    w = torch.linspace(0.5, 1.5, len(flat))[:, None]
    ho = oracle(torch.tensor(flat), cu_host, max_seqlen=600)
    (ho * w).pow(2).mean().backward()
    named = [n for n, p in oracle.named_parameters() if p.grad is not None]
    want = {n: p.grad for n, p in oracle.named_parameters() if p.grad is not None}
    rel = lambda a, b: ((a - b).norm() / b.norm().clamp(min=1e-12)).item()   # noqa: E731
    errs = {}
    for tree in (False, True):
        model.zero_grad()
        if tree:
            h, saving = tree_hidden_for_packed_batch(model, ids, cu, pad_to=128)
            assert saving > 0.4
        else:
            h = model(ids, cu, max_seqlen=600)
        (h.float() * w.cuda()).pow(2).mean().backward()
        got = {n: p.grad.float().cpu() for n, p in model.named_parameters() if p.grad is not None}
        assert sorted(got) == sorted(named)
        errs[tree] = (rel(h.detach().float().cpu(), ho.detach()), {n: rel(got[n], want[n]) for n in named})
    assert errs[True][0] < max(2e-2, 2 * errs[False][0])
    worst = {n: (errs[True][1][n], errs[False][1][n]) for n in named if errs[True][1][n] > max(5e-2, 3 * errs[False][1][n])}
    assert not worst, worst
