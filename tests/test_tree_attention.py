"""Prefix-sharing training: trie packing, ancestor mask, parity with per-sequence forward."""
import torch

from areal_b200.models.config import preset
from areal_b200.models.decoder import build_model
from areal_b200.models.tree_attn import ancestor_mask, build_tree, tree_logprobs


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
