"""Prefix-sharing ("tree") training: sequences that share prefixes (the n samples of a GRPO
group share their prompt) are merged into a trie so that every distinct (prefix, token) is
computed once; attention lets a node see exactly its ancestors.

* :func:`build_tree` merges token sequences into a packed trie (tokens, parent pointers, depth
  as position id, and for every original sequence the node index of each of its tokens);
* :func:`ancestor_mask` is the attention mask of the packed trie;
* :func:`tree_forward_hidden` runs the decoder over the packed trie (masked attention through
  ``scaled_dot_product_attention``; the flash kernels cover causal varlen only, so this path is
  the numerics reference and the memory saver, not yet the fast path);
* :func:`gather_sequence_outputs` maps node outputs back to the original sequences.

Reference: ``areal/models/tree_attn/{tree.py, functional.py, module_*.py}``."""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Sequence

import torch
import torch.nn.functional as F

from ..ops import functional as OF
from .decoder import CausalLM, PackedBatch


@dataclass
class PackedTree:
    tokens: torch.Tensor            # [N] token id of every trie node (depth-first order)
    parent: torch.Tensor            # [N] parent node index, -1 for roots
    depth: torch.Tensor             # [N] position id (0 for the first token of a sequence)
    seq_nodes: list[torch.Tensor]   # per original sequence: node index of each of its tokens
    n_tokens_unpacked: int

    @property
    def num_nodes(self) -> int:
        return int(self.tokens.numel())

    @property
    def saving(self) -> float:
        """Fraction of token computations avoided."""
        return 1.0 - self.num_nodes / max(1, self.n_tokens_unpacked)


def build_tree(sequences: Sequence[Sequence[int]]) -> PackedTree:
    """Merges sequences into a trie. Nodes are emitted in depth-first order, so a node's
    ancestors always precede it (the mask is lower-triangular)."""
    children: list[dict[int, int]] = []      # raw node id -> {token: raw child id}
    tok: list[int] = []
    par: list[int] = []
    roots: dict[int, int] = {}
    seq_raw: list[list[int]] = []
    for s in sequences:
        cur = -1
        path = []
        for t in s:
            t = int(t)
            table = roots if cur < 0 else children[cur]
            nxt = table.get(t)
            if nxt is None:
                nxt = len(tok)
                tok.append(t)
                par.append(cur)
                children.append({})
                table[t] = nxt
            path.append(nxt)
            cur = nxt
        seq_raw.append(path)
    # depth-first renumbering
    order: list[int] = []
    stack = list(reversed(list(roots.values())))
    while stack:
        n = stack.pop()
        order.append(n)
        stack.extend(reversed(list(children[n].values())))
    new_of = {raw: i for i, raw in enumerate(order)}
    tokens = torch.tensor([tok[r] for r in order], dtype=torch.long)
    parent = torch.tensor([new_of[par[r]] if par[r] >= 0 else -1 for r in order], dtype=torch.long)
    depth = torch.zeros(len(order), dtype=torch.long)
    for i in range(len(order)):
        p = int(parent[i])
        depth[i] = 0 if p < 0 else depth[p] + 1
    seq_nodes = [torch.tensor([new_of[r] for r in path], dtype=torch.long) for path in seq_raw]
    return PackedTree(tokens, parent, depth, seq_nodes, sum(len(s) for s in sequences))


def ancestor_mask(parent: torch.Tensor) -> torch.Tensor:
    """bool [N, N]: mask[i, j] is True when j is i or an ancestor of i."""
    N = parent.numel()
    mask = torch.eye(N, dtype=torch.bool, device=parent.device)
    for i in range(N):                       # parents precede children in DFS order
        p = int(parent[i])
        if p >= 0:
            mask[i] |= mask[p]
    return mask


def _masked_attention(q, k, v, mask, scale):
    """q: [N, Hq, D], k/v: [N, Hkv, D], mask bool [N, N]."""
    rep = q.shape[1] // k.shape[1]
    qh = q.transpose(0, 1)[None]
    kh = k.transpose(0, 1).repeat_interleave(rep, 0)[None]
    vh = v.transpose(0, 1).repeat_interleave(rep, 0)[None]
    o = F.scaled_dot_product_attention(qh.float(), kh.float(), vh.float(), attn_mask=mask[None, None], scale=scale)
    return o[0].transpose(0, 1).to(q.dtype)


def tree_forward_hidden(model: CausalLM, tree: PackedTree) -> torch.Tensor:
    """Final normed hidden state of every trie node ``[N, H]``."""
    dev = model.embed_tokens.device
    ids = tree.tokens.to(dev)
    pos = tree.depth.to(dev).int()
    mask = ancestor_mask(tree.parent).to(dev)
    N = ids.numel()
    cu = torch.tensor([0, N], dtype=torch.int32, device=dev)
    pb = PackedBatch(cu, pos, N, int(tree.depth.max().item()) + 1)
    scale = 1.0 / math.sqrt(model.cfg.head_dim)
    fns = [lambda q, k, v: _masked_attention(q, k, v, mask, scale)] * len(model.layers)
    return model.forward_hidden(ids.int() if dev.type == "cuda" else ids, pb, attn_fns=fns)


def gather_sequence_outputs(node_out: torch.Tensor, tree: PackedTree) -> list[torch.Tensor]:
    """Per original sequence, the outputs of its tokens (a view by index)."""
    return [node_out[idx.to(node_out.device)] for idx in tree.seq_nodes]


def tree_logprobs(model: CausalLM, sequences: Sequence[Sequence[int]], temperature: float = 1.0) -> list[torch.Tensor]:
    """Next-token log-probs of every sequence (length L - 1 each) computed on the packed trie:
    identical to running the sequences one by one, at the cost of the distinct prefixes only."""
    tree = build_tree(sequences)
    h = tree_forward_hidden(model, tree)
    out = []
    for s, idx in zip(sequences, tree.seq_nodes):
        hs = h[idx.to(h.device)][:-1]
        labels = torch.tensor(list(s)[1:], dtype=torch.long, device=h.device)
        lp, _ = model.logprobs_entropy(hs.contiguous(), labels, temperature)
        out.append(lp)
    return out
