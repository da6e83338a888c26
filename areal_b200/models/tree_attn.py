"""Prefix-sharing ("tree") training: sequences that share prefixes (the n samples of a GRPO
group share their prompt) are merged into a trie so that every distinct (prefix, token) is
computed once; attention lets a node see exactly its ancestors.

* :func:`build_tree` merges token sequences into a packed trie (tokens, parent pointers, depth
  as position id, and for every original sequence the node index of each of its tokens);
* :func:`ancestor_mask` is the attention mask of the packed trie;
* :func:`tree_forward_hidden` runs the decoder over the packed trie. Every projection, norm and
  MLP runs once per trie node. Attention has two forms: ``flash`` (default) gathers q/k/v of the
  nodes back into the per-sequence layout, runs the causal varlen flash kernels there and keeps
  one copy of each node's output (the copies are identical: a node's output depends on its
  ancestors only). The attention of a shared prefix is then computed once per sequence that
  contains it, which for a group that shares a prompt of length P among responses of length R
  costs P^2 / (P + R)^2 of the attention work extra (4 % at P = 1024, R = 4096) while all the
  GEMM work of the prefix is saved; gradients of shared keys and values add up through the gather.
  ``masked`` materialises the [N, N] ancestor mask for ``scaled_dot_product_attention`` (fp32):
  the numerics oracle;
* :func:`tree_hidden_for_packed_batch` is the trainer's entry: packed micro-batch in, per-token
  hidden states out, with the trie in between;
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
    seq_nodes = [torch.tensor([new_of[r] for r in path], dtype=torch.long) for path in seq_raw]
    depth = torch.zeros(len(order), dtype=torch.long)
    for idx in seq_nodes:                    # a node's depth is its position in any sequence through it
        depth[idx] = torch.arange(idx.numel())
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


@dataclass
class FlashTreePlan:
    """Index tensors of the gather-to-sequences attention: ``node_of[t]`` is the trie node of token ``t`` of
    the per-sequence (packed) layout, ``rep_pos[n]`` the first token that shows node ``n``."""
    node_of: torch.Tensor
    rep_pos: torch.Tensor
    cu_seqlens: torch.Tensor
    tile_info: Optional[torch.Tensor]
    total: int


def flash_tree_plan(tree: PackedTree, device, n_nodes: Optional[int] = None) -> FlashTreePlan:
    N = tree.num_nodes if n_nodes is None else n_nodes       # nodes past the trie (alignment) show token 0's output; nobody reads it
    node_of = torch.cat(tree.seq_nodes) if tree.seq_nodes else torch.zeros(0, dtype=torch.long)
    T = int(node_of.numel())
    rep = torch.full((N,), T, dtype=torch.long)
    rep.scatter_reduce_(0, node_of, torch.arange(T), reduce="amin")
    rep[rep >= T] = 0
    lens = torch.tensor([0] + [int(i.numel()) for i in tree.seq_nodes])
    cu = lens.cumsum(0).to(torch.int32).to(device)
    tile = OF.attn_tile_table(cu, T) if torch.device(device).type == "cuda" else None
    return FlashTreePlan(node_of.to(device), rep.to(device), cu, tile, T)


def _flash_tree_attention(q, k, v, plan: FlashTreePlan, scale):
    """q: [N, Hq, D], k / v: [N, Hkv, D] per trie node -> attention output per trie node."""
    qs, ks, vs = q.index_select(0, plan.node_of), k.index_select(0, plan.node_of), v.index_select(0, plan.node_of)
    o = OF.attention(qs, ks, vs, plan.cu_seqlens, True, scale, plan.tile_info)
    return o.index_select(0, plan.rep_pos)


def tree_forward_hidden(model: CausalLM, tree: PackedTree, attention: str = "flash", pad_to: int = 1) -> torch.Tensor:
    """Final normed hidden state of every trie node ``[N, H]`` (``pad_to``: the node count the kernels see is
    rounded up to a multiple of it; the extra rows are dropped from the result)."""
    dev = model.embed_tokens.device
    N = tree.num_nodes
    Np = -(-N // pad_to) * pad_to
    ids, pos = tree.tokens, tree.depth
    if Np != N:
        ids = torch.cat([ids, ids.new_zeros(Np - N)])
        pos = torch.cat([pos, pos.new_zeros(Np - N)])
    ids, pos = ids.to(dev), pos.to(dev).int()
    cu = torch.tensor([0, Np], dtype=torch.int32, device=dev)
    pb = PackedBatch(cu, pos, Np, int(tree.depth.max().item()) + 1 if N else 1)
    scale = 1.0 / math.sqrt(model.cfg.head_dim)
    if attention == "masked":
        mask = torch.eye(Np, dtype=torch.bool)
        mask[:N, :N] = ancestor_mask(tree.parent)
        mask = mask.to(dev)
        fn = lambda q, k, v: _masked_attention(q, k, v, mask, scale)      # noqa: E731
    else:
        plan = flash_tree_plan(tree, dev, Np)
        fn = lambda q, k, v: _flash_tree_attention(q, k, v, plan, scale)  # noqa: E731
    h = model.forward_hidden(ids.int() if dev.type == "cuda" else ids, pb, attn_fns=[fn] * len(model.layers))
    return h[:N]


def tree_hidden_for_packed_batch(model: CausalLM, input_ids: torch.Tensor, cu_seqlens: torch.Tensor, pad_to: int = 1):
    """Hidden states ``[T, H]`` of a packed micro-batch computed on the trie of its sequences (every segment of
    ``cu_seqlens`` is one sequence; padding segments are sequences like the others). Returns the hidden states
    in the packed order and the fraction of token computations saved."""
    cu = cu_seqlens.tolist()
    flat = input_ids.tolist()
    tree = build_tree([flat[a:b] for a, b in zip(cu[:-1], cu[1:]) if b > a])
    h = tree_forward_hidden(model, tree, "flash", pad_to)
    node_of = torch.cat(tree.seq_nodes).to(h.device)
    return h.index_select(0, node_of), tree.saving


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
