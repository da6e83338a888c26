"""Pipeline parallelism: the decoder's layers are split into contiguous stages, activations
``[tokens, hidden]`` travel between neighbouring stages with point-to-point sends, and
micro-batches follow the 1F1B (one-forward-one-backward) or GPipe schedule.

Every pipeline rank receives the same micro-batch list (token ids, packing metadata), so
shapes are known everywhere and only the hidden state crosses stage boundaries: the stage
boundary folds the residual stream into one tensor (``h + resid``), halving the traffic.
Activations stay on NCCL p2p (the transfers are small next to a stage's compute and overlap
with it). Tied embeddings live on the first and last stage and their gradients are summed
between the two. Reference: ``areal/experimental/engine/archon/pipeline_parallel.py`` (stage
split by FQN :80, schedules from ``torch.distributed.pipelining``), Megatron schedules in
``areal/engine/megatron_engine.py:1112-1329``.
"""
from __future__ import annotations

from typing import Any, Callable, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from ..models.config import ModelConfig
from ..models.decoder import CausalLM, PackedBatch, build_model
from ..ops import functional as OF


def split_layers(n_layers: int, n_stages: int, first_extra: int = 0, last_extra: int = 0) -> list[range]:
    """Contiguous, near-equal layer ranges. ``first_extra`` / ``last_extra`` count the embedding
    and the LM head as that many layers' worth of work when balancing."""
    if n_stages > n_layers:
        raise ValueError(f"{n_stages} pipeline stages for {n_layers} layers")
    total = n_layers + first_extra + last_extra
    out, start = [], 0
    for s in range(n_stages):
        want = (total * (s + 1)) // n_stages - (total * s) // n_stages
        if s == 0:
            want -= first_extra
        if s == n_stages - 1:
            want = n_layers - start
        want = max(1, min(want, n_layers - start - (n_stages - 1 - s)))
        out.append(range(start, start + want))
        start += want
    return out


class PipelineStage(nn.Module):
    """The slice of a :class:`CausalLM` one pipeline rank owns."""

    def __init__(self, cfg: ModelConfig, stage: int, n_stages: int, dtype=torch.bfloat16, device="cpu", seed: Optional[int] = None,
                 layer_ranges: Optional[list[range]] = None, init_full: Optional[Callable] = None, tp: int = 1, tp_rank: int = 0):
        super().__init__()
        self.cfg, self.stage, self.n_stages = cfg, stage, n_stages
        self.tp, self.tp_rank = tp, tp_rank
        self.dtype = dtype
        self.is_first, self.is_last = stage == 0, stage == n_stages - 1
        ranges = layer_ranges or split_layers(cfg.num_layers, n_stages)
        self.layer_range = ranges[stage]
        # build the full model once (same seed on every rank => consistent weights), keep a slice;
        # ``init_full(model)`` may load a checkpoint into it first
        full = build_model(cfg, dtype=dtype, device=device, seed=seed)
        if init_full is not None:
            init_full(full)
        if tp > 1:
            # tensor parallelism inside the stage: the same weights, sliced (heads / MLP columns) for this TP rank
            from . import tp as TP

            local = build_model(TP.local_config(cfg, tp), dtype=dtype, device=device, seed=seed)
            TP.load_sharded_from_full(local, cfg, {n: p.detach() for n, p in full.named_parameters()}, tp, tp_rank)
            full = local
        self.layers = nn.ModuleList([full.layers[i] for i in self.layer_range])
        self.embed_tokens = full.embed_tokens if (self.is_first or (self.is_last and cfg.tie_word_embeddings and not cfg.is_critic)) else None
        self.norm = full.norm if self.is_last else None
        self.lm_head = full.lm_head if self.is_last else None
        self.value_head = full.value_head if self.is_last else None
        self._rope = full.rope
        self._full_ref = full if False else None
        self.gradient_checkpointing = False

    @property
    def output_weight(self):
        return self.embed_tokens if self.lm_head is None else self.lm_head

    def native_name(self, local_name: str) -> str:
        """Name of a stage parameter in the full model (checkpoints, weight updates)."""
        if local_name.startswith("layers."):
            i, rest = local_name[len("layers."):].split(".", 1)
            return f"layers.{self.layer_range[int(i)]}.{rest}"
        return local_name

    def forward(self, x: torch.Tensor, pb: PackedBatch) -> torch.Tensor:
        """First stage: ``x`` = token ids [T]; other stages: hidden state [T, H]. Returns the
        hidden state handed to the next stage, or the final normed hidden state."""
        cos, sin = self._rope(x.device, max(self.cfg.max_position_embeddings, pb.max_seqlen + 1))
        h = OF.embedding(x, self.embed_tokens) if self.is_first else x
        resid = None
        for layer in self.layers:
            if self.gradient_checkpointing and self.training and torch.is_grad_enabled():
                from torch.utils.checkpoint import checkpoint

                h, resid = checkpoint(layer, h, resid, pb, cos, sin, None, use_reentrant=False)
            else:
                h, resid = layer(h, resid, pb, cos, sin, None)
        if self.is_last:
            if self.cfg.rms_norm_offset:           # (1 + w) norms of the hybrid linear-attention family
                from ..models.hybrid import rmsnorm_offset

                out, _ = rmsnorm_offset(h, self.norm, self.cfg.rms_norm_eps, resid)
            else:
                out, _ = OF.rmsnorm(h, self.norm, self.cfg.rms_norm_eps, resid)
            return out
        return h + resid if resid is not None else h

    def logprobs_entropy(self, hidden, labels, temperature: float = 1.0, chunk: int = 2048):
        return OF.lm_head_logprob(hidden, self.output_weight, labels, temperature, chunk)

    def values(self, hidden: torch.Tensor) -> torch.Tensor:
        return torch.nn.functional.linear(hidden.float(), self.value_head.float()).squeeze(-1)

    def aux_loss(self) -> Optional[torch.Tensor]:
        """Router balancing loss of this stage's MoE layers (each stage adds its own to its backward)."""
        tot = None
        for layer in self.layers:
            al = getattr(layer.mlp, "last_aux_loss", None)
            if al is not None:
                tot = al if tot is None else tot + al
                layer.mlp.last_aux_loss = None
        return tot

    def named_native_parameters(self, skip_tied_copy: bool = True):
        """(name in the full model, parameter); the last stage's copy of a tied embedding is left
        out so that the stages' name sets are disjoint."""
        for n, p in self.named_parameters():
            if skip_tied_copy and n == "embed_tokens" and self.is_last and not self.is_first:
                continue
            yield self.native_name(n), p


class PipelineRunner:
    """Runs micro-batches through the stages of ONE pipeline (a process group whose ranks are
    the stages in order)."""

    def __init__(self, stage_module: PipelineStage, group, schedule: str = "1F1B"):
        self.m = stage_module
        self.group = group
        self.rank = dist.get_rank(group)
        self.n = dist.get_world_size(group)
        assert self.rank == stage_module.stage and self.n == stage_module.n_stages
        ranks = dist.get_process_group_ranks(group)
        self.prev = ranks[self.rank - 1] if self.rank > 0 else None
        self.next = ranks[self.rank + 1] if self.rank < self.n - 1 else None
        self.first_rank, self.last_rank = ranks[0], ranks[-1]
        if schedule not in ("1F1B", "GPipe", "ZBH1"):
            raise ValueError("schedule must be 1F1B, GPipe or ZBH1 (interleaved variants need virtual stages)")
        self.schedule = schedule
        p = next(stage_module.parameters())
        self.device, self.dtype = p.device, p.dtype
        self.H = stage_module.cfg.hidden_size
        self._aux: dict[int, torch.Tensor] = {}
        self._pending_wgrad: Optional[list] = None

    # ---- p2p: every exchange is ONE batch of sends and receives, so a stage that sends forward
    # while its neighbour sends backward cannot block the other (NCCL groups the batch)
    def _p2p(self, send_next=None, recv_prev_T: Optional[int] = None, send_prev=None, recv_next_T: Optional[int] = None):
        ops, from_prev, from_next = [], None, None
        keep = []
        if send_prev is not None and self.prev is not None:
            t = send_prev.contiguous()
            keep.append(t)
            ops.append(dist.P2POp(dist.isend, t, self.prev, self.group))
        if recv_prev_T is not None and self.prev is not None:
            from_prev = torch.empty(recv_prev_T, self.H, device=self.device, dtype=self.dtype)
            ops.append(dist.P2POp(dist.irecv, from_prev, self.prev, self.group))
        if send_next is not None and self.next is not None:
            t = send_next.contiguous()
            keep.append(t)
            ops.append(dist.P2POp(dist.isend, t, self.next, self.group))
        if recv_next_T is not None and self.next is not None:
            from_next = torch.empty(recv_next_T, self.H, device=self.device, dtype=self.dtype)
            ops.append(dist.P2POp(dist.irecv, from_next, self.next, self.group))
        if ops:
            works = dist.batch_isend_irecv(ops)
            if self._pending_wgrad:
                # zero-bubble step: the exchange is in flight (the previous stage already has its input
                # gradient on the way) while this stage does the deferred weight-gradient products
                q, self._pending_wgrad = self._pending_wgrad, None
                OF.flush_wgrad(q)
            for r in works:
                r.wait()
        elif self._pending_wgrad:
            q, self._pending_wgrad = self._pending_wgrad, None
            OF.flush_wgrad(q)
        return from_prev, from_next

    # ---- compute of one micro-batch
    def _forward(self, mb, x_in, loss_fn, forward_only: bool):
        if self.m.is_first:
            y = self.m(mb["input_ids"], mb["pb"])
        else:
            if not forward_only:
                x_in.requires_grad_(True)
            y = self.m(x_in, mb["pb"])
        if self.m.is_last:
            return loss_fn(y, mb)
        if not forward_only:
            aux = self.m.aux_loss()      # MoE balancing loss of this stage: joins this stage's backward
            if aux is not None:
                self._aux[id(y)] = aux
        return y

    def _backward(self, x_in, y, dy):
        if self.schedule == "ZBH1":
            # input gradients only; the weight-gradient products wait in a queue that the next exchange runs
            # after it has posted this stage's send (``_p2p``)
            with OF.deferred_wgrad() as q:
                self._backward_now(y, dy)
            self._pending_wgrad = q
        else:
            self._backward_now(y, dy)
        return None if self.m.is_first else x_in.grad

    def _backward_now(self, y, dy):
        if self.m.is_last:
            y.backward()
        else:
            aux = self._aux.pop(id(y), None)
            if aux is not None:
                torch.autograd.backward([y, aux], [dy, torch.ones_like(aux)])
            else:
                y.backward(dy)

    def run(self, microbatches: list[dict[str, Any]], loss_fn: Optional[Callable] = None, forward_only: bool = False) -> list:
        """``microbatches``: dicts with ``input_ids`` [T] and ``pb`` (PackedBatch) plus whatever
        ``loss_fn(hidden, mb)`` needs; identical on every stage. Returns the per-micro-batch
        losses (training) or outputs (forward only) on the last stage and ``[]`` elsewhere."""
        M = len(microbatches)
        Ts = [mb["input_ids"].shape[0] for mb in microbatches]
        results: list = []
        if forward_only:
            with torch.no_grad():
                for i, mb in enumerate(microbatches):
                    x, _ = self._p2p(recv_prev_T=Ts[i])
                    y = self._forward(mb, x, loss_fn, True)
                    if self.m.is_last:
                        results.append(y)
                    else:
                        self._p2p(send_next=y)
            return results
        if self.schedule == "ZBH1":
            OF.SPLIT_BACKWARD = True
            try:
                return self._run_train(microbatches, loss_fn, M, Ts, results)
            finally:
                OF.SPLIT_BACKWARD = False
        return self._run_train(microbatches, loss_fn, M, Ts, results)

    def _run_train(self, microbatches, loss_fn, M, Ts, results):
        warm = M if self.schedule == "GPipe" else min(M, self.n - self.rank - 1)
        rest = M - warm
        inputs, outputs = [], []
        for i in range(warm):                              # warm-up forwards
            x, _ = self._p2p(recv_prev_T=Ts[i])
            y = self._forward(microbatches[i], x, loss_fn, False)
            self._p2p(send_next=None if self.m.is_last else y.detach())
            inputs.append(x)
            outputs.append(y)
        x = None
        if rest > 0:
            x, _ = self._p2p(recv_prev_T=Ts[warm])
        for k in range(rest):                              # steady state: one forward, one backward
            i = warm + k
            y = self._forward(microbatches[i], x, loss_fn, False)
            inputs.append(x)
            outputs.append(y)
            j = len(results)                               # oldest micro-batch still waiting for its backward
            _, dy = self._p2p(send_next=None if self.m.is_last else y.detach(), recv_next_T=Ts[j])
            xb, yb = inputs.pop(0), outputs.pop(0)
            if self.m.is_last:
                results.append(yb.detach())
            else:
                results.append(None)
            dx = self._backward(xb, yb, dy)
            if k == rest - 1:
                self._p2p(send_prev=dx)
                x = None
            else:
                x, _ = self._p2p(send_prev=dx, recv_prev_T=Ts[i + 1])
        while inputs:                                      # cool-down backwards
            j = len(results)
            _, dy = self._p2p(recv_next_T=Ts[j])
            xb, yb = inputs.pop(0), outputs.pop(0)
            results.append(yb.detach() if self.m.is_last else None)
            dx = self._backward(xb, yb, dy)
            self._p2p(send_prev=dx)
        if self._pending_wgrad:
            OF.flush_wgrad(self._pending_wgrad)
            self._pending_wgrad = None
        self.sync_tied_embedding_grads()
        return results if self.m.is_last else []

    def sync_tied_embedding_grads(self):
        """Tied input / output embeddings exist on the first and last stage: sum their grads."""
        m = self.m
        if self.n == 1 or not m.cfg.tie_word_embeddings or m.cfg.is_critic or not (m.is_first or m.is_last):
            return
        g = getattr(m.embed_tokens, "main_grad", None)
        if g is not None and m.embed_tokens.grad is not None:
            # the lookup's gradient arrives through autograd, the head's through the fp32 buffer: one sum
            g.add_(m.embed_tokens.grad.to(g.dtype))
            m.embed_tokens.grad = None
        if g is None:
            g = m.embed_tokens.grad
        if g is None:
            g = torch.zeros_like(m.embed_tokens)
            m.embed_tokens.grad = g
        peer = self.last_rank if m.is_first else self.first_rank
        other = torch.empty_like(g)
        mine = g.contiguous().clone()
        for r in dist.batch_isend_irecv([dist.P2POp(dist.isend, mine, peer, self.group), dist.P2POp(dist.irecv, other, peer, self.group)]):
            r.wait()
        g.add_(other)

    def broadcast_loss(self, loss: Optional[torch.Tensor]) -> torch.Tensor:
        """The last stage's scalar (statistics, early stopping) made known to every stage."""
        t = loss.detach().float().reshape(1).to(self.device) if self.m.is_last else torch.zeros(1, device=self.device)
        dist.broadcast(t, src=self.last_rank, group=self.group)
        return t[0]


# --------------------------------------------------------------------------- virtual stages
def stage_of(rank: int, chunk: int, n_ranks: int, placement: str = "loop") -> int:
    """Global stage of chunk ``chunk`` on rank ``rank``: ``loop`` walks the ranks once per chunk (stage
    ``chunk * P + rank``); ``v`` (two chunks) goes down the ranks and back up, so rank 0 holds the first AND the
    last stage and rank ``P - 1`` two consecutive ones."""
    if placement == "v":
        return rank if chunk == 0 else 2 * n_ranks - 1 - rank
    return chunk * n_ranks + rank


def owner_of(stage: int, n_ranks: int, placement: str = "loop") -> tuple[int, int]:
    """(rank, chunk) that holds ``stage``."""
    if placement == "v":
        return (stage, 0) if stage < n_ranks else (2 * n_ranks - 1 - stage, 1)
    return stage % n_ranks, stage // n_ranks


class InterleavedStages(nn.Module):
    """``V`` model chunks of one pipeline rank (virtual pipeline), placed by :func:`stage_of`. Presents the
    attributes the engine reads from a stage (first / last flags, embedding, heads, native parameter names)."""

    def __init__(self, cfg: ModelConfig, rank: int, n_ranks: int, n_chunks: int, dtype=torch.bfloat16, device="cpu", seed: Optional[int] = None,
                 init_full: Optional[Callable] = None, placement: str = "loop", tp: int = 1, tp_rank: int = 0):
        super().__init__()
        if placement == "v" and n_chunks != 2:
            raise ValueError("the V-shaped placement has exactly two chunks per rank")
        self.cfg, self.dtype, self.stage, self.n_stages = cfg, dtype, rank, n_ranks
        self.n_chunks, self.placement = n_chunks, placement
        total = n_ranks * n_chunks
        self.chunks = nn.ModuleList([PipelineStage(cfg, stage_of(rank, v, n_ranks, placement), total, dtype=dtype, device=device, seed=seed,
                                                   init_full=init_full, tp=tp, tp_rank=tp_rank) for v in range(n_chunks)])
        self.is_first = any(c.is_first for c in self.chunks)
        self.is_last = any(c.is_last for c in self.chunks)
        if self.is_first and self.is_last and n_ranks > 1 and cfg.tie_word_embeddings and not cfg.is_critic:
            # first and last stage on one rank (V placement): the tied embedding is ONE parameter used twice
            self.chunks[-1].embed_tokens = self.chunks[0].embed_tokens
        self.gradient_checkpointing = False

    @property
    def layers(self):
        return [l for c in self.chunks for l in c.layers]

    @property
    def embed_tokens(self):
        return self.chunks[0].embed_tokens if self.is_first else (self.chunks[-1].embed_tokens if self.is_last else None)

    @property
    def lm_head(self):
        return self.chunks[-1].lm_head

    @property
    def value_head(self):
        return self.chunks[-1].value_head

    @property
    def output_weight(self):
        return self.chunks[-1].output_weight

    def logprobs_entropy(self, hidden, labels, temperature: float = 1.0, chunk: int = 2048):
        return self.chunks[-1].logprobs_entropy(hidden, labels, temperature, chunk)

    def values(self, hidden):
        return self.chunks[-1].values(hidden)

    def aux_loss(self):
        return None   # each chunk's balancing loss joins that chunk's backward inside the runner

    def named_native_parameters(self, skip_tied_copy: bool = True):
        for c in self.chunks:
            yield from c.named_native_parameters(skip_tied_copy)

    def native_name(self, local_name: str) -> str:
        v, rest = local_name[len("chunks."):].split(".", 1)
        return self.chunks[int(v)].native_name(rest)


def interleaved_order(n_ranks: int, n_chunks: int, n_micro: int, rank: int) -> list[tuple[str, int, int]]:
    """Operation order ``[(F|B, micro-batch, chunk)]`` of one rank under interleaved 1F1B:
    forwards run in groups of ``P`` micro-batches per chunk, backwards mirror them with the chunks
    reversed, after a warm-up of ``2 (P - r - 1) + (V - 1) P`` forwards (``V = 1`` gives plain
    1F1B). ``n_micro`` must be a multiple of ``P`` when ``V > 1``."""
    P, V, M = n_ranks, n_chunks, n_micro
    if V > 1 and M % P:
        raise ValueError(f"interleaved schedule needs the number of micro-batches ({M}) to be a multiple of the pipeline size ({P})")
    total = M * V

    def fwd(k):
        return ("F", (k // (P * V)) * P + k % P, (k // P) % V) if V > 1 else ("F", k, 0)

    def bwd(k):
        return ("B", (k // (P * V)) * P + k % P, V - 1 - (k // P) % V) if V > 1 else ("B", k, 0)
    warm = min(total, (P - rank - 1) * 2 + (V - 1) * P) if V > 1 else min(total, P - rank - 1)
    ops, f, b = [], 0, 0
    for _ in range(warm):
        ops.append(fwd(f)); f += 1
    while f < total:
        ops.append(fwd(f)); f += 1
        ops.append(bwd(b)); b += 1
    while b < total:
        ops.append(bwd(b)); b += 1
    return ops


def build_timetable(n_ranks: int, n_chunks: int, n_micro: int, schedule: str = "Interleaved1F1B", forward_only: bool = False,
                    placement: str = "loop"):
    """Lock-step timetable every rank derives identically: per tick, the operation each rank runs
    (or None) and the messages ``(src, dst, kind, micro-batch, destination stage)`` delivered at the
    tick's start. An operation runs once its input has been delivered; a message is delivered the
    tick after it was produced. ``schedule="ZBV"`` (V placement) has no fixed order per rank: every tick a
    rank runs the ready backward of the oldest micro-batch, else a ready forward (the deeper chunk first, since it
    leads to a backward sooner) while fewer than ``2 P`` chunk activations are alive on it."""
    P, V, M = n_ranks, n_chunks, n_micro
    S = P * V
    if schedule == "ZBV" and not forward_only:
        return _greedy_timetable(P, V, M, placement)
    if forward_only or schedule == "GPipe":
        orders = [[("F", m, v) for v in range(V) for m in range(M)] + ([] if forward_only else [("B", m, v) for v in reversed(range(V)) for m in range(M)])
                  for _ in range(P)]
    else:
        orders = [interleaved_order(P, V, M, r) for r in range(P)]
    ptr = [0] * P
    have: set = set()                # (kind, micro-batch, stage) inputs present on their rank
    done: set = set()
    ticks = []
    pending: list = []               # messages produced in the previous tick
    while any(ptr[r] < len(orders[r]) for r in range(P)):
        for m in pending:
            have.add((m[2], m[3], m[4]))
        delivered, pending = pending, []
        row = []
        for r in range(P):
            op = orders[r][ptr[r]] if ptr[r] < len(orders[r]) else None
            if op is not None:
                kind, mb, v = op
                s = stage_of(r, v, P, placement)
                ready = (s == 0 or ("act", mb, s) in have) if kind == "F" else \
                    (("F", mb, s) in done and (s == S - 1 or ("grad", mb, s) in have))
                if not ready:
                    op = None
            row.append(op)
        if not delivered and all(o is None for o in row):
            raise RuntimeError(f"pipeline schedule cannot make progress (P={P}, V={V}, M={M})")
        for r, op in enumerate(row):
            if op is None:
                continue
            kind, mb, v = op
            s = stage_of(r, v, P, placement)
            ptr[r] += 1
            done.add((kind, mb, s))
            if kind == "F" and s < S - 1:
                pending.append((r, owner_of(s + 1, P, placement)[0], "act", mb, s + 1))
            if kind == "B" and s > 0:
                pending.append((r, owner_of(s - 1, P, placement)[0], "grad", mb, s - 1))
        ticks.append((row, delivered))
    if pending:
        ticks.append(([None] * P, pending))
    return ticks


def _greedy_timetable(P: int, V: int, M: int, placement: str):
    S = P * V
    todo = [{(k, m, v) for k in "FB" for m in range(M) for v in range(V)} for _ in range(P)]
    have: set = set()
    done: set = set()
    alive = [0] * P                  # chunk activations held (forwards run minus backwards run)
    cap = 2 * P
    ticks, pending = [], []
    while any(todo):
        for msg in pending:
            have.add((msg[2], msg[3], msg[4]))
        delivered, pending = pending, []
        row = []
        for r in range(P):
            best = None
            for (kind, mb, v) in todo[r]:
                s = stage_of(r, v, P, placement)
                if kind == "B":
                    if ("F", mb, s) in done and (s == S - 1 or ("grad", mb, s) in have):
                        key = (0, mb, -s)
                    else:
                        continue
                else:
                    if (s == 0 or ("act", mb, s) in have) and alive[r] < cap:
                        key = (1, -v, mb)
                    else:
                        continue
                if best is None or key < best[0]:
                    best = (key, (kind, mb, v))
            row.append(best[1] if best else None)
        if not delivered and all(o is None for o in row):
            cap += 1                 # the activation bound was the only obstacle: let one more forward in
            if cap > 2 * M * V + 2 * P:
                raise RuntimeError(f"pipeline schedule cannot make progress (P={P}, V={V}, M={M})")
            ticks.append(([None] * P, []))
            continue
        for r, op in enumerate(row):
            if op is None:
                continue
            kind, mb, v = op
            s = stage_of(r, v, P, placement)
            todo[r].discard(op)
            done.add((kind, mb, s))
            alive[r] += 1 if kind == "F" else -1
            if kind == "F" and s < S - 1:
                pending.append((r, owner_of(s + 1, P, placement)[0], "act", mb, s + 1))
            if kind == "B" and s > 0:
                pending.append((r, owner_of(s - 1, P, placement)[0], "grad", mb, s - 1))
        ticks.append((row, delivered))
    if pending:
        ticks.append(([None] * P, pending))
    return ticks


class ScheduledPipelineRunner:
    """Runs micro-batches through ``P`` ranks x ``V`` chunks following a timetable
    (:func:`build_timetable`): every tick starts with ONE batch of sends and receives that both
    sides derive from the same table, then each rank runs at most one forward or backward. Covers
    GPipe, 1F1B (``V = 1``) and interleaved 1F1B."""

    def __init__(self, stages, group, schedule: str = "Interleaved1F1B"):
        self.m = stages
        self.chunks = list(stages.chunks) if isinstance(stages, InterleavedStages) else [stages]
        self.group = group
        self.rank, self.n = dist.get_rank(group), dist.get_world_size(group)
        self.V = len(self.chunks)
        self.ranks = dist.get_process_group_ranks(group)
        self.first_rank, self.last_rank = self.ranks[0], self.ranks[-1]
        self.schedule = {"1f1b": "Interleaved1F1B", "interleaved1f1b": "Interleaved1F1B", "gpipe": "GPipe",
                         "interleavedzerobubble": "Interleaved1F1B", "zbh1": "Interleaved1F1B", "zbv": "ZBV",
                         "zbvzerobubble": "ZBV"}.get(schedule.lower())
        if self.schedule is None:
            raise ValueError(f"unknown pipeline schedule '{schedule}'")
        self.placement = getattr(stages, "placement", "loop")
        if (self.schedule == "ZBV") != (self.placement == "v"):
            raise ValueError("the ZBV schedule runs on the V-shaped placement (two chunks per rank), and only it does")
        # the rank that holds the last stage computes the loss (rank 0 under the V placement)
        self.loss_rank = owner_of(self.n * self.V - 1, self.n, self.placement)[0]
        # zero-bubble variant: same timetable, every backward leaves its weight-gradient products in a queue
        # that runs while the next tick's exchange (which carries this backward's input gradient) is in flight
        self.split_backward = schedule.lower() in ("interleavedzerobubble", "zbh1", "zbv", "zbvzerobubble")
        p = next(self.chunks[0].parameters())
        self.device, self.dtype, self.H = p.device, p.dtype, stages.cfg.hidden_size

    def run(self, microbatches: list[dict[str, Any]], loss_fn: Optional[Callable] = None, forward_only: bool = False) -> list:
        P, V, M = self.n, self.V, len(microbatches)
        S = P * V
        table = build_timetable(P, V, M, self.schedule, forward_only, self.placement)
        Ts = [mb["input_ids"].shape[0] for mb in microbatches]
        inbox: dict = {}             # (kind, mb, stage) -> tensor
        outbox: dict = {}
        saved: dict = {}             # (mb, chunk) -> (x_in, y, aux)
        results: list = [None] * M
        pending: Optional[list] = None
        OF.SPLIT_BACKWARD = self.split_backward and not forward_only
        try:
            return self._run_table(table, microbatches, loss_fn, forward_only, Ts, inbox, outbox, saved, results, pending)
        finally:
            OF.SPLIT_BACKWARD = False

    def _run_table(self, table, microbatches, loss_fn, forward_only, Ts, inbox, outbox, saved, results, pending):
        P, V = self.n, self.V
        S = P * V
        for row, delivered in table:
            ops, keep = [], []
            for (src, dst, kind, mb, s) in delivered:
                if src == self.rank and dst == self.rank:
                    # consecutive stages on one rank (the turn of the V placement): handed over in place
                    inbox[(kind, mb, s)] = outbox.pop((kind, mb, s)).contiguous()
                    continue
                if src == self.rank:
                    t = outbox.pop((kind, mb, s)).contiguous()
                    keep.append(t)
                    ops.append(dist.P2POp(dist.isend, t, self.ranks[dst], self.group))
                if dst == self.rank:
                    buf = torch.empty(Ts[mb], self.H, device=self.device, dtype=self.dtype)
                    inbox[(kind, mb, s)] = buf
                    ops.append(dist.P2POp(dist.irecv, buf, self.ranks[src], self.group))
            works = dist.batch_isend_irecv(ops) if ops else []
            if pending:
                OF.flush_wgrad(pending)
                pending = None
            for w in works:
                w.wait()
            op = row[self.rank]
            if op is None:
                continue
            kind, mb, v = op
            s = stage_of(self.rank, v, P, self.placement)
            chunk, data = self.chunks[v], microbatches[mb]
            if kind == "F":
                with torch.set_grad_enabled(not forward_only):
                    x = data["input_ids"] if s == 0 else inbox.pop(("act", mb, s))
                    if s > 0 and not forward_only:
                        x.requires_grad_(True)
                    y = chunk(x, data["pb"])
                    aux = None if forward_only else chunk.aux_loss()
                    if s == S - 1:
                        y = loss_fn(y, data)
                        if forward_only:
                            results[mb] = y
                    else:
                        outbox[("act", mb, s + 1)] = y.detach()
                if not forward_only:
                    saved[(mb, v)] = (x if s > 0 else None, y, aux)
            else:
                x, y, aux = saved.pop((mb, v))
                ctx = OF.deferred_wgrad() if self.split_backward else None
                q = ctx.__enter__() if ctx is not None else None
                try:
                    if s == S - 1:
                        (y if aux is None else y + aux).backward()
                        results[mb] = y.detach()
                    else:
                        dy = inbox.pop(("grad", mb, s))
                        if aux is not None:
                            torch.autograd.backward([y, aux], [dy, torch.ones_like(aux)])
                        else:
                            y.backward(dy)
                finally:
                    if ctx is not None:
                        ctx.__exit__(None, None, None)
                if q:
                    pending = (pending or []) + q
                if s > 0:
                    outbox[("grad", mb, s - 1)] = x.grad
        if pending:
            OF.flush_wgrad(pending)
        self.sync_tied_embedding_grads()
        return results if self.rank == self.loss_rank else []

    def sync_tied_embedding_grads(self):
        cfg = self.m.cfg
        if self.n * self.V == 1 or not cfg.tie_word_embeddings or cfg.is_critic or self.rank not in (0, self.loss_rank):
            return
        emb = self.chunks[0].embed_tokens if self.rank == 0 else self.chunks[-1].embed_tokens
        if self.loss_rank == 0 and self.n > 1:
            return                   # V placement: both uses share one parameter on rank 0, its gradient is already whole
        if self.n == 1:
            # first and last chunk live on the same rank: the two copies are one gradient
            a, b = self.chunks[0].embed_tokens, self.chunks[-1].embed_tokens
            if a is b:
                return
        g = getattr(emb, "main_grad", None)
        if g is not None and emb.grad is not None:
            g.add_(emb.grad.to(g.dtype))
            emb.grad = None
        if g is None:
            if emb.grad is None:
                emb.grad = torch.zeros_like(emb)
            g = emb.grad
        peer = self.last_rank if self.rank == 0 else self.first_rank
        other, mine = torch.empty_like(g), g.contiguous().clone()
        for w in dist.batch_isend_irecv([dist.P2POp(dist.isend, mine, peer, self.group), dist.P2POp(dist.irecv, other, peer, self.group)]):
            w.wait()
        g.add_(other)

    def broadcast_loss(self, loss: Optional[torch.Tensor]) -> torch.Tensor:
        lr = getattr(self, "loss_rank", self.n - 1)
        t = loss.detach().float().reshape(1).to(self.device) if self.rank == lr else torch.zeros(1, device=self.device)
        dist.broadcast(t, src=self.ranks[lr] if hasattr(self, "ranks") else self.last_rank, group=self.group)
        return t[0]
