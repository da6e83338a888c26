"""Tensor parallelism for the decoder (training and inference).

Every rank builds the SAME model code with a rank-local architecture (heads / kv heads /
intermediate width divided by ``tp``): q/k/v/gate/up projections are split by output features
(column parallel), o/down projections by input features (row parallel), so each block needs
one sum over the TP group after the row-parallel product (forward) and one before the
column-parallel product (backward) — the conjugate pair ``copy_to_tp`` / ``reduce_from_tp``.
Norm weights, embeddings and the LM head stay replicated; their gradients are summed over the
group by :func:`allreduce_replicated_grads`.

The sums use NCCL here (the measured baseline); ``parallel/tp_fused.py`` replaces the
row-parallel product + sum by one GEMM kernel that writes its partial tiles straight into the
peers' buffers. Reference: ``areal/engine/fsdp_utils/parallel.py:227-385`` (Colwise / Rowwise
plans), ``areal/experimental/models/archon/qwen3/infra/parallelize.py:180``.
"""
from __future__ import annotations

import dataclasses
from typing import Optional

import torch
import torch.distributed as dist

from ..models.config import ModelConfig
from .weight_push import tp_layout_of


def local_config(cfg: ModelConfig, tp: int, expert_tp: bool = True) -> ModelConfig:
    """Architecture of one TP rank. ``expert_tp=False``: routed experts keep their full width (they are spread whole
    over an expert-parallel group instead; attention and dense MLPs are still sliced)."""
    if tp == 1:
        return cfg
    if cfg.num_heads % tp:
        raise ValueError(f"num_heads={cfg.num_heads} is not divisible by tp={tp}")
    if cfg.num_kv_heads % tp:
        raise ValueError(f"num_kv_heads={cfg.num_kv_heads} is not divisible by tp={tp} (kv-head replication is not supported)")
    if cfg.intermediate_size % tp or (cfg.num_experts and expert_tp and cfg.moe_intermediate_size % tp):
        raise ValueError("MLP width is not divisible by tp")
    kw = dict(num_heads=cfg.num_heads // tp, num_kv_heads=cfg.num_kv_heads // tp, intermediate_size=cfg.intermediate_size // tp)
    if cfg.num_experts and expert_tp:
        kw["moe_intermediate_size"] = cfg.moe_intermediate_size // tp
        Is = getattr(cfg, "shared_expert_intermediate_size", 0) or 0
        if Is:                                   # the shared expert is a dense MLP beside the routed ones: sliced the same way
            if Is % tp:
                raise ValueError("shared expert width is not divisible by tp")
            kw["shared_expert_intermediate_size"] = Is // tp
    if getattr(cfg, "layer_types", None):
        # linear-attention layers split by heads as well (key heads and value heads keep their grouping)
        nk, nv = cfg.linear_num_key_heads, cfg.linear_num_value_heads
        if nk % tp or nv % tp:
            raise ValueError(f"linear-attention heads ({nk} key, {nv} value) are not divisible by tp={tp}")
        kw.update(linear_num_key_heads=nk // tp, linear_num_value_heads=nv // tp)
    return dataclasses.replace(cfg, **kw)


def _block_rows(full: torch.Tensor, sizes: list[int], tp: int, rank: int) -> torch.Tensor:
    """``full`` is a stack of row blocks of ``sizes`` rows (q | k | v ...): rank ``rank``'s ``1 / tp`` of every block."""
    out, off = [], 0
    for n in sizes:
        out.append(full[off + rank * n // tp: off + (rank + 1) * n // tp])
        off += n
    return torch.cat(out, dim=0).contiguous()


def _unblock_rows(parts: list[torch.Tensor], sizes: list[int]) -> torch.Tensor:
    tp = len(parts)
    out = []
    off = 0
    for n in sizes:
        out += [p[off:off + n // tp] for p in parts]
        off += n // tp
    return torch.cat(out, dim=0)


def _hybrid_blocks(cfg: ModelConfig, name: str) -> Optional[list[int]]:
    """Row-block sizes (in the FULL model) of the head-sliced parameters of the hybrid (linear / gated attention)
    layers, ``None`` for every other parameter."""
    leaf = name.rsplit(".", 1)[-1]
    if ".linear_attn." in name:
        kd = cfg.linear_num_key_heads * cfg.linear_key_head_dim
        vd = cfg.linear_num_value_heads * cfg.linear_value_head_dim
        nv = cfg.linear_num_value_heads
        return {"in_proj_qkv": [kd, kd, vd], "conv1d": [kd, kd, vd], "in_proj_z": [vd], "in_proj_ba": [nv, nv], "dt_bias": [nv],
                "A_log": [nv]}.get(leaf)
    if leaf == "q_proj" and ".self_attn." in name:
        return [cfg.num_heads * 2 * cfg.head_dim]
    if leaf == "kv_proj" and ".self_attn." in name:
        return [cfg.num_kv_heads * cfg.head_dim] * 2
    return None


def shard_tensor(cfg: ModelConfig, name: str, full: torch.Tensor, tp: int, rank: int, expert_tp: bool = True) -> torch.Tensor:
    """Rank-local slice of a full (native-named) parameter."""
    if tp == 1:
        return full
    leaf = name.rsplit(".", 1)[-1]
    if leaf in ("embed_tokens", "lm_head") or name.startswith("visual."):       # replicated here (vocab parallelism is separate)
        return full
    if getattr(cfg, "layer_types", None):
        blocks = _hybrid_blocks(cfg, name)
        if blocks is not None:
            return _block_rows(full, blocks, tp, rank)
        if leaf == "out_proj" and ".linear_attn." in name:
            C = full.shape[1]
            return full[:, rank * C // tp:(rank + 1) * C // tp].contiguous()
    if leaf in ("shared_gate_up", "shared_down", "shared_expert_gate"):
        if not expert_tp or leaf == "shared_expert_gate":
            return full                             # whole experts (row shares): the shared expert stays whole as well
        if leaf == "shared_gate_up":
            I = full.shape[0] // 2
            a, b = rank * I // tp, (rank + 1) * I // tp
            return torch.cat([full[a:b], full[I + a:I + b]], dim=0).contiguous()
        C = full.shape[1]
        return full[:, rank * C // tp:(rank + 1) * C // tp].contiguous()
    if full.dim() == 3:                             # stacked experts [E, rows, cols]
        if not expert_tp:
            return full
        if leaf == "w_gate_up":
            I = full.shape[1] // 2
            a, b = rank * I // tp, (rank + 1) * I // tp
            return torch.cat([full[:, a:b], full[:, I + a:I + b]], dim=1).contiguous()
        if leaf == "w_down":
            C = full.shape[2]
            return full[:, :, rank * C // tp:(rank + 1) * C // tp].contiguous()
        return full
    shape = tuple(full.shape) if full.dim() == 2 else (full.shape[0],)
    blocks = tp_layout_of(cfg, leaf, shape, tp)[rank]
    if full.dim() == 1:
        return torch.cat([full[r0:r1] for (r0, r1, _, _) in blocks]).contiguous()
    return torch.cat([full[r0:r1, c0:c1] for (r0, r1, c0, c1) in blocks], dim=0).contiguous()


def unshard_tensors(cfg: ModelConfig, name: str, parts: list[torch.Tensor], expert_tp: bool = True) -> torch.Tensor:
    """Inverse of :func:`shard_tensor` (checkpoint export, weight push to a TP=1 consumer)."""
    tp = len(parts)
    if tp == 1:
        return parts[0]
    leaf = name.rsplit(".", 1)[-1]
    p0 = parts[0]
    if (p0.dim() == 3 and not expert_tp) or name.startswith("visual."):
        return p0
    if leaf in ("shared_gate_up", "shared_down", "shared_expert_gate"):
        if not expert_tp or leaf == "shared_expert_gate":
            return p0
        if leaf == "shared_gate_up":
            h = p0.shape[0] // 2
            return torch.cat([p[:h] for p in parts] + [p[h:] for p in parts], dim=0)
        return torch.cat(parts, dim=1)
    if getattr(cfg, "layer_types", None):
        blocks = _hybrid_blocks(cfg, name)
        if blocks is not None:
            return _unblock_rows(parts, blocks)
        if leaf == "out_proj" and ".linear_attn." in name:
            return torch.cat(parts, dim=1)
    if leaf in ("embed_tokens", "lm_head") or (p0.dim() == 1 and leaf != "qkv_bias") or leaf in ("router",):
        return p0
    if p0.dim() == 3:
        if leaf == "w_gate_up":
            h = p0.shape[1] // 2
            return torch.cat([p[:, :h] for p in parts] + [p[:, h:] for p in parts], dim=1)
        if leaf == "w_down":
            return torch.cat(parts, dim=2)
        return p0
    if leaf in ("o_proj", "down_proj"):
        return torch.cat(parts, dim=1)
    if leaf == "gate_up_proj":
        h = p0.shape[0] // 2
        return torch.cat([p[:h] for p in parts] + [p[h:] for p in parts], dim=0)
    if leaf in ("qkv_proj", "qkv_bias"):
        D = cfg.head_dim
        nq, nkv = cfg.num_heads // tp * D, cfg.num_kv_heads // tp * D
        return torch.cat([p[:nq] for p in parts] + [p[nq:nq + nkv] for p in parts] + [p[nq + nkv:] for p in parts], dim=0)
    return p0


class _CopyToTP(torch.autograd.Function):
    """Identity forward, sum over the TP group backward (input of a column-parallel product)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        dist.all_reduce(g, group=ctx.group)
        return g, None


class _ReduceFromTP(torch.autograd.Function):
    """Sum over the TP group forward, identity backward (output of a row-parallel product)."""

    @staticmethod
    def forward(ctx, x, group):
        x = x.contiguous()
        dist.all_reduce(x, group=group)
        return x

    @staticmethod
    def backward(ctx, g):
        return g, None


def copy_to_tp(x, group):
    return _CopyToTP.apply(x, group) if group is not None else x


def reduce_from_tp(x, group):
    return _ReduceFromTP.apply(x, group) if group is not None else x


def _gather_rows_uneven(x: torch.Tensor, T: int, group, tp: int) -> torch.Tensor:
    """Rank r holds rows [T r // tp, T (r + 1) // tp) of a [T, ...] tensor; returns all of it."""
    per = -(-T // tp)
    pad = x.new_zeros((per,) + tuple(x.shape[1:]))
    pad[: x.shape[0]] = x
    parts = [torch.empty_like(pad) for _ in range(tp)]
    dist.all_gather(parts, pad, group=group)
    return torch.cat([parts[r][: T * (r + 1) // tp - T * r // tp] for r in range(tp)], dim=0)


class _SliceRows(torch.autograd.Function):
    """This rank's share of rows that every TP rank holds (forward); the shares' gradients gathered back (backward)."""

    @staticmethod
    def forward(ctx, x, group, tp, rank):
        ctx.group, ctx.tp, ctx.T = group, tp, x.shape[0]
        return x[x.shape[0] * rank // tp: x.shape[0] * (rank + 1) // tp]

    @staticmethod
    def backward(ctx, g):
        return _gather_rows_uneven(g.contiguous(), ctx.T, ctx.group, ctx.tp), None, None, None


class _GatherRows(torch.autograd.Function):
    """Inverse of :class:`_SliceRows`: every rank ends up with all rows; each keeps its own rows' gradient (the
    gradient of the gathered tensor is the same on every TP rank)."""

    @staticmethod
    def forward(ctx, x, group, tp, rank, T):
        ctx.a, ctx.b = T * rank // tp, T * (rank + 1) // tp
        return _gather_rows_uneven(x.contiguous(), T, group, tp)

    @staticmethod
    def backward(ctx, g):
        return g[ctx.a:ctx.b], None, None, None, None


def moe_on_row_share(mlp, x: torch.Tensor, group, tp: int, rank: int) -> torch.Tensor:
    """A mixture-of-experts block whose experts are NOT sliced over the TP group: the group's ranks hold the same
    ``x``, so each routes its own share of the rows through the (expert-parallel) block and the outputs are gathered.
    Role of the attention-TP / expert-EP folding of the reference's hybrid layouts
    (``areal/api/alloc_mode.py:955-1054``, Megatron's ``expert_tensor_parallel_size=1``)."""
    T = x.shape[0]
    return _GatherRows.apply(mlp(_SliceRows.apply(x, group, tp, rank)), group, tp, rank, T)


def install_tp(model, group, tp_size: int, tp_rank: int, sequence_parallel: bool = False, fused=None, expert_tp: bool = True):
    """Marks every decoder layer of a rank-local model as tensor parallel. Default: the layer's forward brackets
    attention and MLP with the conjugate pair (identity / all-reduce) and every rank carries all tokens.
    ``sequence_parallel``: the residual stream is split by rows over the group as well (each rank holds ``T / P``
    tokens between the blocks; norms, residual adds and the LM head run on local rows only); the QKV and gate/up
    projections gather the rows in front of their product and the output / down projections reduce-scatter their
    result, as ONE kernel each when ``fused`` (a ``tp_fused.FusedTPLinear``) is given. Reference: Megatron's
    sequence-parallel linear layers, which ``areal/engine/megatron_engine.py`` turns on with tensor parallelism."""
    on = tp_size > 1
    for layer in model.layers:
        if sequence_parallel and on:
            if type(layer.mlp).__name__ != "DenseMLP":
                raise NotImplementedError("sequence-parallel tensor parallelism covers dense MLP layers")
            layer.tp_group = None
            layer.self_attn.tp_sp = layer.mlp.tp_sp = (group, fused)
        else:
            layer.tp_group = group if on else None
            if on and not expert_tp and hasattr(layer.mlp, "w_gate_up"):
                layer.moe_row_share = (group, tp_size, tp_rank)
                layer.mlp.aux_scale = 1.0 / tp_size         # every TP rank adds the balancing loss of its own share
    model.tp_expert_tp = bool(expert_tp)
    model.tp_group, model.tp_size, model.tp_rank = (group if on else None), tp_size, tp_rank
    model.tp_sequence_parallel = bool(sequence_parallel and on)
    return model


def replicated_parameter_names(model) -> list[str]:
    """Parameters every TP rank holds in full (their gradients must be summed over the group)."""
    out = []
    for n, p in model.named_parameters():
        leaf = n.rsplit(".", 1)[-1]
        whole_shared = not getattr(model, "tp_expert_tp", True) and leaf in ("shared_gate_up", "shared_down")
        if p.dim() == 1 and leaf not in ("qkv_bias", "dt_bias", "A_log") or leaf in ("embed_tokens", "lm_head", "router", "value_head", "shared_expert_gate") \
                or n.startswith("visual.") or whole_shared:
            out.append(n)            # (the image tower of a vision-language model is not sliced: every rank runs all of it)
    return out


def partial_grad_names(model) -> set[str]:
    """Replicated parameters whose gradient on one TP rank is only that rank's part (per-head norms, routers; every
    replicated parameter when the residual stream is split by rows): they must be summed over the TP group."""
    all_partial = getattr(model, "tp_sequence_parallel", False)
    out = set()
    for n in replicated_parameter_names(model):
        leaf = n.rsplit(".", 1)[-1]
        if all_partial or leaf in ("q_norm", "k_norm", "router", "shared_expert_gate", "shared_gate_up", "shared_down") or n.endswith("linear_attn.norm"):
            out.add(n)             # (a whole shared expert is listed as replicated only when each TP rank ran it on its own row share)
    return out


@torch.no_grad()
def allreduce_replicated_grads(model, group, grad_of=lambda p: getattr(p, "main_grad", None) if getattr(p, "main_grad", None) is not None else p.grad):
    """Sums the gradients of replicated parameters over the TP group (each rank saw only its
    heads' / columns' contribution to them ... except norms applied to full activations, which
    already hold the full gradient: those are averaged consistently by using SUM of 1/tp-scaled
    copies). Replicated weights consumed by full (unsharded) activations receive identical
    gradients on every rank, so they are left alone; per-head norms (q_norm / k_norm) see only
    local heads and are summed."""
    if group is None:
        return
    params = dict(model.named_parameters())
    # with the residual stream split by rows every replicated parameter saw only this rank's tokens (or heads)
    all_partial = getattr(model, "tp_sequence_parallel", False)
    for n in replicated_parameter_names(model):
        leaf = n.rsplit(".", 1)[-1]
        if all_partial or leaf in ("q_norm", "k_norm", "router", "shared_expert_gate", "shared_gate_up", "shared_down") or n.endswith("linear_attn.norm"):     # (per-head norms saw the local heads only)
            g = grad_of(params[n])
            if g is not None:
                dist.all_reduce(g, group=group)


def load_sharded_from_full(model, cfg: ModelConfig, full_state: dict, tp: int, rank: int, expert_tp: bool = True):
    """Copies the rank-local slices of a full state dict into a rank-local model."""
    with torch.no_grad():
        for n, p in model.named_parameters():
            p.copy_(shard_tensor(cfg, n, full_state[n], tp, rank, expert_tp).to(p.dtype))
    return model


# --------------------------------------------------------------------------- sequence-parallel TP
# Megatron-style sequence parallelism: between blocks, activations are sharded by rows
# ([T/P, H] per rank). A column-parallel product starts with an all-gather of the rows, a
# row-parallel product ends with a reduce-scatter; forward and input-gradient of both are
# exactly the two fused primitives of ``parallel/tp_fused.py`` (weight gradients gather once
# more with the library collective).
def _ag_rows(x, group):
    P = dist.get_world_size(group)
    out = x.new_empty((x.shape[0] * P,) + tuple(x.shape[1:]))
    if dist.get_backend(group) == "nccl":
        dist.all_gather_into_tensor(out, x.contiguous(), group=group)
    else:
        dist.all_gather(list(out.chunk(P, 0)), x.contiguous(), group=group)
    return out


def _rs_rows(x, group):
    P, r = dist.get_world_size(group), dist.get_rank(group)
    if dist.get_backend(group) == "nccl":
        out = x.new_empty((x.shape[0] // P,) + tuple(x.shape[1:]))
        dist.reduce_scatter_tensor(out, x.contiguous(), group=group)
        return out
    x = x.contiguous().clone()
    dist.all_reduce(x, group=group)
    return x.chunk(P, 0)[r].clone()


def _mm(a, b, b_mn: bool = False):
    """``a @ b^T`` (``b_mn``: ``a @ b``): the library GEMM on CUDA, plain matmul in the tensors' precision elsewhere."""
    if a.is_cuda:
        from ..ops import functional as OF

        return OF.gemm(a, b, b_mn=b_mn)
    return a @ (b if b_mn else b.t())


def _wgrad(w, dy_full, x_full):
    """dW = dy^T x, accumulated in fp32 into ``w.main_grad`` when the parameter carries one (returns None then)."""
    from ..ops import functional as OF

    mg = getattr(w, "main_grad", None)
    if not dy_full.is_cuda:
        g = dy_full.t() @ x_full
        if mg is not None:
            mg.add_(g.to(mg.dtype))
            return None
        return g
    if mg is not None:
        OF.gemm(dy_full, x_full, a_mn=True, b_mn=True, out=mg, epi=OF.EPI_F32_ACC)
        return None
    return OF.gemm(dy_full, x_full, a_mn=True, b_mn=True)


class _ColumnParallelSP(torch.autograd.Function):
    """``y[T, N/P] = gather_rows(x[T/P, K]) @ W[N/P, K]^T``."""

    @staticmethod
    def forward(ctx, x, w, group, fused):
        ctx.group, ctx.fused = group, fused
        ctx.save_for_backward(x, w)
        if fused is not None and x.is_cuda:
            return fused.allgather_gemm(x, w)
        return _mm(_ag_rows(x, group), w)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        g, fused = ctx.group, ctx.fused
        dy = dy.contiguous()
        if fused is not None and dy.is_cuda:
            dx = fused.gemm_reduce_scatter(dy, w, b_mn=True)           # rows of dy @ W that this rank owns
        else:
            dx = _rs_rows(_mm(dy, w, b_mn=True), g)
        dw = _wgrad(w, dy, _ag_rows(x, g)) if ctx.needs_input_grad[1] else None
        return dx, dw, None, None


class _RowParallelSP(torch.autograd.Function):
    """``y[T/P, N] = reduce_scatter_rows(x[T, K/P] @ W[N, K/P]^T)``."""

    @staticmethod
    def forward(ctx, x, w, group, fused):
        ctx.group, ctx.fused = group, fused
        ctx.save_for_backward(x, w)
        if fused is not None and x.is_cuda:
            return fused.gemm_reduce_scatter(x, w)
        return _rs_rows(_mm(x, w), group)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        g, fused = ctx.group, ctx.fused
        dy = dy.contiguous()
        if fused is not None and dy.is_cuda:
            dx = fused.allgather_gemm(dy, w, b_mn=True)                # gather_rows(dy) @ W
            dy_full = None
        else:
            dy_full = _ag_rows(dy, g)
            dx = _mm(dy_full, w, b_mn=True)
        dw = None
        if ctx.needs_input_grad[1]:
            dy_full = dy_full if dy_full is not None else _ag_rows(dy, g)
            dw = _wgrad(w, dy_full, x)
        return dx, dw, None, None


def column_parallel_sp(x_rows: torch.Tensor, w_local: torch.Tensor, group, fused=None) -> torch.Tensor:
    return _ColumnParallelSP.apply(x_rows, w_local, group, fused)


def row_parallel_sp(x_full: torch.Tensor, w_local: torch.Tensor, group, fused=None) -> torch.Tensor:
    return _RowParallelSP.apply(x_full, w_local, group, fused)
