"""Ulysses sequence parallelism: activations are sharded along the sequence everywhere except
inside attention, where an all-to-all turns the layout into "all tokens, a slice of heads".

Per layer forward: q, k, v ``[T/n, h, D] -> [T, h/n, D]`` (3 all-to-all), attention over the
full packed batch, output ``[T, hq/n, D] -> [T/n, hq, D]`` (1 all-to-all); autograd runs the
inverse exchanges. KV heads are replicated when ``n_kv_heads < n``. Same data movement as the
reference's ``areal/models/fsdp/ulysses.py:153-190`` and
``areal/models/transformers/ulyssess_patch.py:39-78``; here the exchange is expressed on the
packed token dimension so no padding per sequence is needed (the engine pads the packed
length to a multiple of ``n``).
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def _a2a(x: torch.Tensor, group) -> torch.Tensor:
    out = torch.empty_like(x)
    dist.all_to_all_single(out, x.contiguous(), group=group)
    return out


class SeqToHead(torch.autograd.Function):
    """[t, h, D] (local tokens, all heads) -> [n*t, h/n, D] (all tokens, local heads)."""

    @staticmethod
    def forward(ctx, x, group, n):
        ctx.group, ctx.n = group, n
        t, h, D = x.shape
        xs = x.reshape(t, n, h // n, D).permute(1, 0, 2, 3).contiguous()   # [n(dst), t, h/n, D]
        out = _a2a(xs, group)                                               # [n(src), t, h/n, D]
        return out.reshape(n * t, h // n, D)

    @staticmethod
    def backward(ctx, g):
        n = ctx.n
        T, hl, D = g.shape
        t = T // n
        gs = _a2a(g.reshape(n, t, hl, D).contiguous(), ctx.group)           # [n(head group), t, hl, D]
        return gs.permute(1, 0, 2, 3).reshape(t, n * hl, D), None, None


class HeadToSeq(torch.autograd.Function):
    """[n*t, h/n, D] -> [t, h, D]: inverse of :class:`SeqToHead`."""

    @staticmethod
    def forward(ctx, x, group, n):
        ctx.group, ctx.n = group, n
        T, hl, D = x.shape
        t = T // n
        out = _a2a(x.reshape(n, t, hl, D).contiguous(), group)
        return out.permute(1, 0, 2, 3).reshape(t, n * hl, D)

    @staticmethod
    def backward(ctx, g):
        n = ctx.n
        t, h, D = g.shape
        gs = g.reshape(t, n, h // n, D).permute(1, 0, 2, 3).contiguous()
        return _a2a(gs, ctx.group).reshape(n * t, h // n, D), None, None


def install_ulysses(model, group, sp_size: int, sp_rank: int) -> None:
    """Marks every attention module of ``model`` as sequence-parallel."""
    nq, nkv = model.cfg.num_heads, model.cfg.num_kv_heads
    if nq % sp_size != 0:
        raise ValueError(f"sequence-parallel degree {sp_size} must divide the number of query heads {nq}")
    for layer in model.layers:
        a = getattr(layer, "self_attn", None)
        if a is None:
            # linear-attention layer of a hybrid stack: the same exchange pair around the delta rule
            a = layer.linear_attn
            if a.nk % sp_size or a.nv % sp_size:
                raise ValueError(f"sequence-parallel degree {sp_size} must divide the linear-attention head counts ({a.nk}, {a.nv})")
        a.sp_group, a.sp_size, a.sp_rank = group, sp_size, sp_rank


def install_fused_ulysses(model, fused) -> None:
    """Routes every attention block of a sequence-parallel model through
    :func:`fused_ulysses_attention_block`; ``fused`` (one ``FusedUlyssesLinear``) is shared by all layers."""
    for layer in model.layers:
        layer.self_attn.sp_fused = fused


def ulysses_attention(attn_module, q, k, v, full_cu_seqlens, causal, scale, tile_info, attention_fn):
    """q/k/v: local slices ``[T/n, heads, D]``; returns the local slice of the output."""
    n, group = attn_module.sp_size, attn_module.sp_group
    nkv = k.shape[1]
    if nkv < n:
        rep = n // nkv
        k = k.repeat_interleave(rep, dim=1)
        v = v.repeat_interleave(rep, dim=1)
    elif nkv % n:
        raise ValueError("number of KV heads must divide or be divisible by the sequence-parallel degree")
    qf = SeqToHead.apply(q, group, n)
    kf = SeqToHead.apply(k.contiguous(), group, n)
    vf = SeqToHead.apply(v.contiguous(), group, n)
    o = attention_fn(qf, kf, vf, full_cu_seqlens, causal, scale, tile_info)
    return HeadToSeq.apply(o, group, n)


# --------------------------------------------------------------------------- fused exchanges (CUDA)
class _ProjectScatter(torch.autograd.Function):
    """``x_local[T/P, K] @ w[perm][N, K]^T`` landing as ``[T, N/P]`` on the column owners (one
    kernel). ``perm`` orders the weight rows (output columns) by owner. Backward:
    ``dx_local = gather_cols(dy) @ w[perm]`` (one kernel); ``dw`` is non-zero only in the rows this
    rank owns, ``dy^T @ gather_rows(x)``, and goes straight into ``w.main_grad`` when present."""

    @staticmethod
    def forward(ctx, x, w, fused, perm):
        ctx.fused = fused
        w_perm = w if perm is None else w.index_select(0, perm)
        ctx.save_for_backward(x, w, perm)
        return fused.project_scatter(x, w_perm).clone()

    @staticmethod
    def backward(ctx, dy):
        from ..ops import functional as OF

        x, w, perm = ctx.saved_tensors
        f = ctx.fused
        dy = dy.contiguous()
        w_perm = w if perm is None else w.index_select(0, perm)
        dx = f.gather_project(dy, w_perm, b_mn=True)                # [T/P, K]
        dw = None
        if ctx.needs_input_grad[1]:
            P, r = f.world, f.rank
            xf = x.new_empty(x.shape[0] * P, x.shape[1])
            dist.all_gather_into_tensor(xf, x.contiguous(), group=f.group)
            cpr = w.shape[0] // P
            own = OF.gemm(dy, xf, a_mn=True, b_mn=True)             # [N/P, K]: the rows this rank owns
            rows = torch.arange(r * cpr, (r + 1) * cpr, device=w.device) if perm is None else perm[r * cpr:(r + 1) * cpr]
            mg = getattr(w, "main_grad", None)
            if mg is not None:
                mg.index_add_(0, rows, own.to(mg.dtype))
            else:
                dw = torch.zeros_like(w)
                dw.index_copy_(0, rows, own)
        return dx, dw, None, None


class _GatherProject(torch.autograd.Function):
    """``gather_cols(o_full[T, K/P])[T/P, K] @ w[N, K]^T`` (one kernel). Backward:
    ``do_full = scatter_cols(dy @ w)`` (one kernel), ``dw = dy^T @ gathered``."""

    @staticmethod
    def forward(ctx, o_full, w, fused):
        ctx.fused = fused
        y = fused.gather_project(o_full, w)
        Kl = o_full.shape[1]
        M, K = y.shape[0], Kl * fused.world
        # the kernel's scratch holds the peers' panels; this rank's own panel is read in place
        a = fused.gathered[: M * K].view(M, K).clone()
        r = fused.rank
        a[:, r * Kl:(r + 1) * Kl] = o_full[r * M:(r + 1) * M]
        ctx.save_for_backward(a, w)
        return y

    @staticmethod
    def backward(ctx, dy):
        from ..ops import functional as OF

        a, w = ctx.saved_tensors
        f = ctx.fused
        dy = dy.contiguous()
        do = f.project_scatter(dy, w, b_mn=True).clone()            # [T, K/P]
        dw = None
        if ctx.needs_input_grad[1]:
            mg = getattr(w, "main_grad", None)
            if mg is not None:
                OF.gemm(dy, a, a_mn=True, b_mn=True, out=mg, epi=OF.EPI_F32_ACC)
            else:
                dw = OF.gemm(dy, a, a_mn=True, b_mn=True)
        return do, dw, None


def head_owner_permutation(nq: int, nkv: int, D: int, P: int, device) -> torch.Tensor:
    """Row order of a fused QKV weight such that rank r's column slice is ``[q heads of r | k
    heads of r | v heads of r]``."""
    nql, nkl = nq // P, nkv // P
    q = torch.arange(nq * D, device=device).view(P, nql * D)
    k = (nq * D + torch.arange(nkv * D, device=device)).view(P, nkl * D)
    v = ((nq + nkv) * D + torch.arange(nkv * D, device=device)).view(P, nkl * D)
    return torch.cat([q, k, v], dim=1).reshape(-1)


def fused_ulysses_attention_block(attn_module, x: torch.Tensor, pb, cos, sin, fused) -> torch.Tensor:
    """Whole attention block under Ulysses SP with both exchanges inside the projection
    kernels: x_local [T/P, H] -> y_local [T/P, H]. The QKV weight rows are re-ordered by head
    owner (one gather of the weight per call), so one projection kernel scatters every rank its
    ``[q | k | v]`` head group for all tokens, which the fused QK-norm + RoPE + attention kernels
    consume in place; the output projection pulls the other ranks' head outputs as it runs."""
    import math

    from ..ops import functional as OF

    a = attn_module
    P = fused.world
    D, nq, nkv = a.D, a.nq, a.nkv
    if nq % P or nkv % P or a.qkv_bias is not None:
        raise ValueError("the fused Ulysses block needs q and kv heads divisible by the group size and no QKV bias")
    nql, nkl = nq // P, nkv // P
    perm = getattr(a, "_sp_perm", None)
    if perm is None or perm.device != x.device:
        perm = a._sp_perm = head_owner_permutation(nq, nkv, D, P, x.device)
    qkv = _ProjectScatter.apply(x, a.qkv_proj, fused, perm)                  # [T, (nql + 2 nkl) D]: all tokens, my heads
    pos = getattr(pb, "full_position_ids", None)
    if pos is None:
        pos = pb.position_ids
    o = OF.qknorm_rope_attention(qkv, a.q_norm, a.k_norm, pos, cos, sin, pb.cu_seqlens, nql, nkl, D, a.cfg.rms_norm_eps,
                                 1.0 / math.sqrt(D), pb.tile_info)
    return _GatherProject.apply(o.reshape(o.shape[0], nql * D), a.o_proj, fused)
