"""Hybrid decoder layers: gated-delta-rule linear attention interleaved with gated full
attention (the Qwen3.5 text stack).

Three of every four layers replace softmax attention with a *gated delta rule*: per head a
``d_k x d_v`` state ``S`` is decayed, corrected towards the new value along the new key and read
with the query,

    S_t = exp(g_t) * S_{t-1} + k_t (beta_t * (v_t - (exp(g_t) S_{t-1})^T k_t))^T ,   o_t = S_t^T q_t ,

computed here in chunks of 64 tokens (the in-chunk dependence is a unit-lower-triangular solve,
the cross-chunk part a short recurrence over chunk states), on sequences un-packed into a padded
batch. q/k/v come from one projection followed by a depth-wise causal convolution (kernel 4) and
SiLU; the output is RMS-normalised per head, gated by ``silu(z)`` and projected back. The full
attention layers double the query projection into (query, gate), rotate only the first quarter
of each head and multiply the attention output by ``sigmoid(gate)``. All RMSNorm weights of the
stack (not the per-head norm inside the linear layers) are stored as offsets from one.

Everything here is plain differentiable PyTorch on top of the library's GEMM entry point
(``ops.functional.linear``); the recurrence runs in fp32.

Reference: ``areal/experimental/models/archon/qwen3_5/model/model.py`` (gated delta net block,
gated attention, zero-centred RMSNorm), ``.../qwen3_5/model/rope.py`` (partial rotation),
``.../qwen3_5/model/state_dict_adapter.py`` (checkpoint names).
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import functional as OF
from .config import ModelConfig

CHUNK = 64


def rmsnorm_offset(x, w, eps: float, resid=None):
    """RMSNorm whose stored weight is an offset from one: ``y = x_hat * (1 + w)`` in fp32.
    Returns ``(normed, residual_stream)`` like ``ops.functional.rmsnorm``."""
    if resid is not None:
        x = (x.float() + resid.float()).to(x.dtype)
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * (1.0 + w.float())
    return y.to(x.dtype), x


def partial_rope(x, pos, cos, sin, rotary_dim: int):
    """Rotates the first ``rotary_dim`` features of every head of ``x`` [T, heads, D]; ``cos`` /
    ``sin`` are tables of ``rotary_dim / 2`` frequencies."""
    if rotary_dim >= x.shape[-1]:
        return OF.rope_ref(x, pos.long(), cos, sin)
    rot = OF.rope_ref(x[..., :rotary_dim], pos.long(), cos, sin)
    return torch.cat([rot, x[..., rotary_dim:]], dim=-1)


def sdpa_varlen(q, k, v, cu_seqlens, scale: float):
    """Causal attention per packed sequence through ``scaled_dot_product_attention`` (any head size)."""
    cu = cu_seqlens.tolist()
    rep = q.shape[1] // k.shape[1]
    out = torch.empty_like(q)
    for a, b in zip(cu[:-1], cu[1:]):
        if b <= a:
            continue
        qi = q[a:b].transpose(0, 1).unsqueeze(0)
        ki = k[a:b].transpose(0, 1).repeat_interleave(rep, dim=0).unsqueeze(0)
        vi = v[a:b].transpose(0, 1).repeat_interleave(rep, dim=0).unsqueeze(0)
        out[a:b] = F.scaled_dot_product_attention(qi, ki, vi, is_causal=True, scale=scale)[0].transpose(0, 1)
    return out


# ----------------------------------------------------------------------------- packed <-> padded
def pad_index(cu_seqlens: torch.Tensor, total: int, max_len: int):
    """Index tensors between a packed token axis [T] and a padded batch [B, max_len]:
    ``gather`` [B, max_len] (row ``total`` = padding) and ``scatter`` [T] (flat position of token t).
    Built on the device without a host round trip."""
    cu = cu_seqlens.long()
    B = cu.numel() - 1
    dev = cu.device
    pos = torch.arange(max_len, device=dev)[None, :]
    lens = (cu[1:] - cu[:-1])[:, None]
    gather = torch.where(pos < lens, cu[:-1, None] + pos, torch.full_like(pos, total))
    t = torch.arange(total, device=dev)
    seq = torch.searchsorted(cu[1:].contiguous(), t, right=True).clamp(max=B - 1)
    pis = (t - cu[seq]).clamp(min=0, max=max_len - 1)
    return gather, seq * max_len + pis, pis


def causal_conv_packed(x, w, pos_in_seq):
    """Depth-wise causal convolution over a packed token axis that never reads across a sequence
    start. x [T, C]; w [C, K] with tap K-1 on the current token; returns silu(conv) in x's dtype."""
    K = w.shape[1]
    wf = w.float()
    xf = x.float()
    out = xf * wf[:, K - 1]
    for j in range(1, K):
        shifted = torch.roll(xf, j, 0)
        out = out + torch.where((pos_in_seq >= j)[:, None], shifted, torch.zeros_like(shifted)) * wf[:, K - 1 - j]
    return F.silu(out).to(x.dtype)


# ----------------------------------------------------------------------------- the delta rule
def gated_delta_rule_recurrent(q, k, v, g, beta, state=None):
    """Token-by-token statement of the rule (fp32): q, k [B, L, h, dk]; v [B, L, h, dv]; g (log
    decay) and beta [B, L, h]. Returns (o [B, L, h, dv], final state [B, h, dk, dv]). Used for
    decoding one token at a time and as the oracle of the chunked form."""
    B, L, h, dk = k.shape
    dv = v.shape[-1]
    q, k, v, g, beta = (t.float() for t in (q, k, v, g, beta))
    q = q * dk ** -0.5
    S = torch.zeros(B, h, dk, dv, device=q.device) if state is None else state.float()
    outs = []
    for t in range(L):
        S = S * g[:, t].exp()[..., None, None]
        mem = (S * k[:, t][..., None]).sum(-2)
        delta = (v[:, t] - mem) * beta[:, t][..., None]
        S = S + k[:, t][..., None] * delta[..., None, :]
        outs.append((S * q[:, t][..., None]).sum(-2))
    return torch.stack(outs, 1), S


def gated_delta_rule_chunked(q, k, v, g, beta, chunk: int = CHUNK, state=None):
    """Same function in chunks: inside a chunk the corrected values solve a unit lower
    triangular system, across chunks only the ``dk x dv`` state is carried."""
    B, L, h, dk = k.shape
    dv = v.shape[-1]
    pad = (-L) % chunk
    q, k, v = (F.pad(t.float().transpose(1, 2), (0, 0, 0, pad)) for t in (q, k, v))      # [B, h, Lp, d]
    g, beta = (F.pad(t.float().transpose(1, 2), (0, pad)) for t in (g, beta))             # [B, h, Lp]
    n = (L + pad) // chunk
    q = q * dk ** -0.5
    q, k, v = (t.reshape(B, h, n, chunk, t.shape[-1]) for t in (q, k, v))
    g, beta = g.reshape(B, h, n, chunk), beta.reshape(B, h, n, chunk)
    gc = g.cumsum(-1)
    decay = (gc[..., :, None] - gc[..., None, :]).tril().exp().tril()                     # exp(gc_i - gc_j), i >= j
    kb, vb = k * beta[..., None], v * beta[..., None]
    eye = torch.eye(chunk, device=q.device, dtype=torch.float32)
    M = (kb @ k.transpose(-1, -2) * decay).tril(-1)
    Tm = torch.linalg.solve_triangular(eye + M, eye.expand_as(M).contiguous(), upper=False)
    u = Tm @ vb
    w = Tm @ (kb * gc.exp()[..., None])
    S = torch.zeros(B, h, dk, dv, device=q.device) if state is None else state.float()
    outs = []
    for i in range(n):
        qi, ki, gi = q[:, :, i], k[:, :, i], gc[:, :, i]
        attn = (qi @ ki.transpose(-1, -2) * decay[:, :, i]).tril()
        v_new = u[:, :, i] - w[:, :, i] @ S
        outs.append((qi * gi.exp()[..., None]) @ S + attn @ v_new)
        S = S * gi[..., -1].exp()[..., None, None] + (ki * (gi[..., -1:] - gi).exp()[..., None]).transpose(-1, -2) @ v_new
    o = torch.stack(outs, 2).reshape(B, h, n * chunk, dv)[:, :, :L]
    return o.transpose(1, 2), S


def l2norm(x, eps: float = 1e-6):
    xf = x.float()
    return xf * torch.rsqrt((xf * xf).sum(-1, keepdim=True) + eps)


class GatedDeltaNet(nn.Module):
    def __init__(self, cfg: ModelConfig, dtype, device):
        super().__init__()
        self.cfg = cfg
        H = cfg.hidden_size
        self.nk, self.nv = cfg.linear_num_key_heads, cfg.linear_num_value_heads
        self.dk, self.dv = cfg.linear_key_head_dim, cfg.linear_value_head_dim
        self.key_dim, self.value_dim = self.nk * self.dk, self.nv * self.dv
        conv_dim = 2 * self.key_dim + self.value_dim
        mk = lambda *s: nn.Parameter(torch.empty(*s, dtype=dtype, device=device))  # noqa: E731
        self.in_proj_qkv = mk(conv_dim, H)
        self.in_proj_z = mk(self.value_dim, H)
        self.in_proj_ba = mk(2 * self.nv, H)          # rows [0, nv): beta logits; [nv, 2nv): decay inputs
        self.conv1d = mk(conv_dim, cfg.linear_conv_kernel_dim)
        self.dt_bias = mk(self.nv)
        self.A_log = mk(self.nv)
        self.norm = mk(self.dv)
        self.out_proj = mk(H, self.value_dim)

    capture = None      # a list: forward() appends (pre-convolution projections [T, C], final states [B, nv, dk, dv])

    def _inputs(self, x: torch.Tensor):
        """Projections of ``x`` [T, H]: pre-convolution q|k|v, output gate z, write strength beta, log decay g."""
        ba = F.linear(x, self.in_proj_ba).float()                 # 2 * nv columns: too narrow for the tiled GEMM
        beta = ba[:, : self.nv].sigmoid()
        g = -self.A_log.float().exp() * F.softplus(ba[:, self.nv:] + self.dt_bias.float())
        return OF.linear(x, self.in_proj_qkv), OF.linear(x, self.in_proj_z), beta, g

    def _heads(self, mixed: torch.Tensor, nk: Optional[int] = None, nv: Optional[int] = None):
        """Post-convolution q|k|v [T, C] -> unit-norm q, k [T, nv, dk] and v [T, nv, dv] (fp32); ``nk`` / ``nv``:
        the head counts present in ``mixed`` (a slice of the heads under sequence parallelism)."""
        nk, nv = nk or self.nk, nv or self.nv
        T = mixed.shape[0]
        q, k, v = torch.split(mixed, [nk * self.dk, nk * self.dk, nv * self.dv], dim=-1)
        q = l2norm(q.reshape(T, nk, self.dk))
        k = l2norm(k.reshape(T, nk, self.dk))
        rep = nv // nk
        if rep > 1:
            q, k = q.repeat_interleave(rep, dim=1), k.repeat_interleave(rep, dim=1)
        return q, k, v.reshape(T, nv, self.dv).float()

    sp_group = None     # set by parallel.ulysses.install_ulysses: tokens split over the group outside this block
    sp_size = 1
    sp_rank = 0

    def _to_heads(self, pre, beta, g):
        """Sequence-parallel exchange in front of the rule: local rows, all heads -> all rows, this rank's heads
        (``[t, C] -> [n t, C / n]`` for q | k | v, ``[t, nv] -> [n t, nv / n]`` for beta and g) plus the
        convolution taps of the local channels. The convolution and the recurrence run along the sequence, so they
        need whole sequences; heads are independent (role of the cp2hp all-to-all of the reference's linear
        attention, areal/models/mcore/lightning_attention.py:134-172)."""
        from ..parallel.ulysses import SeqToHead

        n, r, grp = self.sp_size, self.sp_rank, self.sp_group
        t = pre.shape[0]
        q, k, v = torch.split(pre, [self.key_dim, self.key_dim, self.value_dim], dim=-1)
        qf = SeqToHead.apply(q.reshape(t, self.nk, self.dk), grp, n)
        kf = SeqToHead.apply(k.reshape(t, self.nk, self.dk), grp, n)
        vf = SeqToHead.apply(v.reshape(t, self.nv, self.dv), grp, n)
        T = qf.shape[0]
        mixed = torch.cat([qf.reshape(T, -1), kf.reshape(T, -1), vf.reshape(T, -1)], dim=-1)
        bf = SeqToHead.apply(beta.reshape(t, self.nv, 1), grp, n).reshape(T, -1)
        gf = SeqToHead.apply(g.reshape(t, self.nv, 1), grp, n).reshape(T, -1)
        kq, kv_ = self.key_dim // n, self.value_dim // n
        w = self.conv1d
        taps = torch.cat([w[r * kq:(r + 1) * kq], w[self.key_dim + r * kq: self.key_dim + (r + 1) * kq],
                          w[2 * self.key_dim + r * kv_: 2 * self.key_dim + (r + 1) * kv_]], dim=0)
        return mixed, bf, gf, taps

    def _output(self, o: torch.Tensor, z: torch.Tensor, dtype) -> torch.Tensor:
        """Per-head RMSNorm of the rule's output [T, nv, dv] (fp32), gate by silu(z), project back."""
        T = o.shape[0]
        o = o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + self.cfg.rms_norm_eps)
        o = (self.norm.float() * o.to(dtype).float()) * F.silu(z.reshape(T, self.nv, self.dv).float())
        return OF.linear(o.to(dtype).reshape(T, self.value_dim), self.out_proj)

    def forward(self, x: torch.Tensor, pb) -> torch.Tensor:
        T = x.shape[0] * (self.sp_size if self.sp_group is not None else 1)      # tokens the rule sees
        max_len = int(pb.max_seqlen) or int((pb.cu_seqlens[1:] - pb.cu_seqlens[:-1]).max())
        key = (T, max_len)
        idx = getattr(pb, "_pad_index", None)
        if idx is None or idx[0] != key:
            idx = (key, pad_index(pb.cu_seqlens, T, max_len))
            pb._pad_index = idx
        gather, scatter, pis = idx[1]
        pre, z, beta, g = self._inputs(x)
        nk, nv, taps = self.nk, self.nv, self.conv1d
        if self.sp_group is not None:
            pre, beta, g, taps = self._to_heads(pre, beta, g)
            nk, nv = self.nk // self.sp_size, self.nv // self.sp_size
        q, k, v = self._heads(causal_conv_packed(pre, taps, pis), nk, nv)

        def padded(t):                                            # [T, ...] -> [B, max_len, ...]
            zero = torch.zeros((1,) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
            return torch.cat([t, zero], 0)[gather]
        # rows past a sequence's end carry k = 0 and beta = 0: they leave its state untouched
        o, S = gated_delta_rule_chunked(padded(q), padded(k), padded(v), padded(g), padded(beta))
        if self.capture is not None:
            self.capture.append((pre, S))
        o = o.reshape(-1, nv, self.dv)[scatter]
        if self.sp_group is not None:
            from ..parallel.ulysses import HeadToSeq

            o = HeadToSeq.apply(o.contiguous(), self.sp_group, self.sp_size)      # back to local rows, all heads
        return self._output(o, z, x.dtype)

    def step(self, x: torch.Tensor, conv_state: torch.Tensor, S: torch.Tensor):
        """One new token per sequence: x [B, H], conv_state [B, K-1, C] (the last pre-convolution
        rows), S [B, nv, dk, dv]. Returns (y [B, H], new conv_state, new S)."""
        pre, z, beta, g = self._inputs(x)
        window = torch.cat([conv_state.to(pre.dtype), pre[:, None, :]], dim=1)                # [B, K, C]
        mixed = F.silu((window.float() * self.conv1d.float().t()[None]).sum(1)).to(x.dtype)
        q, k, v = self._heads(mixed)
        o, S = gated_delta_rule_recurrent(q[:, None], k[:, None], v[:, None], g[:, None], beta[:, None], S)
        return self._output(o[:, 0], z, x.dtype), window[:, 1:], S


class GatedAttention(nn.Module):
    """Full attention of the hybrid stack: (query, gate) from one projection, offset QK-norm,
    partial rotation, sigmoid output gate."""

    def __init__(self, cfg: ModelConfig, dtype, device):
        super().__init__()
        self.cfg = cfg
        H, D = cfg.hidden_size, cfg.head_dim
        self.nq, self.nkv, self.D = cfg.num_heads, cfg.num_kv_heads, D
        self.q_proj = nn.Parameter(torch.empty(self.nq * 2 * D, H, dtype=dtype, device=device))   # per head: D query rows, D gate rows
        self.kv_proj = nn.Parameter(torch.empty(2 * self.nkv * D, H, dtype=dtype, device=device))
        self.o_proj = nn.Parameter(torch.empty(H, self.nq * D, dtype=dtype, device=device))
        self.q_norm = nn.Parameter(torch.zeros(D, dtype=dtype, device=device))
        self.k_norm = nn.Parameter(torch.zeros(D, dtype=dtype, device=device))

    capture = None      # a list: forward() appends (k [T, nkv, D] after norm and rotation, v [T, nkv, D])

    def _qkv(self, x: torch.Tensor, positions, cos, sin):
        T, D, nq, nkv, eps = x.shape[0], self.D, self.nq, self.nkv, self.cfg.rms_norm_eps
        qg = OF.linear(x, self.q_proj).view(T, nq, 2 * D)
        q, gate = qg[..., :D], qg[..., D:].reshape(T, nq * D)
        kv = OF.linear(x, self.kv_proj)
        k, v = kv[:, : nkv * D].view(T, nkv, D), kv[:, nkv * D:].view(T, nkv, D)
        q, _ = rmsnorm_offset(q, self.q_norm, eps)
        k, _ = rmsnorm_offset(k, self.k_norm, eps)
        rd = self.cfg.rotary_dim
        q = partial_rope(q, positions, cos, sin, rd).to(x.dtype)
        k = partial_rope(k, positions, cos, sin, rd).to(x.dtype)
        return q, k, v, gate

    def step(self, x: torch.Tensor, positions, cos, sin, ks: list, vs: list):
        """One new token per sequence: x [B, H]; ``ks[i]`` / ``vs[i]`` [L_i, nkv, D] are sequence
        i's cached keys / values. Returns (y [B, H], new keys [B, nkv, D], new values)."""
        B, D, nq = x.shape[0], self.D, self.nq
        q, k, v, gate = self._qkv(x, positions, cos, sin)
        rep = nq // self.nkv
        outs = []
        for i in range(B):
            K = torch.cat([ks[i], k[i:i + 1]], 0).transpose(0, 1).repeat_interleave(rep, dim=0)      # [nq, L+1, D]
            V = torch.cat([vs[i], v[i:i + 1]], 0).transpose(0, 1).repeat_interleave(rep, dim=0)
            outs.append(F.scaled_dot_product_attention(q[i][None, :, None, :], K[None], V[None], scale=1.0 / math.sqrt(D))[0, :, 0])
        o = torch.stack(outs, 0).reshape(B, nq * D) * torch.sigmoid(gate.float()).to(x.dtype)
        return OF.linear(o, self.o_proj), k, v

    def forward(self, x: torch.Tensor, pb, cos, sin, attn_fn=None) -> torch.Tensor:
        T, D, nq, nkv = x.shape[0], self.D, self.nq, self.nkv
        q, k, v, gate = self._qkv(x, pb.position_ids, cos, sin)
        if self.capture is not None:
            self.capture.append((k, v))
        scale = 1.0 / math.sqrt(D)
        if attn_fn is not None:
            o = attn_fn(q, k, v)
        elif getattr(self, "sp_size", 1) > 1:
            from ..parallel.ulysses import ulysses_attention

            impl = OF.attention if (not x.is_cuda or D in (64, 128)) else (lambda q_, k_, v_, cu, causal, sc, ti: sdpa_varlen(q_, k_, v_, cu, sc))
            o = ulysses_attention(self, q.contiguous(), k.contiguous(), v.contiguous(), pb.cu_seqlens, True, scale, pb.tile_info, impl)
        elif x.is_cuda and D in (64, 128):
            o = OF.attention(q.contiguous(), k.contiguous(), v.contiguous(), pb.cu_seqlens, True, scale, pb.tile_info)
        elif x.is_cuda:
            o = sdpa_varlen(q, k, v, pb.cu_seqlens, scale)
        else:
            o = OF.attention(q, k.contiguous(), v.contiguous(), pb.cu_seqlens, True, scale, pb.tile_info)
        o = o.reshape(T, nq * D) * torch.sigmoid(gate.float()).to(x.dtype)
        return OF.linear(o, self.o_proj)


class HybridDecoderLayer(nn.Module):
    """Drop-in for ``DecoderLayer`` (same call signature) with the token mixer chosen per layer."""

    tp_group = None
    moe_row_share = None     # (group, tp, rank), see DecoderLayer

    def __init__(self, cfg: ModelConfig, idx: int, dtype, device):
        super().__init__()
        from .decoder import DenseMLP

        self.cfg = cfg
        H = cfg.hidden_size
        self.input_layernorm = nn.Parameter(torch.zeros(H, dtype=dtype, device=device))
        self.post_attention_layernorm = nn.Parameter(torch.zeros(H, dtype=dtype, device=device))
        self.is_linear = cfg.layer_is_linear(idx)
        if self.is_linear:
            self.linear_attn = GatedDeltaNet(cfg, dtype, device)
        else:
            self.self_attn = GatedAttention(cfg, dtype, device)
        if cfg.layer_is_moe(idx):
            from .decoder import MoEMLP

            self.mlp = MoEMLP(cfg, dtype, device)        # routed experts + sigmoid-gated shared expert (Qwen3.5-MoE)
        else:
            self.mlp = DenseMLP(H, cfg.intermediate_size, dtype, device)

    def forward(self, h, resid, pb, cos, sin, attn_fn=None):
        eps = self.cfg.rms_norm_eps
        x, resid = rmsnorm_offset(h, self.input_layernorm, eps, resid)
        g = self.tp_group
        if g is not None:
            # tensor parallel: this rank holds a slice of the heads (of either mixer) and of the MLP columns
            from ..parallel.tp import copy_to_tp, reduce_from_tp

            x = copy_to_tp(x, g)
            h = reduce_from_tp(self.linear_attn(x, pb) if self.is_linear else self.self_attn(x, pb, cos, sin, attn_fn), g)
            x, resid = rmsnorm_offset(h, self.post_attention_layernorm, eps, resid)
            if self.moe_row_share is not None:     # whole experts: each TP rank routes its own share of the rows
                from ..parallel.tp import moe_on_row_share

                return moe_on_row_share(self.mlp, x, *self.moe_row_share), resid
            return reduce_from_tp(self.mlp(copy_to_tp(x, g)), g), resid
        h = self.linear_attn(x, pb) if self.is_linear else self.self_attn(x, pb, cos, sin, attn_fn)
        x, resid = rmsnorm_offset(h, self.post_attention_layernorm, eps, resid)
        return self.mlp(x), resid


@torch.no_grad()
def init_hybrid_parameters(model, gen: Optional[torch.Generator] = None) -> None:
    """Values that are not plain normal draws: offset norms start at zero, the per-head norm of
    the linear layers at one, the decay parameters as in the published initialisation
    (``A ~ U(0, 16)`` stored as a log, unit time-step bias)."""
    for name, p in model.named_parameters():
        if name.endswith("linear_attn.norm") or name.endswith("dt_bias"):
            p.fill_(1.0)
        elif name.endswith("A_log"):
            a = torch.rand(p.shape, device=p.device, dtype=torch.float32, generator=gen) * 16.0
            p.copy_(a.clamp_min(1e-3).log().to(p.dtype))
        elif name.endswith("norm") or name.endswith("layernorm"):
            p.zero_()


# ----------------------------------------------------------------------------- generation with carried state
class SequenceState:
    """What one sequence carries between decode steps: per linear layer the last ``K - 1``
    pre-convolution rows and the ``nv x dk x dv`` rule state, per full-attention layer its keys and
    values. ``length`` = tokens absorbed so far (the rotary position of the next token)."""

    __slots__ = ("layers", "length")

    def __init__(self, layers: list, length: int):
        self.layers, self.length = layers, length


@torch.no_grad()
def prefill_states(model, input_ids: torch.Tensor, cu_seqlens: torch.Tensor, max_seqlen: int):
    """One packed forward over whole sequences that also returns every sequence's carried state:
    ``(hidden [T, H], [SequenceState])``."""
    mixers = [(l.linear_attn if l.is_linear else l.self_attn) for l in model.layers]
    for mx in mixers:
        mx.capture = []
    try:
        hidden = model(input_ids, cu_seqlens, max_seqlen=max_seqlen)
        caps = [mx.capture[0] for mx in mixers]
    finally:
        for mx in mixers:
            mx.capture = None
    cu = cu_seqlens.tolist()
    states = []
    for si, (a, b) in enumerate(zip(cu[:-1], cu[1:])):
        per_layer = []
        for layer, cap in zip(model.layers, caps):
            if layer.is_linear:
                pre, S = cap
                keep = layer.linear_attn.conv1d.shape[1] - 1
                tail = pre[max(a, b - keep):b]
                if tail.shape[0] < keep:
                    tail = torch.cat([tail.new_zeros(keep - tail.shape[0], tail.shape[1]), tail], 0)
                per_layer.append((tail.clone(), S[si].clone()))
            else:
                k, v = cap
                per_layer.append((k[a:b].clone(), v[a:b].clone()))
        states.append(SequenceState(per_layer, b - a))
    return hidden, states


@torch.no_grad()
def decode_states(model, tokens: torch.Tensor, states: list) -> torch.Tensor:
    """Absorbs one new token per sequence (``tokens`` [B]) into ``states`` (updated in place) and
    returns the final normed hidden states [B, H]: constant work per token in the linear layers, one
    attention row in the full layers."""
    cfg = model.cfg
    dev = tokens.device
    pos = torch.tensor([st.length for st in states], dtype=torch.int32, device=dev)
    cos, sin = model.rope(dev, max(cfg.max_position_embeddings, int(pos.max()) + 2))
    h = OF.embedding(tokens, model.embed_tokens)
    resid = None
    eps = cfg.rms_norm_eps
    for li, layer in enumerate(model.layers):
        x, resid = rmsnorm_offset(h, layer.input_layernorm, eps, resid)
        if layer.is_linear:
            conv = torch.stack([st.layers[li][0] for st in states], 0)
            S = torch.stack([st.layers[li][1] for st in states], 0)
            h, conv, S = layer.linear_attn.step(x, conv, S)
            for i, st in enumerate(states):
                st.layers[li] = (conv[i], S[i])
        else:
            h, k, v = layer.self_attn.step(x, pos, cos, sin, [st.layers[li][0] for st in states], [st.layers[li][1] for st in states])
            for i, st in enumerate(states):
                st.layers[li] = (torch.cat([st.layers[li][0], k[i:i + 1]], 0), torch.cat([st.layers[li][1], v[i:i + 1]], 0))
        x, resid = rmsnorm_offset(h, layer.post_attention_layernorm, eps, resid)
        h = layer.mlp(x)
    for st in states:
        st.length += 1
    out, _ = rmsnorm_offset(h, model.norm, eps, resid)
    return out
