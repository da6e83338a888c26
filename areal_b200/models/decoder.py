"""Decoder-only transformer (Qwen2 / Qwen2.5 / Qwen3 / Qwen3-MoE) on packed variable-length
batches, written against :mod:`areal_b200.ops.functional` so every hot op runs on the
sm_100a kernels on CUDA tensors and on the fp32 reference on CPU tensors.

Layout choices (differ from HF, converted by :mod:`areal_b200.models.hf_io`):

* ``qkv_proj.weight``   ``[(Hq + 2*Hkv) * D, H]``   q rows | k rows | v rows
* ``gate_up_proj.weight`` ``[2 * I, H]``            gate rows | up rows
* experts: ``w_gate_up [E, 2*Im, H]``, ``w_down [E, H, Im]``

The residual stream is carried separately from the sublayer output and added inside the
next RMSNorm kernel (one read-modify-write instead of two).

Reference behaviour: ``areal/experimental/models/archon/qwen2/model/model.py``,
``qwen3/model/model.py`` (RMSNorm in fp32, rotate-half RoPE, SwiGLU, QK-norm, GQA, tied
embeddings) and ``archon/moe/{router,moe,grouped_experts}.py``.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.utils.checkpoint import checkpoint

from ..ops import functional as OF
from .config import ModelConfig


class PackedBatch:
    """Per-forward metadata of a packed batch (built once, shared by all layers)."""

    def __init__(self, cu_seqlens: torch.Tensor, position_ids: torch.Tensor, total_tokens: int, max_seqlen: int = 0):
        self.cu_seqlens = cu_seqlens.to(torch.int32)
        self.position_ids = position_ids.to(torch.int32)
        self.total_tokens = total_tokens
        self.max_seqlen = max_seqlen
        self.tile_info = OF.attn_tile_table(self.cu_seqlens, total_tokens) if cu_seqlens.is_cuda else None


def _lin(mod, name: str, x: torch.Tensor, resid: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x @ W^T (+ resid)`` for ``W = mod.<name>`` plus its low-rank adapter when one is attached
    (and not merged into ``W``)."""
    ex = getattr(mod, "tp_exchange", None)
    if ex is not None and name in ("o_proj", "down_proj") and x.is_cuda and not torch.is_grad_enabled() and resid is None:
        # tensor-parallel inference: the partial product goes straight into every rank's receive
        # slots from the GEMM epilogue; the caller gets a handle that the next norm kernel sums
        return ex.linear_bcast(x if x.stride(-1) == 1 else x.contiguous(), getattr(mod, name))
    sp = getattr(mod, "tp_sp", None)
    if sp is not None:
        # tensor parallel with the residual stream split by rows: gather rows -> product, product -> reduce-scatter rows
        from ..parallel.tp import column_parallel_sp, row_parallel_sp

        if getattr(mod, "lora", None) is not None or getattr(mod, "use_fp8", False):
            raise NotImplementedError("LoRA / fp8 projections with sequence-parallel tensor parallelism")
        if name in ("qkv_proj", "gate_up_proj"):
            return column_parallel_sp(x, getattr(mod, name), sp[0], sp[1])
        y = row_parallel_sp(x if x.stride(-1) == 1 else x.contiguous(), getattr(mod, name), sp[0], sp[1])
        return y + resid if resid is not None else y
    if getattr(mod, "use_fp8", False):
        # block-scaled e4m3 operands in forward and input gradient, fp32 accumulation
        y = OF.fp8_linear(x, getattr(mod, name))
        if resid is not None:
            y = y + resid
    else:
        y = OF.linear(x, getattr(mod, name), resid)
    st = getattr(mod, "lora", None)
    if st is not None and not st.merged and name in getattr(mod, "lora_targets", ()):
        y = y + st.scale * OF.linear(OF.linear(x, getattr(mod, name + "_lora_A")), getattr(mod, name + "_lora_B"))
    return y


class Attention(nn.Module):
    def __init__(self, cfg: ModelConfig, dtype, device):
        super().__init__()
        self.cfg = cfg
        H, D = cfg.hidden_size, cfg.head_dim
        self.nq, self.nkv, self.D = cfg.num_heads, cfg.num_kv_heads, D
        qkv_out = (self.nq + 2 * self.nkv) * D
        self.qkv_proj = nn.Parameter(torch.empty(qkv_out, H, dtype=dtype, device=device))
        self.qkv_bias = nn.Parameter(torch.zeros(qkv_out, dtype=dtype, device=device)) if cfg.attention_bias else None
        self.o_proj = nn.Parameter(torch.empty(H, self.nq * D, dtype=dtype, device=device))
        if cfg.qk_norm:
            self.q_norm = nn.Parameter(torch.ones(D, dtype=dtype, device=device))
            self.k_norm = nn.Parameter(torch.ones(D, dtype=dtype, device=device))
        else:
            self.q_norm = self.k_norm = None

    def project_qkv(self, x: torch.Tensor, pb_positions: torch.Tensor, cos, sin):
        """Returns q [T,nq,D], k [T,nkv,D], v [T,nkv,D] with QK-norm and RoPE applied."""
        D, nq, nkv = self.D, self.nq, self.nkv
        qkv = _lin(self, "qkv_proj", x)
        T = qkv.shape[0]               # all tokens, also when x holds this rank's rows only (sequence-parallel TP)
        if self.qkv_bias is not None:
            qkv = qkv + self.qkv_bias
        if qkv.is_cuda and not torch.is_grad_enabled() and D in (64, 128):
            # inference: one fused kernel for norm + rotation; v stays a strided view
            qk, _ = OF.qknorm_rope_fwd(qkv, self.q_norm, self.k_norm, pb_positions, cos, sin, nq, nkv, D, self.cfg.rms_norm_eps)
            return qk[:, :nq], qk[:, nq:], qkv[:, (nq + nkv) * D:].view(T, nkv, D)   # strided views: no copies
        q = qkv[:, : nq * D].view(T, nq, D)
        k = qkv[:, nq * D: (nq + nkv) * D].view(T, nkv, D)
        v = qkv[:, (nq + nkv) * D:].view(T, nkv, D)
        if self.q_norm is not None:
            q, _ = OF.rmsnorm(q.reshape(T * nq, D), self.q_norm, self.cfg.rms_norm_eps)
            k, _ = OF.rmsnorm(k.reshape(T * nkv, D), self.k_norm, self.cfg.rms_norm_eps)
            q, k = q.view(T, nq, D), k.view(T, nkv, D)
        q = OF.rope(q, pb_positions, cos, sin)
        k = OF.rope(k, pb_positions, cos, sin)
        return q, k, v

    def forward(self, x: torch.Tensor, pb: PackedBatch, cos, sin, attn_fn=None) -> torch.Tensor:
        T = x.shape[0]
        if attn_fn is None and getattr(self, "sp_size", 1) == 1 and x.is_cuda and self.D in (64, 128):
            qkv = _lin(self, "qkv_proj", x)
            if self.qkv_bias is not None:
                qkv = qkv + self.qkv_bias
            o = OF.qknorm_rope_attention(qkv, self.q_norm, self.k_norm, pb.position_ids, cos, sin, pb.cu_seqlens, self.nq,
                                         self.nkv, self.D, self.cfg.rms_norm_eps, 1.0 / math.sqrt(self.D), pb.tile_info)
            return _lin(self, "o_proj", o.reshape(qkv.shape[0], self.nq * self.D))
        if attn_fn is None and getattr(self, "sp_fused", None) is not None and x.is_cuda:
            from ..parallel.ulysses import fused_ulysses_attention_block

            return fused_ulysses_attention_block(self, x, pb, cos, sin, self.sp_fused)
        q, k, v = self.project_qkv(x, pb.position_ids, cos, sin)
        if attn_fn is not None:
            o = attn_fn(q, k, v)
        elif getattr(self, "sp_size", 1) > 1:
            from ..parallel.ulysses import ulysses_attention

            o = ulysses_attention(self, q, k, v, pb.cu_seqlens, True, 1.0 / math.sqrt(self.D), pb.tile_info, OF.attention)
        else:
            o = OF.attention(q, k.contiguous() if not k.is_cuda else k, v.contiguous() if not v.is_cuda else v,
                             pb.cu_seqlens, True, 1.0 / math.sqrt(self.D), pb.tile_info)
        return _lin(self, "o_proj", o.reshape(o.shape[0], self.nq * self.D))


class DenseMLP(nn.Module):
    def __init__(self, hidden: int, inter: int, dtype, device):
        super().__init__()
        self.gate_up_proj = nn.Parameter(torch.empty(2 * inter, hidden, dtype=dtype, device=device))
        self.down_proj = nn.Parameter(torch.empty(hidden, inter, dtype=dtype, device=device))

    def forward(self, x):
        return _lin(self, "down_proj", OF.swiglu(_lin(self, "gate_up_proj", x)))


class MoEMLP(nn.Module):
    """Token-choice top-k routed experts (softmax router in fp32, optional renormalisation of
    the top-k weights). Tokens are sorted by expert and each expert's slice goes through the
    dense GEMM kernel; expert parallelism re-homes the slices (see ``parallel/ep.py``)."""

    def __init__(self, cfg: ModelConfig, dtype, device):
        super().__init__()
        self.cfg = cfg
        E, H, Im = cfg.num_experts, cfg.hidden_size, cfg.moe_intermediate_size
        self.router = nn.Parameter(torch.empty(E, H, dtype=dtype, device=device))
        self.w_gate_up = nn.Parameter(torch.empty(E, 2 * Im, H, dtype=dtype, device=device))
        self.w_down = nn.Parameter(torch.empty(E, H, Im, dtype=dtype, device=device))
        self.ep_dispatcher = None  # set by parallel.ep.ExpertParallel
        if cfg.shared_expert_intermediate_size > 0:
            Is = cfg.shared_expert_intermediate_size
            self.shared_gate_up = nn.Parameter(torch.empty(2 * Is, H, dtype=dtype, device=device))
            self.shared_down = nn.Parameter(torch.empty(H, Is, dtype=dtype, device=device))
            self.shared_expert_gate = nn.Parameter(torch.empty(1, H, dtype=dtype, device=device))
        else:
            self.shared_gate_up = None
        if cfg.router_bias_update_rate > 0:
            self.register_buffer("expert_bias", torch.zeros(E, dtype=torch.float32, device=device), persistent=True)
            self.register_buffer("tokens_per_expert", torch.zeros(E, dtype=torch.float32, device=device), persistent=False)
        else:
            self.expert_bias = None
        self.last_aux_loss: Optional[torch.Tensor] = None
        self.last_routed_experts: Optional[torch.Tensor] = None

    def route(self, x):
        """Gate weights and expert ids per token (fp32). Scores are softmax or sigmoid gates; the
        *choice* of experts may add a balancing bias and be limited to the best expert groups,
        while the returned weights are always the unbiased scores of the chosen experts
        (reference: areal/experimental/models/archon/moe/router.py:234-297)."""
        cfg = self.cfg
        E, k = cfg.num_experts, cfg.num_experts_per_tok
        logits = F.linear(x.float(), self.router.float())
        probs = torch.sigmoid(logits) if cfg.router_score_func == "sigmoid" else torch.softmax(logits, dim=-1)
        choice = probs if self.expert_bias is None else probs + self.expert_bias
        if cfg.num_expert_groups > 0:
            ng, keep = cfg.num_expert_groups, max(1, cfg.num_limited_groups)
            per = E // ng
            grouped = choice.view(-1, ng, per)
            # a group's score: its two best experts when a bias is in play (DeepSeek-V3), else its best expert
            gscore = grouped.topk(min(2, per), dim=-1).values.sum(-1) if self.expert_bias is not None else grouped.max(-1).values
            gidx = gscore.topk(keep, dim=-1).indices
            gmask = torch.zeros_like(gscore, dtype=torch.bool).scatter_(1, gidx, True)
            choice = grouped.masked_fill(~gmask.unsqueeze(-1), float("-inf")).view(-1, E)
        # the choice, its stable sort by expert, the group sizes and the GEMM tile list come from one
        # device-side routing pass (no host read); the weights stay a differentiable gather of ``probs``
        if cfg.num_expert_groups > 0:
            tope = torch.topk(choice, k, dim=-1).indices
            routing = OF.moe_route(logits.detach(), k, tope=tope)
        else:
            routing = OF.moe_route(logits.detach(), k, bias=self.expert_bias, sigmoid=cfg.router_score_func == "sigmoid",
                                   norm=cfg.norm_topk_prob, scale=cfg.router_scale, want_probs=False)
            tope = routing.tope.long()
        topw = probs.gather(1, tope)
        if cfg.norm_topk_prob:
            topw = topw / topw.sum(-1, keepdim=True).clamp(min=1e-20)
        if cfg.router_scale != 1.0:
            topw = topw * cfg.router_scale
        if self.training and (cfg.router_aux_loss_coef > 0 or self.expert_bias is not None):
            load = routing.counts.float()
            if self.expert_bias is not None:
                self.tokens_per_expert.add_(load)
            if cfg.router_aux_loss_coef > 0:
                mean_p = probs.mean(0) if cfg.router_score_func != "sigmoid" else (probs / probs.sum(-1, keepdim=True).clamp(min=1e-20)).mean(0)
                self.last_aux_loss = E * (load / tope.numel() * mean_p).sum() * (cfg.router_aux_loss_coef * getattr(self, "aux_scale", 1.0))
        self.last_routed_experts = tope
        return topw, tope, routing

    @torch.no_grad()
    def update_expert_bias(self, group=None) -> None:
        """Auxiliary-loss-free balancing: after an optimizer step, move each expert's selection bias
        by ``router_bias_update_rate`` against its load since the last call (summed over ``group``)
        (reference: areal/experimental/models/archon/moe/moe.py:119-146, DeepSeek-V3 sec. 2.1.2)."""
        if self.expert_bias is None:
            return
        load = self.tokens_per_expert
        if group is not None and torch.distributed.is_initialized():
            torch.distributed.all_reduce(load, group=group)
        self.expert_bias.add_(self.cfg.router_bias_update_rate * torch.sign(load.mean() - load))
        self.expert_bias.sub_(self.expert_bias.mean())
        load.zero_()

    def experts_forward(self, xs: torch.Tensor, counts, first_expert: int = 0) -> torch.Tensor:
        """xs: tokens sorted by (local) expert; counts[e] tokens for expert first_expert+e, or the
        device-made routing of all experts (then nothing is read back to the host)."""
        if isinstance(counts, OF.Routing):
            if xs.is_cuda and xs.shape[0] > 0 and getattr(self, "use_grouped_gemm", True):
                h = OF.grouped_linear(xs, self.w_gate_up, counts)
                return OF.grouped_linear(OF.swiglu(h), self.w_down, counts)
            counts = counts.host_counts()
        if xs.is_cuda and xs.shape[0] > 0 and getattr(self, "use_grouped_gemm", True):
            # one grouped kernel per projection instead of a launch per expert
            E_local = self.w_gate_up.shape[0]
            cnt = [0] * first_expert + [int(c) for c in counts]
            cnt += [0] * (E_local - len(cnt))
            h = OF.grouped_linear(xs, self.w_gate_up, cnt)
            return OF.grouped_linear(OF.swiglu(h), self.w_down, cnt)
        outs = []
        off = 0
        mg_gu = getattr(self.w_gate_up, "main_grad", None)
        mg_dn = getattr(self.w_down, "main_grad", None)
        direct = xs.is_cuda and mg_gu is not None and mg_dn is not None and torch.is_grad_enabled()
        for e, n in enumerate(counts):
            if n == 0:
                continue
            xe = xs[off:off + n]
            ge = first_expert + e
            if direct:  # weight gradients accumulate straight into the fp32 buffers of expert ge
                h = OF.linear(xe, self.w_gate_up.detach()[ge], None, mg_gu[ge])
                outs.append(OF.linear(OF.swiglu(h), self.w_down.detach()[ge], None, mg_dn[ge]))
            else:
                outs.append(OF.linear(OF.swiglu(OF.linear(xe, self.w_gate_up[ge])), self.w_down[ge]))
            off += n
        if not outs:
            # no token reached this rank's experts: keep the (empty) result attached to ``xs`` so that
            # the backward of the surrounding all-to-alls still runs here. Peers that did send tokens
            # wait for this rank in those collectives; autograd would otherwise prune them.
            return xs[:0] * 0.0
        return torch.cat(outs, dim=0)

    def forward(self, x):
        T, H = x.shape
        k = self.cfg.num_experts_per_tok
        topw, tope, routing = self.route(x)
        out = None
        if self.ep_dispatcher is not None:
            flat_e = tope.reshape(-1)
            order = routing.order.long()
            if x.is_cuda and hasattr(self.ep_dispatcher, "fused_forward"):
                # dispatch and combine as one peer-memory kernel each (parallel/ep_fused.py)
                out = self.ep_dispatcher.fused_forward(self, x, order, flat_e, topw)
            if out is None:
                token_of = routing.token_of.long()
                ys = self.ep_dispatcher(self, x[token_of], flat_e[order])
                w = topw.reshape(-1)[order].to(ys.dtype).unsqueeze(-1)
                out = torch.zeros(T, H, dtype=ys.dtype, device=x.device)
                out.index_add_(0, token_of, ys * w)
        else:
            ys = self.experts_forward(x.index_select(0, routing.token_of), routing)
            # every (token, slot) entry reads its row back: a gather and one sum over the k slots, the same
            # bits run after run (no atomics)
            out = (ys.index_select(0, routing.inv).view(T, k, H) * topw.to(ys.dtype).unsqueeze(-1)).sum(1)
        if self.shared_gate_up is not None:
            # the shared expert sees every token; its output is scaled by a per-token sigmoid gate
            sh = OF.linear(OF.swiglu(OF.linear(x, self.shared_gate_up)), self.shared_down)
            gate = torch.sigmoid(F.linear(x.float(), self.shared_expert_gate.float())).to(sh.dtype)
            out = out + gate * sh
        return out


def norm_or_reduce(h, w, eps, resid):
    """``OF.rmsnorm`` for a tensor; for the handle of a tensor-parallel partial sum the fused
    sum-over-ranks + residual + RMSNorm kernel."""
    if hasattr(h, "set_idx"):
        return h.ex.reduce_rmsnorm(h, w, eps, resid)
    return OF.rmsnorm(h, w, eps, resid)


class DecoderLayer(nn.Module):
    def __init__(self, cfg: ModelConfig, idx: int, dtype, device):
        super().__init__()
        self.cfg = cfg
        H = cfg.hidden_size
        self.input_layernorm = nn.Parameter(torch.ones(H, dtype=dtype, device=device))
        self.post_attention_layernorm = nn.Parameter(torch.ones(H, dtype=dtype, device=device))
        self.self_attn = Attention(cfg, dtype, device)
        self.mlp = MoEMLP(cfg, dtype, device) if cfg.layer_is_moe(idx) else DenseMLP(H, cfg.intermediate_size, dtype, device)

    tp_group = None  # set by parallel.tp.install_tp
    moe_row_share = None  # (group, tp, rank): whole experts under tensor-parallel attention (parallel.tp.moe_on_row_share)
    tp_exchange = None  # set by parallel.tp_decode.install_tp_decode (inference: fused partial-sum exchange)

    def forward(self, h, resid, pb: PackedBatch, cos, sin, attn_fn=None):
        if self.tp_exchange is not None and not torch.is_grad_enabled():
            # the attention and MLP blocks return handles of partial sums; each norm kernel below
            # waits for the peers' parts, sums them, adds the residual stream and normalises
            x, resid = norm_or_reduce(h, self.input_layernorm, self.cfg.rms_norm_eps, resid)
            h = self.self_attn(x, pb, cos, sin, attn_fn)
            x, resid = norm_or_reduce(h, self.post_attention_layernorm, self.cfg.rms_norm_eps, resid)
            return self.mlp(x), resid
        x, resid = OF.rmsnorm(h, self.input_layernorm, self.cfg.rms_norm_eps, resid)
        g = self.tp_group
        if g is None:
            h = self.self_attn(x, pb, cos, sin, attn_fn)
            x, resid = OF.rmsnorm(h, self.post_attention_layernorm, self.cfg.rms_norm_eps, resid)
            h = self.mlp(x)
            return h, resid
        # tensor parallel: this rank holds a slice of the heads / MLP columns; partial block
        # outputs are summed over the group
        from ..parallel.tp import copy_to_tp, reduce_from_tp

        h = reduce_from_tp(self.self_attn(copy_to_tp(x, g), pb, cos, sin, attn_fn), g)
        x, resid = OF.rmsnorm(h, self.post_attention_layernorm, self.cfg.rms_norm_eps, resid)
        if self.moe_row_share is not None:
            from ..parallel.tp import moe_on_row_share

            return moe_on_row_share(self.mlp, x, *self.moe_row_share), resid
        h = reduce_from_tp(self.mlp(copy_to_tp(x, g)), g)
        return h, resid


class CausalLM(nn.Module):
    """Embedding -> N decoder layers -> final norm -> (LM head | value head)."""

    def __init__(self, cfg: ModelConfig, dtype=torch.bfloat16, device="cpu", init_std: float = 0.02, seed: Optional[int] = None):
        super().__init__()
        self.cfg = cfg
        self.dtype = dtype
        H = cfg.hidden_size
        self.embed_tokens = nn.Parameter(torch.empty(cfg.vocab_size, H, dtype=dtype, device=device))
        if cfg.layer_types:
            from .hybrid import HybridDecoderLayer as layer_cls   # linear / gated full attention per layer (Qwen3.5)
        else:
            layer_cls = DecoderLayer
        self.layers = nn.ModuleList([layer_cls(cfg, i, dtype, device) for i in range(cfg.num_layers)])
        self.norm = nn.Parameter(torch.ones(H, dtype=dtype, device=device))
        if cfg.is_critic:
            self.value_head = nn.Parameter(torch.zeros(1, H, dtype=dtype, device=device))
            self.lm_head = None
        else:
            self.value_head = None
            self.lm_head = None if cfg.tie_word_embeddings else nn.Parameter(torch.empty(cfg.vocab_size, H, dtype=dtype, device=device))
        self.gradient_checkpointing = False
        self._rope_cache: dict = {}
        self.reset_parameters(init_std, seed)

    @torch.no_grad()
    def reset_parameters(self, std: float = 0.02, seed: Optional[int] = None):
        if self.embed_tokens.device.type == "meta":
            return          # shapes only (layout planning): nothing to draw
        gen = None
        if seed is not None:
            gen = torch.Generator(device=self.embed_tokens.device)
            gen.manual_seed(seed)
        for name, p in self.named_parameters():
            if name.endswith("layernorm") or name.endswith("norm") or name.endswith("q_norm") or name.endswith("k_norm"):
                p.fill_(1.0)
            elif name.endswith("bias") or name.endswith("value_head"):
                p.zero_()
            else:
                # draw in fp32 chunks to keep peak memory small for multi-GB tensors
                flat = p.view(-1)
                step = 1 << 26
                for a in range(0, flat.numel(), step):
                    b = min(flat.numel(), a + step)
                    flat[a:b] = (torch.randn(b - a, device=p.device, dtype=torch.float32, generator=gen) * std).to(p.dtype)
        if self.cfg.layer_types:
            from .hybrid import init_hybrid_parameters

            init_hybrid_parameters(self, gen)

    @property
    def output_weight(self) -> torch.Tensor:
        return self.embed_tokens if self.lm_head is None else self.lm_head

    def rope(self, device, max_pos: Optional[int] = None):
        max_pos = max_pos or self.cfg.max_position_embeddings
        key = (str(device), max_pos)
        if key not in self._rope_cache:
            self._rope_cache = {key: OF.rope_tables(max_pos, self.cfg.rotary_dim, self.cfg.rope_theta, device)}
        return self._rope_cache[key]

    def forward_hidden(self, input_ids: torch.Tensor, pb: PackedBatch, attn_fns=None, inputs_embeds: Optional[torch.Tensor] = None,
                       rope: Optional[tuple] = None, deepstack: Optional[tuple] = None) -> torch.Tensor:
        """input_ids: [T] -> final normed hidden states [T, H]. ``inputs_embeds`` replaces the
        embedding lookup; ``rope = (cos, sin)`` replaces the position tables (rows are then
        selected by ``pb.position_ids`` exactly like the default tables)."""
        cos, sin = rope if rope is not None else self.rope(input_ids.device, max(self.cfg.max_position_embeddings, pb.max_seqlen + 1))
        h = inputs_embeds if inputs_embeds is not None else OF.embedding(input_ids, self.embed_tokens)
        resid = None
        units = getattr(self, "param_units", None)      # sharded parameters: a layer's weights exist only between enter and leave
        for i, layer in enumerate(self.layers):
            fn = attn_fns[i] if attn_fns is not None else None
            if units is not None:
                h, resid = units.enter(i, h, resid)
            if self.training and torch.is_grad_enabled() and self._recompute_layer(i):
                h, resid = checkpoint(layer, h, resid, pb, cos, sin, fn, use_reentrant=False)
            else:
                h, resid = layer(h, resid, pb, cos, sin, fn)
            if units is not None:
                h, resid = units.leave(i, h, resid)
            if deepstack is not None and i < len(deepstack[1]):
                # deep-stack features of the image tower join the hidden state (= resid + h) after the first layers
                h = h.index_add(0, deepstack[0], deepstack[1][i].to(h.dtype))
        if self.cfg.rms_norm_offset:
            from .hybrid import rmsnorm_offset

            x, _ = rmsnorm_offset(h, self.norm, self.cfg.rms_norm_eps, resid)
        else:
            x, _ = norm_or_reduce(h, self.norm, self.cfg.rms_norm_eps, resid)
        return x

    def set_fp8(self, dense: bool = True) -> int:
        """Routes the dense projections (attention QKV / output, dense MLP) through the
        block-scaled fp8 GEMM. Returns the number of modules switched."""
        n = 0
        for layer in self.layers:
            mods = [layer.self_attn] + ([layer.mlp] if isinstance(layer.mlp, DenseMLP) else [])
            for m in mods:
                m.use_fp8 = bool(dense)
                n += 1
        return n

    def set_activation_checkpointing(self, mode: str = "none", fraction: float = 0.5) -> None:
        """``none`` keeps every activation; ``full`` recomputes every layer in the backward;
        ``selective`` recomputes every second layer; ``memory_budget`` recomputes the first
        ``round(fraction * num_layers)`` layers (their activations live longest), keeping the
        rest: pick the fraction from the memory that is left after parameters and optimizer
        state. Reference: ``areal/experimental/models/archon/activation_checkpoint.py``."""
        n = len(self.layers)
        if mode in ("none", None, False):
            self.gradient_checkpointing, self._ckpt_layers = False, frozenset()
        elif mode in ("full", True):
            self.gradient_checkpointing, self._ckpt_layers = True, frozenset(range(n))
        elif mode == "selective":
            self.gradient_checkpointing, self._ckpt_layers = False, frozenset(range(0, n, 2))
        elif mode == "memory_budget":
            if not 0.0 <= fraction <= 1.0:
                raise ValueError("memory_budget fraction must be in [0, 1]")
            self.gradient_checkpointing, self._ckpt_layers = False, frozenset(range(int(round(fraction * n))))
        else:
            raise ValueError(f"unknown activation checkpointing mode '{mode}'")

    def _recompute_layer(self, i: int) -> bool:
        return self.gradient_checkpointing or i in getattr(self, "_ckpt_layers", ())

    def logits(self, hidden: torch.Tensor) -> torch.Tensor:
        """Full fp32 logits (small batches / sampling only)."""
        if hidden.is_cuda:
            return OF.gemm(hidden.contiguous(), self.output_weight, epi=OF.EPI_F32)
        return F.linear(hidden, self.output_weight).float()

    def logprobs_entropy(self, hidden: torch.Tensor, labels: torch.Tensor, temperature: float = 1.0, chunk: int = 2048):
        return OF.lm_head_logprob(hidden, self.output_weight, labels, temperature, chunk)

    def values(self, hidden: torch.Tensor) -> torch.Tensor:
        return F.linear(hidden.float(), self.value_head.float()).squeeze(-1)

    def aux_loss(self) -> Optional[torch.Tensor]:
        tot = None
        for layer in self.layers:
            al = getattr(layer.mlp, "last_aux_loss", None)
            if al is not None:
                tot = al if tot is None else tot + al
                layer.mlp.last_aux_loss = None
        return tot

    def forward(self, input_ids, cu_seqlens, position_ids=None, max_seqlen: int = 0, **kw):
        from ..utils.data import positions_from_cu_seqlens

        T = input_ids.shape[0]
        if position_ids is None:
            position_ids = positions_from_cu_seqlens(cu_seqlens, T)
        pb = PackedBatch(cu_seqlens, position_ids, T, max_seqlen)
        return self.forward_hidden(input_ids, pb, **kw)


def build_model(cfg: ModelConfig, dtype=torch.bfloat16, device="cpu", seed: Optional[int] = None) -> CausalLM:
    if cfg.is_vlm:
        from .vlm import VisionLanguageModel

        return VisionLanguageModel(cfg, dtype=dtype, device=device, seed=seed)
    return CausalLM(cfg, dtype=dtype, device=device, seed=seed)
