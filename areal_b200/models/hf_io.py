"""Hugging Face checkpoint interop: name mapping between this framework's fused parameter
layout and HF's per-projection names, sharded safetensors reading and writing
(``model-0000i-of-0000N.safetensors`` + ``model.safetensors.index.json``).

Reference behaviour: HF save/load in ``areal/engine/fsdp_engine.py:1787-1818`` and the
state-dict adapters ``areal/experimental/models/archon/qwen*/model/state_dict_adapter.py``,
``archon/moe_weight_converter.py`` (per-expert <-> grouped expert tensors).
"""
from __future__ import annotations

import json
import os
import re
from typing import Iterable, Iterator, Optional

import torch

from .config import ModelConfig


# --------------------------------------------------------------------------- name mapping
def hf_to_native_plan(cfg: ModelConfig) -> dict[str, list[tuple[str, Optional[tuple[int, int]], Optional[int]]]]:
    """native name -> list of (hf name, row range in the native tensor or None, expert idx or None)."""
    D, nq, nkv = cfg.head_dim, cfg.num_heads, cfg.num_kv_heads
    plan: dict = {"embed_tokens": [("model.embed_tokens.weight", None, None)], "norm": [("model.norm.weight", None, None)]}
    if cfg.is_critic:
        plan["value_head"] = [("score.weight", None, None)]
    elif not cfg.tie_word_embeddings:
        plan["lm_head"] = [("lm_head.weight", None, None)]
    if cfg.is_vlm:
        from .vision import vision_param_names

        for n in vision_param_names(cfg.vision_config()):
            plan["visual." + n] = [("visual." + n, None, None)]
    for i in range(cfg.num_layers):
        p, h = f"layers.{i}.", f"model.layers.{i}."
        plan[p + "input_layernorm"] = [(h + "input_layernorm.weight", None, None)]
        plan[p + "post_attention_layernorm"] = [(h + "post_attention_layernorm.weight", None, None)]
        q_rows, k_rows = nq * D, nkv * D
        if cfg.layer_types:
            # hybrid stack: gated-delta-rule layers and gated full attention keep their own projections
            if cfg.layer_is_moe(i):
                Is, Im = cfg.shared_expert_intermediate_size, cfg.moe_intermediate_size
                plan[p + "mlp.router"] = [(h + "mlp.gate.weight", None, None)]
                gu, dn = [], []
                for e in range(cfg.num_experts):
                    gu.append((h + f"mlp.experts.{e}.gate_proj.weight", (0, Im), e))
                    gu.append((h + f"mlp.experts.{e}.up_proj.weight", (Im, 2 * Im), e))
                    dn.append((h + f"mlp.experts.{e}.down_proj.weight", None, e))
                plan[p + "mlp.w_gate_up"], plan[p + "mlp.w_down"] = gu, dn
                plan[p + "mlp.shared_gate_up"] = [(h + "mlp.shared_expert.gate_proj.weight", (0, Is), None),
                                                  (h + "mlp.shared_expert.up_proj.weight", (Is, 2 * Is), None)]
                plan[p + "mlp.shared_down"] = [(h + "mlp.shared_expert.down_proj.weight", None, None)]
                plan[p + "mlp.shared_expert_gate"] = [(h + "mlp.shared_expert_gate.weight", None, None)]
            else:
                I = cfg.intermediate_size
                plan[p + "mlp.gate_up_proj"] = [(h + "mlp.gate_proj.weight", (0, I), None), (h + "mlp.up_proj.weight", (I, 2 * I), None)]
                plan[p + "mlp.down_proj"] = [(h + "mlp.down_proj.weight", None, None)]
            if cfg.layer_is_linear(i):
                la, nv = h + "linear_attn.", cfg.linear_num_value_heads
                plan[p + "linear_attn.in_proj_qkv"] = [(la + "in_proj_qkv.weight", None, None)]
                plan[p + "linear_attn.in_proj_z"] = [(la + "in_proj_z.weight", None, None)]
                plan[p + "linear_attn.in_proj_ba"] = [(la + "in_proj_b.weight", (0, nv), None), (la + "in_proj_a.weight", (nv, 2 * nv), None)]
                plan[p + "linear_attn.conv1d"] = [(la + "conv1d.weight", None, None)]        # checkpoint shape [C, 1, K]
                plan[p + "linear_attn.dt_bias"] = [(la + "dt_bias", None, None)]
                plan[p + "linear_attn.A_log"] = [(la + "A_log", None, None)]
                plan[p + "linear_attn.norm"] = [(la + "norm.weight", None, None)]
                plan[p + "linear_attn.out_proj"] = [(la + "out_proj.weight", None, None)]
            else:
                plan[p + "self_attn.q_proj"] = [(h + "self_attn.q_proj.weight", None, None)]
                plan[p + "self_attn.kv_proj"] = [(h + "self_attn.k_proj.weight", (0, k_rows), None),
                                                 (h + "self_attn.v_proj.weight", (k_rows, 2 * k_rows), None)]
                plan[p + "self_attn.o_proj"] = [(h + "self_attn.o_proj.weight", None, None)]
                plan[p + "self_attn.q_norm"] = [(h + "self_attn.q_norm.weight", None, None)]
                plan[p + "self_attn.k_norm"] = [(h + "self_attn.k_norm.weight", None, None)]
            continue
        plan[p + "self_attn.qkv_proj"] = [
            (h + "self_attn.q_proj.weight", (0, q_rows), None),
            (h + "self_attn.k_proj.weight", (q_rows, q_rows + k_rows), None),
            (h + "self_attn.v_proj.weight", (q_rows + k_rows, q_rows + 2 * k_rows), None),
        ]
        if cfg.attention_bias:
            plan[p + "self_attn.qkv_bias"] = [
                (h + "self_attn.q_proj.bias", (0, q_rows), None),
                (h + "self_attn.k_proj.bias", (q_rows, q_rows + k_rows), None),
                (h + "self_attn.v_proj.bias", (q_rows + k_rows, q_rows + 2 * k_rows), None),
            ]
        plan[p + "self_attn.o_proj"] = [(h + "self_attn.o_proj.weight", None, None)]
        if cfg.qk_norm:
            plan[p + "self_attn.q_norm"] = [(h + "self_attn.q_norm.weight", None, None)]
            plan[p + "self_attn.k_norm"] = [(h + "self_attn.k_norm.weight", None, None)]
        if cfg.layer_is_moe(i):
            Im = cfg.moe_intermediate_size
            plan[p + "mlp.router"] = [(h + "mlp.gate.weight", None, None)]
            gu, dn = [], []
            for e in range(cfg.num_experts):
                gu.append((h + f"mlp.experts.{e}.gate_proj.weight", (0, Im), e))
                gu.append((h + f"mlp.experts.{e}.up_proj.weight", (Im, 2 * Im), e))
                dn.append((h + f"mlp.experts.{e}.down_proj.weight", None, e))
            plan[p + "mlp.w_gate_up"] = gu
            plan[p + "mlp.w_down"] = dn
            if cfg.shared_expert_intermediate_size:
                Is = cfg.shared_expert_intermediate_size
                plan[p + "mlp.shared_gate_up"] = [(h + "mlp.shared_expert.gate_proj.weight", (0, Is), None),
                                                  (h + "mlp.shared_expert.up_proj.weight", (Is, 2 * Is), None)]
                plan[p + "mlp.shared_down"] = [(h + "mlp.shared_expert.down_proj.weight", None, None)]
                plan[p + "mlp.shared_expert_gate"] = [(h + "mlp.shared_expert_gate.weight", None, None)]
        else:
            I = cfg.intermediate_size
            plan[p + "mlp.gate_up_proj"] = [(h + "mlp.gate_proj.weight", (0, I), None),
                                            (h + "mlp.up_proj.weight", (I, 2 * I), None)]
            plan[p + "mlp.down_proj"] = [(h + "mlp.down_proj.weight", None, None)]
    return plan


def native_to_hf_tensors(cfg: ModelConfig, named: Iterable[tuple[str, torch.Tensor]]) -> Iterator[tuple[str, torch.Tensor]]:
    """Splits native (fused) tensors into HF-named tensors (views; no copies)."""
    plan = hf_to_native_plan(cfg)
    # checkpoints of the newer vision-language families nest the decoder and the tower under ``model.``
    nested = cfg.is_vlm and cfg.vision.get("model_type") == "qwen3_vl"
    for name, t in named:
        if name not in plan:
            raise KeyError(f"no HF mapping for parameter '{name}'")
        for hf_name, rows, expert in plan[name]:
            if nested:
                hf_name = ("model." + hf_name if hf_name.startswith("visual.") else
                           "model.language_model." + hf_name[len("model."):] if hf_name.startswith("model.") else hf_name)
            src = t if expert is None else t[expert]
            src = src if rows is None else src[rows[0]:rows[1]]
            yield hf_name, (src.unsqueeze(1) if hf_name.endswith("linear_attn.conv1d.weight") else src)


@torch.no_grad()
def load_hf_tensors_into(cfg: ModelConfig, params: Optional[dict[str, torch.Tensor]], hf_tensors: Iterable[tuple[str, torch.Tensor]],
                         strict: bool = True, writer=None) -> set[str]:
    """Copies HF-named tensors into native parameters. Returns the set of HF names consumed. ``writer(native name,
    expert index or None, row range or None, tensor)`` takes the pieces instead when the native tensors do not exist
    as a whole (sharded parameters)."""
    plan = hf_to_native_plan(cfg)
    inverse: dict[str, tuple[str, Optional[tuple[int, int]], Optional[int]]] = {}
    for native, parts in plan.items():
        for hf_name, rows, expert in parts:
            inverse[hf_name] = (native, rows, expert)
    seen = set()
    for hf_name, t in hf_tensors:
        # newer VLM checkpoints nest the decoder and the tower under ``model.``
        if hf_name.startswith("model.language_model."):
            hf_name = "model." + hf_name[len("model.language_model."):]
        elif hf_name.startswith("model.visual."):
            hf_name = hf_name[len("model."):]
        if hf_name not in inverse:
            if hf_name == "lm_head.weight" and cfg.tie_word_embeddings:
                continue
            if strict:
                raise KeyError(f"unexpected tensor '{hf_name}' in checkpoint")
            continue
        native, rows, expert = inverse[hf_name]
        if hf_name.endswith("linear_attn.conv1d.weight") and t.dim() == 3:
            t = t.squeeze(1)
        if writer is not None:
            writer(native, expert, rows, t)
            seen.add(hf_name)
            continue
        dst = params[native]
        dst = dst if expert is None else dst[expert]
        dst = dst if rows is None else dst[rows[0]:rows[1]]
        if dst.shape != t.shape:
            raise ValueError(f"shape mismatch for {hf_name}: checkpoint {tuple(t.shape)} vs model {tuple(dst.shape)}")
        dst.copy_(t.to(dst.dtype))
        seen.add(hf_name)
    if strict:
        missing = set(inverse) - seen
        if missing:
            raise KeyError(f"{len(missing)} tensors missing from checkpoint, e.g. {sorted(missing)[:3]}")
    return seen


# --------------------------------------------------------------------------- safetensors IO
def dequant_block_fp8(w8: torch.Tensor, scale_inv: torch.Tensor, block: tuple[int, int] = (128, 128), dtype=torch.bfloat16) -> torch.Tensor:
    """``w[i, j] = fp8[i, j] * scale_inv[i // bm, j // bn]`` (block-quantised checkpoints keep one fp32 multiplier per
    ``bm x bn`` block under ``<name>_scale_inv``). Stacked tensors ``[E, R, C]`` carry scales ``[E, R / bm, C / bn]``."""
    bm, bn = block
    R, C = w8.shape[-2:]
    if tuple(scale_inv.shape[-2:]) != (-(-R // bm), -(-C // bn)):
        raise ValueError(f"scale grid {tuple(scale_inv.shape)} does not fit a {R} x {C} tensor in {bm} x {bn} blocks")
    s = scale_inv.float().repeat_interleave(bm, dim=-2)[..., :R, :].repeat_interleave(bn, dim=-1)[..., :C]
    return (w8.float() * s).to(dtype)


def _fp8_block_of(path: str) -> Optional[tuple[int, int]]:
    """Block shape from ``config.json`` (``quantization_config.weight_block_size``) when the checkpoint is fp8."""
    cj = os.path.join(path, "config.json")
    if not os.path.exists(cj):
        return None
    with open(cj) as f:
        q = (json.load(f).get("quantization_config") or {})
    if str(q.get("quant_method", "")).lower() != "fp8" and "weight_block_size" not in q:
        return None
    b = q.get("weight_block_size") or [128, 128]
    return int(b[0]), int(b[1])


def iter_safetensors(path: str, device: str = "cpu", dequant_fp8: bool = True) -> Iterator[tuple[str, torch.Tensor]]:
    """(name, tensor) of every tensor under ``path``. Block-quantised fp8 weights (a ``float8_e4m3fn`` tensor with a
    ``<name>_scale_inv`` companion, as written for DeepSeek-V3 / Qwen3-FP8 style checkpoints) come out dequantised to
    bf16 and their scale tensors are not listed: the loaders above see an ordinary checkpoint. Reference:
    ``areal/experimental/models/archon/fp8_checkpoint.py:36-330`` (dequantise on load)."""
    from safetensors import safe_open

    files = sorted(f for f in os.listdir(path) if f.endswith(".safetensors"))
    if not files:
        raise FileNotFoundError(f"no .safetensors files under {path}")
    block = _fp8_block_of(path) if dequant_fp8 else None
    where: dict[str, str] = {}
    ij = os.path.join(path, "model.safetensors.index.json")
    if dequant_fp8 and os.path.exists(ij):
        with open(ij) as f:
            where = json.load(f).get("weight_map", {})
    fp8 = getattr(torch, "float8_e4m3fn", None)
    for fn in files:
        with safe_open(os.path.join(path, fn), framework="pt", device=device) as f:
            keys = list(f.keys())
            for k in keys:
                if dequant_fp8 and k.endswith("_scale_inv"):
                    continue
                t = f.get_tensor(k)
                if dequant_fp8 and fp8 is not None and t.dtype == fp8:
                    sk = k + "_scale_inv"
                    if sk in keys:
                        sc = f.get_tensor(sk)
                    elif sk in where:                  # the scale lives in another shard
                        with safe_open(os.path.join(path, where[sk]), framework="pt", device=device) as g:
                            sc = g.get_tensor(sk)
                    else:
                        raise KeyError(f"fp8 tensor '{k}' has no '{sk}' in the checkpoint")
                    t = dequant_block_fp8(t, sc, block or (128, 128))
                yield k, t


def save_hf_sharded(path: str, cfg: ModelConfig, hf_named: Iterable[tuple[str, torch.Tensor]],
                    max_shard_bytes: int = 5 * 1024 ** 3, shard_prefix: str = "model", rank_tag: Optional[str] = None,
                    write_index: bool = True) -> dict[str, str]:
    """Writes HF-layout safetensors shards; returns the tensor -> file map. ``rank_tag``
    lets several ranks write disjoint tensors into the same directory (the caller merges the
    maps and writes the index once)."""
    from safetensors.torch import save_file

    os.makedirs(path, exist_ok=True)
    shards: list[dict[str, torch.Tensor]] = [{}]
    size = 0
    for name, t in hf_named:
        nbytes = t.numel() * t.element_size()
        if size + nbytes > max_shard_bytes and shards[-1]:
            shards.append({})
            size = 0
        shards[-1][name] = t.detach().to("cpu").contiguous()
        size += nbytes
    n = len(shards)
    weight_map = {}
    total = 0
    for i, sh in enumerate(shards):
        tag = f"{shard_prefix}-{rank_tag}-" if rank_tag else f"{shard_prefix}-"
        fn = f"{tag}{i + 1:05d}-of-{n:05d}.safetensors" if (n > 1 or rank_tag) else f"{shard_prefix}.safetensors"
        save_file(sh, os.path.join(path, fn), metadata={"format": "pt"})
        for k, t in sh.items():
            weight_map[k] = fn
            total += t.numel() * t.element_size()
    if write_index:
        write_hf_index(path, weight_map, total)
        cfg.save_pretrained(path)
    return weight_map


def write_hf_index(path: str, weight_map: dict[str, str], total_size: int) -> None:
    if len(set(weight_map.values())) > 1:
        with open(os.path.join(path, "model.safetensors.index.json"), "w") as f:
            json.dump({"metadata": {"total_size": total_size}, "weight_map": dict(sorted(weight_map.items()))}, f, indent=2)


def save_model_hf(model, path: str, max_shard_bytes: int = 5 * 1024 ** 3, skip=None) -> None:
    named = [(n, p.detach()) for n, p in model.named_parameters() if skip is None or not skip(n)]
    save_hf_sharded(path, model.cfg, native_to_hf_tensors(model.cfg, named), max_shard_bytes)


def load_model_hf(model, path: str, strict: bool = True) -> None:
    params = {n: p.data for n, p in model.named_parameters()}
    load_hf_tensors_into(model.cfg, params, iter_safetensors(path), strict=strict)
