"""Low-rank adapters for the decoder's linear layers.

``apply_lora`` attaches, to every targeted weight ``W [out, in]`` of every layer, a pair
``A [r, in]`` (Kaiming-uniform) and ``B [out, r]`` (zeros) and freezes the base parameters; the
layers then compute ``x W^T + (alpha / r) (x A^T) B^T`` (two extra skinny GEMMs on the same
tcgen05 kernel). ``merge_lora_`` folds the adapters into the base weights for serving / weight
updates, ``unmerge_lora_`` undoes it. Adapter checkpoints use the PEFT tensor naming
(``...lora_A.weight`` / ``...lora_B.weight``) under the Hugging Face module path so they load
into PEFT. Reference: ``TrainEngineConfig.use_lora / lora_rank / lora_alpha / target_modules``
(``areal/api/cli_args.py``) and the PEFT wrapping in ``areal/engine/fsdp_engine.py``.
"""
from __future__ import annotations

import json
import math
import os
from typing import Iterable, Optional

import torch
import torch.nn as nn

# user-facing (HF) module names -> fused native parameters that carry them
_TARGET_ALIASES = {
    "q_proj": "qkv_proj", "k_proj": "qkv_proj", "v_proj": "qkv_proj", "qkv_proj": "qkv_proj", "o_proj": "o_proj",
    "gate_proj": "gate_up_proj", "up_proj": "gate_up_proj", "gate_up_proj": "gate_up_proj", "down_proj": "down_proj",
    "all-linear": "*",
}
_ALL = ("qkv_proj", "o_proj", "gate_up_proj", "down_proj")


class LoRAState:
    def __init__(self, rank: int, alpha: float):
        self.rank, self.alpha = rank, alpha
        self.scale = alpha / rank
        self.merged = False


def resolve_targets(target_modules: Iterable[str]) -> set[str]:
    out: set[str] = set()
    for t in target_modules or ["all-linear"]:
        n = _TARGET_ALIASES.get(t)
        if n is None:
            raise ValueError(f"unknown LoRA target module '{t}'")
        out |= set(_ALL) if n == "*" else {n}
    return out


def _modules_with(model, name: str):
    for lname, layer in model.layers.named_children():
        for sub_name in ("self_attn", "mlp"):
            sub = getattr(layer, sub_name)
            if isinstance(getattr(sub, name, None), nn.Parameter):
                yield f"layers.{lname}.{sub_name}", sub


def apply_lora(model, rank: int = 32, alpha: float = 16.0, target_modules: Optional[Iterable[str]] = None, seed: int = 0):
    targets = resolve_targets(target_modules)
    gen = torch.Generator(device="cpu").manual_seed(seed)
    for p in model.parameters():
        p.requires_grad_(False)
    n = 0
    for t in sorted(targets):
        for path, mod in _modules_with(model, t):
            w = getattr(mod, t)
            out_f, in_f = w.shape
            bound = 1.0 / math.sqrt(in_f)
            a = (torch.rand(rank, in_f, generator=gen) * 2 - 1) * bound * math.sqrt(3.0)
            setattr(mod, f"{t}_lora_A", nn.Parameter(a.to(w.device, w.dtype)))
            setattr(mod, f"{t}_lora_B", nn.Parameter(torch.zeros(out_f, rank, device=w.device, dtype=w.dtype)))
            if not hasattr(mod, "lora_targets"):
                mod.lora_targets = set()
            mod.lora_targets.add(t)
            n += 1
    model.lora = LoRAState(rank, alpha)
    for layer in model.layers:
        layer.self_attn.lora = model.lora
        layer.mlp.lora = model.lora
    if n == 0:
        raise ValueError("no LoRA target matched the model")
    return model


def lora_named_parameters(model):
    return [(n, p) for n, p in model.named_parameters() if "_lora_" in n]


@torch.no_grad()
def merge_lora_(model, sign: float = 1.0):
    st = getattr(model, "lora", None)
    if st is None or st.merged == (sign > 0):
        return model
    for t in _ALL:
        for _, mod in _modules_with(model, t):
            if t in getattr(mod, "lora_targets", ()):
                A, B = getattr(mod, f"{t}_lora_A"), getattr(mod, f"{t}_lora_B")
                getattr(mod, t).add_((B.float() @ A.float()).to(A.dtype), alpha=sign * st.scale)
    st.merged = sign > 0
    return model


def unmerge_lora_(model):
    return merge_lora_(model, -1.0)


def _hf_names(cfg, native_path: str, target: str) -> list[tuple[str, Optional[tuple[int, int]]]]:
    """HF module(s) behind a fused native weight with the row range each one covers."""
    base = "model." + native_path
    D, nq, nkv = cfg.head_dim, cfg.num_heads, cfg.num_kv_heads
    if target == "qkv_proj":
        return [(f"{base}.q_proj", (0, nq * D)), (f"{base}.k_proj", (nq * D, (nq + nkv) * D)), (f"{base}.v_proj", ((nq + nkv) * D, (nq + 2 * nkv) * D))]
    if target == "gate_up_proj":
        I = cfg.intermediate_size
        return [(f"{base}.gate_proj", (0, I)), (f"{base}.up_proj", (I, 2 * I))]
    return [(f"{base}.{target}", None)]


def save_adapter(model, path: str, base_model_name_or_path: str = "") -> None:
    """PEFT layout: ``adapter_model.safetensors`` + ``adapter_config.json``. A fused weight's
    ``B`` is split by rows over its HF modules, ``A`` is shared (copied)."""
    from safetensors.torch import save_file

    os.makedirs(path, exist_ok=True)
    st = model.lora
    tensors, targets = {}, set()
    for t in _ALL:
        for native_path, mod in _modules_with(model, t):
            if t not in getattr(mod, "lora_targets", ()):
                continue
            A, B = getattr(mod, f"{t}_lora_A").detach().cpu(), getattr(mod, f"{t}_lora_B").detach().cpu()
            for hf, rows in _hf_names(model.cfg, native_path, t):
                tensors[f"base_model.model.{hf}.lora_A.weight"] = A.clone().contiguous()
                tensors[f"base_model.model.{hf}.lora_B.weight"] = (B if rows is None else B[rows[0]:rows[1]]).clone().contiguous()
                targets.add(hf.rsplit(".", 1)[-1])
    save_file(tensors, os.path.join(path, "adapter_model.safetensors"), metadata={"format": "pt"})
    with open(os.path.join(path, "adapter_config.json"), "w") as f:
        json.dump({"peft_type": "LORA", "r": st.rank, "lora_alpha": st.alpha, "target_modules": sorted(targets), "bias": "none",
                   "task_type": "CAUSAL_LM", "base_model_name_or_path": base_model_name_or_path, "lora_dropout": 0.0}, f, indent=1)


def load_adapter(model, path: str) -> None:
    """Inverse of :func:`save_adapter` for adapters written by it (shared ``A`` per fused weight)."""
    from safetensors.torch import load_file

    tensors = load_file(os.path.join(path, "adapter_model.safetensors"))
    with torch.no_grad():
        for t in _ALL:
            for native_path, mod in _modules_with(model, t):
                if t not in getattr(mod, "lora_targets", ()):
                    continue
                A, B = getattr(mod, f"{t}_lora_A"), getattr(mod, f"{t}_lora_B")
                parts = _hf_names(model.cfg, native_path, t)
                A.copy_(tensors[f"base_model.model.{parts[0][0]}.lora_A.weight"].to(A.dtype))
                for hf, rows in parts:
                    b = tensors[f"base_model.model.{hf}.lora_B.weight"].to(B.dtype)
                    if rows is None:
                        B.copy_(b)
                    else:
                        B[rows[0]:rows[1]].copy_(b)
