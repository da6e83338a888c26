"""Architecture description of the supported decoder families (Qwen2 / Qwen2.5, Qwen3,
Qwen3-MoE) and conversion from / to Hugging Face ``config.json``.

Reference model zoo: ``areal/experimental/models/archon/{qwen2,qwen3}/model/args.py`` and
the HF path of ``areal/engine/fsdp_engine.py:375-560``.
"""
from __future__ import annotations

import json
import os
from dataclasses import asdict, dataclass, field
from typing import Optional


@dataclass
class ModelConfig:
    arch: str = "qwen2"                 # qwen2 | qwen3 | qwen3_moe | qwen2_moe
    vocab_size: int = 151936
    hidden_size: int = 1536
    num_layers: int = 28
    num_heads: int = 12
    num_kv_heads: int = 2
    head_dim: int = 128
    intermediate_size: int = 8960
    rope_theta: float = 1e6
    rms_norm_eps: float = 1e-6
    tie_word_embeddings: bool = True
    attention_bias: bool = True         # Qwen2: bias on q/k/v projections
    qk_norm: bool = False               # Qwen3: RMSNorm on q and k per head
    max_position_embeddings: int = 32768
    # MoE (Qwen3-MoE)
    num_experts: int = 0
    num_experts_per_tok: int = 0
    moe_intermediate_size: int = 0
    norm_topk_prob: bool = True
    router_aux_loss_coef: float = 0.0
    shared_expert_intermediate_size: int = 0   # > 0: a dense expert every token visits, gated by sigmoid(w . x) (Qwen2-MoE)
    router_score_func: str = "softmax"      # softmax | sigmoid (DeepSeek-V3 style gates)
    router_scale: float = 1.0               # multiplies the selected gate weights
    num_expert_groups: int = 0              # > 0: group-limited routing (experts chosen inside the best groups only)
    num_limited_groups: int = 0
    router_bias_update_rate: float = 0.0    # > 0: auxiliary-loss-free balancing (selection bias nudged against expert load)
    decoder_sparse_step: int = 1
    mlp_only_layers: list[int] = field(default_factory=list)
    # critic / reward heads
    is_critic: bool = False
    # vision-language models (Qwen2-VL / Qwen2.5-VL): HF ``vision_config`` dict, placeholder ids, M-RoPE sections
    vision: Optional[dict] = None
    image_token_id: int = 151655
    video_token_id: int = 151656
    vision_start_token_id: int = 151652
    mrope_section: list[int] = field(default_factory=list)
    mrope_interleaved: bool = False         # Qwen3-VL: the three position streams alternate over the frequencies
    # hybrid linear / full attention stacks (Qwen3.5): per-layer token mixer, gated-delta-rule dimensions,
    # rotation of only the leading part of each head, sigmoid output gate on full attention, RMSNorm weights
    # stored as offsets from one
    layer_types: list[str] = field(default_factory=list)    # "linear_attention" | "full_attention" per layer; empty = all full
    linear_conv_kernel_dim: int = 4
    linear_key_head_dim: int = 128
    linear_value_head_dim: int = 128
    linear_num_key_heads: int = 16
    linear_num_value_heads: int = 32
    partial_rotary_factor: float = 1.0
    attn_output_gate: bool = False
    rms_norm_offset: bool = False

    @property
    def is_hybrid(self) -> bool:
        return any(t == "linear_attention" for t in self.layer_types)

    def layer_is_linear(self, i: int) -> bool:
        return bool(self.layer_types) and self.layer_types[i] == "linear_attention"

    @property
    def rotary_dim(self) -> int:
        return int(self.head_dim * self.partial_rotary_factor)

    @property
    def is_vlm(self) -> bool:
        return self.vision is not None

    def vision_config(self):
        from .vision import VisionConfig

        return VisionConfig.from_hf_dict(self.vision, self.hidden_size, self.vision.get("model_type", "qwen2_vl"))

    @property
    def q_size(self) -> int:
        return self.num_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_kv_heads * self.head_dim

    @property
    def is_moe(self) -> bool:
        return self.num_experts > 0

    def layer_is_moe(self, i: int) -> bool:
        return self.is_moe and i not in self.mlp_only_layers and (i + 1) % max(1, self.decoder_sparse_step) == 0

    def num_params(self) -> int:
        H, V, L = self.hidden_size, self.vocab_size, self.num_layers
        attn = H * (self.q_size + 2 * self.kv_size) + self.q_size * H
        if self.attention_bias:
            attn += self.q_size + 2 * self.kv_size
        if self.qk_norm:
            attn += 2 * self.head_dim
        dense_mlp = 3 * H * self.intermediate_size
        moe_mlp = self.num_experts * 3 * H * self.moe_intermediate_size + H * self.num_experts
        if self.shared_expert_intermediate_size:
            moe_mlp += 3 * H * self.shared_expert_intermediate_size + H
        if self.attn_output_gate:
            attn += H * self.q_size
        kd, vd = self.linear_num_key_heads * self.linear_key_head_dim, self.linear_num_value_heads * self.linear_value_head_dim
        nv = self.linear_num_value_heads
        linear = H * (2 * kd + 2 * vd + 2 * nv) + (2 * kd + vd) * self.linear_conv_kernel_dim + 2 * nv + self.linear_value_head_dim + vd * H
        total = V * H * (1 if self.tie_word_embeddings else 2) + H
        for i in range(L):
            total += (linear if self.layer_is_linear(i) else attn) + 2 * H + (moe_mlp if self.layer_is_moe(i) else dense_mlp)
        return total

    def flops_per_token(self, seq_len: int = 0, backward: bool = True) -> float:
        """Approximate training FLOPs per token (matmuls + causal attention)."""
        H, L = self.hidden_size, self.num_layers
        attn_proj = 2 * H * (self.q_size + 2 * self.kv_size) + 2 * self.q_size * H
        mlp = 0.0
        for i in range(L):
            if self.layer_is_moe(i):
                mlp += 6 * H * self.moe_intermediate_size * self.num_experts_per_tok + 2 * H * self.num_experts
            else:
                mlp += 6 * H * self.intermediate_size
        attn_core = L * 4 * self.q_size * (seq_len / 2)
        fwd = L * attn_proj + mlp + attn_core + 2 * H * self.vocab_size
        return fwd * (3 if backward else 1)

    # ------------------------------------------------------------------ HF interop
    @classmethod
    def from_hf_dict(cls, d: dict) -> "ModelConfig":
        mt = d.get("model_type", "qwen2")
        vl = None
        if mt == "qwen3_vl":
            vl = dict(d.get("vision_config") or {})
            vl["model_type"] = mt
            top = d
            d = dict(d.get("text_config") or {})
            for k in ("image_token_id", "video_token_id", "vision_start_token_id", "tie_word_embeddings"):
                if k in top:
                    d.setdefault(k, top[k])
            rs = d.get("rope_parameters") or d.get("rope_scaling") or {}
            d["_mrope_section"] = list(rs.get("mrope_section", [24, 20, 20]))
            d["_mrope_interleaved"] = bool(rs.get("mrope_interleaved", True))
            d.setdefault("rope_theta", rs.get("rope_theta", 5e6))
            d["attention_bias"] = bool(d.get("attention_bias", False))
            mt = "qwen3"
        if mt in ("qwen2_vl", "qwen2_5_vl"):
            # text fields sit at the top level (older checkpoints) or under ``text_config``
            vl = dict(d.get("vision_config") or {})
            vl["model_type"] = mt
            top = d
            d = dict(d.get("text_config") or {})
            for k, v in top.items():
                if k not in ("text_config", "vision_config"):
                    d.setdefault(k, v)
            rs = d.get("rope_scaling") or d.get("rope_parameters") or {}
            d["_mrope_section"] = list(rs.get("mrope_section", [16, 24, 24]))
            d["attention_bias"] = True
            mt = "qwen2"
        hybrid = {}
        if mt in ("qwen3_5", "qwen3_5_text", "qwen3_5_moe", "qwen3_5_moe_text"):
            moe5 = "moe" in mt
            # text-only use of the hybrid stack: the decoder's fields sit under ``text_config`` in full checkpoints
            if "text_config" in d:
                top, d = d, dict(d["text_config"])
                d.setdefault("tie_word_embeddings", top.get("tie_word_embeddings", False))
            rp = d.get("rope_parameters") or d.get("rope_scaling") or {}
            n_l = d["num_hidden_layers"]
            lt = d.get("layer_types")
            if not lt:
                iv = int(d.get("full_attention_interval", 4))
                lt = ["linear_attention" if (i + 1) % iv else "full_attention" for i in range(n_l)]
            hybrid = dict(layer_types=list(lt), linear_conv_kernel_dim=int(d.get("linear_conv_kernel_dim", 4)),
                          linear_key_head_dim=int(d.get("linear_key_head_dim", 128)), linear_value_head_dim=int(d.get("linear_value_head_dim", 128)),
                          linear_num_key_heads=int(d.get("linear_num_key_heads", 16)), linear_num_value_heads=int(d.get("linear_num_value_heads", 32)),
                          partial_rotary_factor=float(rp.get("partial_rotary_factor", d.get("partial_rotary_factor", 0.25))),
                          attn_output_gate=True, rms_norm_offset=True)
            d = dict(d)
            d.setdefault("rope_theta", rp.get("rope_theta", 1e7))
            d["attention_bias"] = bool(d.get("attention_bias", False))
            mt = "qwen3_5_moe" if moe5 else "qwen3_5"
            if moe5:
                d["norm_topk_prob"] = True
        arch = {"qwen2": "qwen2", "qwen3": "qwen3", "qwen3_moe": "qwen3_moe", "qwen2_moe": "qwen2_moe", "llama": "qwen2",
                "qwen3_5": "qwen3_5", "qwen3_5_moe": "qwen3_5_moe"}.get(mt)
        if arch is None:
            raise ValueError(f"unsupported model_type '{mt}'")
        heads = d["num_attention_heads"]
        hd = d.get("head_dim") or d["hidden_size"] // heads
        return cls(
            arch=arch, vocab_size=d["vocab_size"], hidden_size=d["hidden_size"], num_layers=d["num_hidden_layers"],
            num_heads=heads, num_kv_heads=d.get("num_key_value_heads", heads), head_dim=hd,
            intermediate_size=d.get("intermediate_size", 0), rope_theta=float(d.get("rope_theta", 1e4)),
            rms_norm_eps=float(d.get("rms_norm_eps", 1e-6)), tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            attention_bias=bool(d.get("attention_bias", mt in ("qwen2", "qwen2_moe"))), qk_norm=(mt in ("qwen3", "qwen3_moe", "qwen3_5", "qwen3_5_moe")),
            max_position_embeddings=d.get("max_position_embeddings", 32768),
            num_experts=d.get("num_experts") or d.get("num_local_experts") or 0, num_experts_per_tok=d.get("num_experts_per_tok", 0) or 0,
            moe_intermediate_size=d.get("moe_intermediate_size", 0) or 0, norm_topk_prob=bool(d.get("norm_topk_prob", mt != "qwen2_moe")),
            router_aux_loss_coef=float(d.get("router_aux_loss_coef", 0.0) or 0.0),
            shared_expert_intermediate_size=int(d.get("shared_expert_intermediate_size", 0) or 0) if mt in ("qwen2_moe", "qwen3_5_moe") else 0,
            router_score_func=d.get("scoring_func", d.get("router_score_func", "softmax")) or "softmax",
            router_scale=float(d.get("routed_scaling_factor", d.get("router_scale", 1.0)) or 1.0),
            num_expert_groups=int(d.get("n_group", d.get("num_expert_groups", 0)) or 0),
            num_limited_groups=int(d.get("topk_group", d.get("num_limited_groups", 0)) or 0),
            router_bias_update_rate=float(d.get("router_bias_update_rate", 0.0) or 0.0),
            decoder_sparse_step=d.get("decoder_sparse_step", 1) or 1, mlp_only_layers=list(d.get("mlp_only_layers", []) or []),
            vision=vl, mrope_section=list(d.get("_mrope_section", [])), mrope_interleaved=bool(d.get("_mrope_interleaved", False)),
            image_token_id=int(d.get("image_token_id", 151655)), video_token_id=int(d.get("video_token_id", 151656)),
            vision_start_token_id=int(d.get("vision_start_token_id", 151652)), **hybrid,
        )

    @classmethod
    def from_pretrained(cls, path: str) -> "ModelConfig":
        with open(os.path.join(path, "config.json")) as f:
            return cls.from_hf_dict(json.load(f))

    def to_hf_dict(self) -> dict:
        mt = self.arch
        d = dict(
            model_type=mt, architectures=[{"qwen2": "Qwen2ForCausalLM", "qwen3": "Qwen3ForCausalLM", "qwen3_5": "Qwen3_5ForCausalLM", "qwen3_5_moe": "Qwen3_5MoeForCausalLM",
                                           "qwen3_moe": "Qwen3MoeForCausalLM", "qwen2_moe": "Qwen2MoeForCausalLM"}[mt]],
            vocab_size=self.vocab_size, hidden_size=self.hidden_size, num_hidden_layers=self.num_layers,
            num_attention_heads=self.num_heads, num_key_value_heads=self.num_kv_heads, head_dim=self.head_dim,
            intermediate_size=self.intermediate_size, rope_theta=self.rope_theta, rms_norm_eps=self.rms_norm_eps,
            tie_word_embeddings=self.tie_word_embeddings, attention_bias=self.attention_bias,
            max_position_embeddings=self.max_position_embeddings, hidden_act="silu", torch_dtype="bfloat16",
        )
        if self.arch in ("qwen3_5", "qwen3_5_moe"):
            d.update(model_type=self.arch + "_text", layer_types=list(self.layer_types), linear_conv_kernel_dim=self.linear_conv_kernel_dim,
                     linear_key_head_dim=self.linear_key_head_dim, linear_value_head_dim=self.linear_value_head_dim,
                     linear_num_key_heads=self.linear_num_key_heads, linear_num_value_heads=self.linear_num_value_heads,
                     rope_parameters=dict(rope_type="default", rope_theta=self.rope_theta, partial_rotary_factor=self.partial_rotary_factor))
            d.pop("rope_theta", None)
        if self.is_vlm and self.vision.get("model_type") == "qwen3_vl":
            text = {k: v for k, v in d.items() if k not in ("model_type", "architectures", "rope_theta")}
            text.update(model_type="qwen3_vl_text", rope_parameters=dict(rope_type="default", rope_theta=self.rope_theta,
                                                                         mrope_section=list(self.mrope_section), mrope_interleaved=True))
            return dict(model_type="qwen3_vl", architectures=["Qwen3VLForConditionalGeneration"], text_config=text,
                        vision_config=dict(self.vision), image_token_id=self.image_token_id, video_token_id=self.video_token_id,
                        vision_start_token_id=self.vision_start_token_id, tie_word_embeddings=self.tie_word_embeddings,
                        torch_dtype="bfloat16")
        if self.is_vlm:
            vmt = self.vision.get("model_type", "qwen2_vl")
            d.update(model_type=vmt, architectures=[{"qwen2_vl": "Qwen2VLForConditionalGeneration",
                                                     "qwen2_5_vl": "Qwen2_5_VLForConditionalGeneration"}[vmt]],
                     vision_config=dict(self.vision), image_token_id=self.image_token_id, video_token_id=self.video_token_id,
                     vision_start_token_id=self.vision_start_token_id,
                     rope_scaling=dict(type="mrope", mrope_section=list(self.mrope_section)))
        if self.is_moe:
            d.update(num_experts=self.num_experts, num_experts_per_tok=self.num_experts_per_tok,
                     moe_intermediate_size=self.moe_intermediate_size, norm_topk_prob=self.norm_topk_prob,
                     router_aux_loss_coef=self.router_aux_loss_coef, decoder_sparse_step=self.decoder_sparse_step,
                     mlp_only_layers=self.mlp_only_layers)
            if self.shared_expert_intermediate_size:
                d["shared_expert_intermediate_size"] = self.shared_expert_intermediate_size
            if self.router_score_func != "softmax" or self.num_expert_groups or self.router_scale != 1.0 or self.router_bias_update_rate:
                d.update(scoring_func=self.router_score_func, routed_scaling_factor=self.router_scale, n_group=self.num_expert_groups,
                         topk_group=self.num_limited_groups, router_bias_update_rate=self.router_bias_update_rate)
        return d

    def save_pretrained(self, path: str) -> None:
        os.makedirs(path, exist_ok=True)
        with open(os.path.join(path, "config.json"), "w") as f:
            json.dump(self.to_hf_dict(), f, indent=2)


# named presets used by benchmarks and tests (random-init experiments)
PRESETS = {
    "tiny-qwen2": dict(arch="qwen2", vocab_size=1024, hidden_size=256, num_layers=4, num_heads=4, num_kv_heads=2,
                       head_dim=64, intermediate_size=688, rope_theta=1e4, tie_word_embeddings=True, attention_bias=True),
    "tiny-qwen3": dict(arch="qwen3", vocab_size=1024, hidden_size=256, num_layers=2, num_heads=4, num_kv_heads=2,
                       head_dim=64, intermediate_size=512, rope_theta=1e4, tie_word_embeddings=False,
                       attention_bias=False, qk_norm=True),
    "tiny-qwen3-moe": dict(arch="qwen3_moe", vocab_size=1024, hidden_size=256, num_layers=2, num_heads=4, num_kv_heads=2,
                           head_dim=64, intermediate_size=512, rope_theta=1e4, tie_word_embeddings=False,
                           attention_bias=False, qk_norm=True, num_experts=8, num_experts_per_tok=2,
                           moe_intermediate_size=128),
    "tiny-qwen3.5": dict(arch="qwen3_5", vocab_size=1024, hidden_size=128, num_layers=4, num_heads=4, num_kv_heads=2, head_dim=32,
                         intermediate_size=256, rope_theta=1e4, tie_word_embeddings=False, attention_bias=False, qk_norm=True,
                         layer_types=["linear_attention", "linear_attention", "linear_attention", "full_attention"],
                         linear_conv_kernel_dim=4, linear_key_head_dim=16, linear_value_head_dim=16, linear_num_key_heads=2,
                         linear_num_value_heads=4, partial_rotary_factor=0.25, attn_output_gate=True, rms_norm_offset=True),
    "tiny-qwen3.5-moe": dict(arch="qwen3_5_moe", vocab_size=1024, hidden_size=128, num_layers=4, num_heads=4, num_kv_heads=2, head_dim=32,
                             intermediate_size=0, rope_theta=1e4, tie_word_embeddings=False, attention_bias=False, qk_norm=True,
                             layer_types=["linear_attention", "linear_attention", "linear_attention", "full_attention"],
                             linear_conv_kernel_dim=4, linear_key_head_dim=16, linear_value_head_dim=16, linear_num_key_heads=2,
                             linear_num_value_heads=4, partial_rotary_factor=0.25, attn_output_gate=True, rms_norm_offset=True,
                             num_experts=8, num_experts_per_tok=2, moe_intermediate_size=64, shared_expert_intermediate_size=96,
                             norm_topk_prob=True),
    "qwen3.5-9b": dict(arch="qwen3_5", vocab_size=248320, hidden_size=4096, num_layers=32, num_heads=16, num_kv_heads=4, head_dim=256,
                       intermediate_size=12288, rope_theta=1e7, tie_word_embeddings=False, attention_bias=False, qk_norm=True,
                       layer_types=[("linear_attention" if (i + 1) % 4 else "full_attention") for i in range(32)],
                       linear_conv_kernel_dim=4, linear_key_head_dim=128, linear_value_head_dim=128, linear_num_key_heads=16,
                       linear_num_value_heads=32, partial_rotary_factor=0.25, attn_output_gate=True, rms_norm_offset=True),
    "tiny-qwen3-vl": dict(arch="qwen3", vocab_size=1024, hidden_size=256, num_layers=3, num_heads=4, num_kv_heads=2,
                          head_dim=64, intermediate_size=512, rope_theta=1e4, tie_word_embeddings=False, attention_bias=False, qk_norm=True,
                          image_token_id=1000, video_token_id=1001, vision_start_token_id=1002, mrope_section=[12, 10, 10],
                          mrope_interleaved=True,
                          vision=dict(model_type="qwen3_vl", depth=3, hidden_size=64, num_heads=4, intermediate_size=128, in_channels=3,
                                      patch_size=16, temporal_patch_size=2, spatial_merge_size=2, out_hidden_size=256,
                                      num_position_embeddings=64, deepstack_visual_indexes=[0, 1])),
    "tiny-qwen2-vl": dict(arch="qwen2", vocab_size=1024, hidden_size=256, num_layers=2, num_heads=4, num_kv_heads=2,
                          head_dim=64, intermediate_size=512, rope_theta=1e4, tie_word_embeddings=False, attention_bias=True,
                          image_token_id=1000, video_token_id=1001, vision_start_token_id=1002, mrope_section=[8, 12, 12],
                          vision=dict(model_type="qwen2_vl", depth=2, embed_dim=64, num_heads=4, mlp_ratio=2, in_chans=3, patch_size=14,
                                      temporal_patch_size=2, spatial_merge_size=2, hidden_size=256)),
    "tiny-qwen2.5-vl": dict(arch="qwen2", vocab_size=1024, hidden_size=256, num_layers=2, num_heads=4, num_kv_heads=2,
                            head_dim=64, intermediate_size=512, rope_theta=1e4, tie_word_embeddings=False, attention_bias=True,
                            image_token_id=1000, video_token_id=1001, vision_start_token_id=1002, mrope_section=[8, 12, 12],
                            vision=dict(model_type="qwen2_5_vl", depth=2, hidden_size=64, intermediate_size=96, num_heads=4, in_chans=3,
                                        patch_size=14, temporal_patch_size=2, spatial_merge_size=2, out_hidden_size=256, window_size=56,
                                        fullatt_block_indexes=[1])),
    "qwen2.5-vl-7b": dict(arch="qwen2", vocab_size=152064, hidden_size=3584, num_layers=28, num_heads=28, num_kv_heads=4,
                          head_dim=128, intermediate_size=18944, rope_theta=1e6, tie_word_embeddings=False, attention_bias=True,
                          max_position_embeddings=128000, mrope_section=[16, 24, 24],
                          vision=dict(model_type="qwen2_5_vl", depth=32, hidden_size=1280, intermediate_size=3420, num_heads=16, in_chans=3,
                                      patch_size=14, temporal_patch_size=2, spatial_merge_size=2, out_hidden_size=3584, window_size=112,
                                      fullatt_block_indexes=[7, 15, 23, 31])),
    "tiny-qwen2-moe": dict(arch="qwen2_moe", vocab_size=1024, hidden_size=256, num_layers=2, num_heads=4, num_kv_heads=2,
                           head_dim=64, intermediate_size=512, rope_theta=1e4, tie_word_embeddings=False, attention_bias=True,
                           num_experts=8, num_experts_per_tok=2, moe_intermediate_size=128, shared_expert_intermediate_size=256,
                           norm_topk_prob=False),
    "qwen2.5-1.5b": dict(arch="qwen2", vocab_size=151936, hidden_size=1536, num_layers=28, num_heads=12, num_kv_heads=2,
                         head_dim=128, intermediate_size=8960, rope_theta=1e6, tie_word_embeddings=True,
                         attention_bias=True),
    "qwen3-8b": dict(arch="qwen3", vocab_size=151936, hidden_size=4096, num_layers=36, num_heads=32, num_kv_heads=8,
                     head_dim=128, intermediate_size=12288, rope_theta=1e6, tie_word_embeddings=False,
                     attention_bias=False, qk_norm=True, max_position_embeddings=40960),
    "qwen3-30b-a3b": dict(arch="qwen3_moe", vocab_size=151936, hidden_size=2048, num_layers=48, num_heads=32,
                          num_kv_heads=4, head_dim=128, intermediate_size=6144, rope_theta=1e6,
                          tie_word_embeddings=False, attention_bias=False, qk_norm=True, num_experts=128,
                          num_experts_per_tok=8, moe_intermediate_size=768, max_position_embeddings=40960),
}


def preset(name: str, **overrides) -> ModelConfig:
    if name not in PRESETS:
        raise KeyError(f"unknown model preset '{name}' (have {sorted(PRESETS)})")
    d = dict(PRESETS[name])
    d.update(overrides)
    return ModelConfig(**d)
