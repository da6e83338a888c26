"""Logit parity of the decoder families against the Hugging Face implementations: a random tiny HF
model is saved, loaded through ``hf_io`` into this framework's model (fused QKV / gate-up layout,
stacked experts), and both are run on the same packed batch (CPU, fp32). Mirrors the reference's
``tests/experimental/archon/test_hf_parity_*.py``."""
import tempfile

import pytest
import torch

from areal_b200.models import hf_io
from areal_b200.models.config import ModelConfig
from areal_b200.models.decoder import build_model

COMMON = dict(vocab_size=512, hidden_size=128, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2, intermediate_size=256,
              rope_theta=1e4, max_position_embeddings=512, rms_norm_eps=1e-6)


def _hf_model(family):
    tr = pytest.importorskip("transformers")
    torch.manual_seed(0)
    if family == "qwen2":
        cfg = tr.Qwen2Config(**COMMON, tie_word_embeddings=True)
        return tr.Qwen2ForCausalLM(cfg)
    if family == "qwen3":
        cfg = tr.Qwen3Config(**COMMON, head_dim=64, tie_word_embeddings=False)
        return tr.Qwen3ForCausalLM(cfg)
    if family == "qwen3_moe":
        if not hasattr(tr, "Qwen3MoeForCausalLM"):
            pytest.skip("transformers without Qwen3-MoE")
        cfg = tr.Qwen3MoeConfig(**COMMON, head_dim=64, tie_word_embeddings=False, num_experts=8, num_experts_per_tok=2, moe_intermediate_size=64,
                                norm_topk_prob=True, decoder_sparse_step=1, mlp_only_layers=[])
        return tr.Qwen3MoeForCausalLM(cfg)
    if family == "qwen2_moe":
        if not hasattr(tr, "Qwen2MoeForCausalLM"):
            pytest.skip("transformers without Qwen2-MoE")
        cfg = tr.Qwen2MoeConfig(**COMMON, tie_word_embeddings=False, num_experts=8, num_experts_per_tok=2, moe_intermediate_size=64,
                                shared_expert_intermediate_size=96, norm_topk_prob=False, decoder_sparse_step=1, mlp_only_layers=[])
        return tr.Qwen2MoeForCausalLM(cfg)
    if family == "qwen3_5":
        if not hasattr(tr, "Qwen3_5ForCausalLM"):
            pytest.skip("transformers without Qwen3.5")
        cfg = tr.Qwen3_5TextConfig(**{**COMMON, "num_hidden_layers": 4}, head_dim=32, tie_word_embeddings=False,
                                   layer_types=["linear_attention", "linear_attention", "full_attention", "linear_attention"],
                                   linear_conv_kernel_dim=4, linear_key_head_dim=16, linear_value_head_dim=24, linear_num_key_heads=2,
                                   linear_num_value_heads=4)
        return tr.Qwen3_5ForCausalLM(cfg)
    if family == "qwen3_5_moe":
        if not hasattr(tr, "Qwen3_5MoeForCausalLM"):
            pytest.skip("transformers without Qwen3.5-MoE")
        c = {k: v for k, v in COMMON.items() if k != "intermediate_size"}
        cfg = tr.Qwen3_5MoeTextConfig(**{**c, "num_hidden_layers": 4}, head_dim=32, tie_word_embeddings=False,
                                      layer_types=["linear_attention", "full_attention", "linear_attention", "linear_attention"],
                                      linear_conv_kernel_dim=4, linear_key_head_dim=16, linear_value_head_dim=24, linear_num_key_heads=2,
                                      linear_num_value_heads=4, num_experts=8, num_experts_per_tok=2, moe_intermediate_size=64,
                                      shared_expert_intermediate_size=96)
        return tr.Qwen3_5MoeForCausalLM(cfg)
    raise ValueError(family)


@pytest.mark.parametrize("family", ["qwen2", "qwen3", "qwen3_moe", "qwen2_moe", "qwen3_5", "qwen3_5_moe"])
def test_logits_match_hf(family):
    hf = _hf_model(family).float().eval()
    # make the parameters non-trivial where HF initialises constants (norm weights, biases)
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if p.dim() == 1:
                p.add_(torch.randn_like(p) * 0.1)
    with tempfile.TemporaryDirectory() as d:
        hf.save_pretrained(d, safe_serialization=True)
        mc = ModelConfig.from_pretrained(d)
        m = build_model(mc, dtype=torch.float32, device="cpu", seed=1)
        hf_io.load_model_hf(m, d)
        with tempfile.TemporaryDirectory() as d2:          # and our export is a checkpoint HF reads back identically
            hf_io.save_model_hf(m, d2)
            mc.save_pretrained(d2)
            back = type(hf).from_pretrained(d2, torch_dtype=torch.float32).eval()
            for (n, p), (_, q) in zip(hf.state_dict().items(), back.state_dict().items()):
                assert torch.equal(p, q), n
    m.eval()
    g = torch.Generator().manual_seed(3)
    lens = [17, 5, 29]
    seqs = [torch.randint(0, mc.vocab_size, (n,), generator=g) for n in lens]
    ids = torch.cat(seqs)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    with torch.no_grad():
        ours = m.logits(m(ids, cu, max_seqlen=max(lens)))
        theirs = torch.cat([hf(input_ids=s[None]).logits[0] for s in seqs])
    assert ours.shape == theirs.shape
    assert (ours - theirs).abs().max().item() < 2e-4, (ours - theirs).abs().max().item()


def test_block_quantised_fp8_checkpoint_is_dequantised_on_load(tmp_path):
    """A checkpoint whose projection weights are ``float8_e4m3fn`` with one fp32 multiplier per 128 x 128 block
    (``<name>_scale_inv``, ``quantization_config`` in ``config.json``) loads like an ordinary one: weights come out within
    fp8 rounding of the originals, scale tensors are not reported as unexpected, a scale kept in another shard is found
    through the index."""
    import json

    import torch
    from safetensors.torch import save_file

    from areal_b200.models import hf_io
    from areal_b200.models.config import preset
    from areal_b200.models.decoder import build_model

    cfg = preset("tiny-qwen3")
    src = build_model(cfg, dtype=torch.bfloat16, device="cpu", seed=4)
    named = dict(hf_io.native_to_hf_tensors(cfg, [(n, p.detach()) for n, p in src.named_parameters()]))

    def quant(w, bm=128, bn=128):
        R, C = w.shape
        gr, gc = -(-R // bm), -(-C // bn)
        pad = torch.zeros(gr * bm, gc * bn)
        pad[:R, :C] = w.float()
        amax = pad.view(gr, bm, gc, bn).abs().amax(dim=(1, 3)).clamp(min=1e-12)
        scale = amax / 448.0
        q = (pad.view(gr, bm, gc, bn) / scale[:, None, :, None]).view(gr * bm, gc * bn)[:R, :C].to(torch.float8_e4m3fn)
        return q, scale

    a, b = {}, {}
    for k, t in named.items():
        if k.endswith("proj.weight") and t.dim() == 2:
            q, sc = quant(t)
            a[k] = q
            (b if "layers.1." in k else a)[k + "_scale_inv"] = sc            # layer 1's scales go to the other shard
        else:
            a[k] = t.contiguous()
    save_file(a, str(tmp_path / "model-00001-of-00002.safetensors"))
    save_file(b, str(tmp_path / "model-00002-of-00002.safetensors"))
    wm = {k: "model-00001-of-00002.safetensors" for k in a}
    wm.update({k: "model-00002-of-00002.safetensors" for k in b})
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"metadata": {}, "weight_map": wm}))
    cfg.save_pretrained(str(tmp_path))
    cj = json.loads((tmp_path / "config.json").read_text())
    cj["quantization_config"] = {"quant_method": "fp8", "fmt": "e4m3", "weight_block_size": [128, 128]}
    (tmp_path / "config.json").write_text(json.dumps(cj))
    dst = build_model(cfg, dtype=torch.bfloat16, device="cpu", seed=9)
    hf_io.load_model_hf(dst, str(tmp_path))
    n_q = 0
    for (n, p), (_, q) in zip(src.named_parameters(), dst.named_parameters()):
        if n.endswith("_proj"):
            n_q += 1
            rel = float((p.detach().float() - q.detach().float()).norm() / p.detach().float().norm())
            assert 0 < rel < 0.05, (n, rel)                                   # e4m3 keeps 3 mantissa bits
        else:
            assert torch.equal(p, q), n
    assert n_q >= 4 * cfg.num_layers
    raw = dict(hf_io.iter_safetensors(str(tmp_path), dequant_fp8=False))
    assert any(k.endswith("_scale_inv") for k in raw) and any(t.dtype == torch.float8_e4m3fn for t in raw.values())
    w = torch.randn(200, 300)
    q, sc = quant(w)
    assert float((hf_io.dequant_block_fp8(q, sc).float() - w).norm() / w.norm()) < 0.05        # ragged last blocks
    import pytest

    with pytest.raises(ValueError, match="scale grid"):
        hf_io.dequant_block_fp8(q, sc[:1])
