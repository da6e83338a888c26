"""Vision-language path: image pre-processing, M-RoPE ids, tower + decoder parity against the
Hugging Face implementations (random tiny models, weights moved through a saved checkpoint),
train-engine step and rollout with images on CPU."""
import asyncio
import tempfile

import numpy as np
import pytest
import torch

from areal_b200.models import hf_io
from areal_b200.models.config import ModelConfig, preset
from areal_b200.models.decoder import PackedBatch, build_model
from areal_b200.models.vision import mrope_position_ids, num_image_tokens, preprocess_images, smart_resize

TEXT = dict(vocab_size=1024, hidden_size=256, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, intermediate_size=512,
            rope_theta=1e4, max_position_embeddings=4096, tie_word_embeddings=False, rms_norm_eps=1e-6,
            rope_scaling=dict(type="mrope", mrope_section=[8, 12, 12]))
IDS = dict(image_token_id=1000, video_token_id=1001, vision_start_token_id=1002)


def _images():
    rng = np.random.default_rng(0)
    return [rng.integers(0, 255, (60, 100, 3), dtype=np.uint8), rng.integers(0, 255, (150, 120, 3), dtype=np.uint8)]


def test_smart_resize_and_patch_order():
    assert smart_resize(60, 100, 28, 28 * 28, 28 * 28 * 36) == (56, 112)
    h, w = smart_resize(3000, 4000, 28, 56 * 56, 28 * 28 * 1280)
    assert h % 28 == 0 and w % 28 == 0 and h * w <= 28 * 28 * 1280
    cfg = preset("tiny-qwen2-vl").vision_config()
    img = np.zeros((56, 56, 3), dtype=np.uint8)
    img[:28, 28:] = 255                      # the top-right 28x28 merge block is white
    px, grid = preprocess_images([img], cfg, 28 * 28, 28 * 28 * 4)
    assert grid.tolist() == [[1, 4, 4]] and px.shape == (16, cfg.patch_dim)
    # merge-block order: rows 4..7 are the four patches of block (0, 1)
    bright = px.mean(-1) > 0
    assert bright.tolist() == [False] * 4 + [True] * 4 + [False] * 8


def test_mrope_positions():
    grid = torch.tensor([[1, 4, 8]])
    ids = torch.tensor([5, 6, 1002] + [1000] * 8 + [7, 8])
    pos, delta = mrope_position_ids(ids, grid, 1000)
    assert pos[0].tolist() == [0, 1, 2] + [3] * 8 + [7, 8]
    assert pos[1].tolist() == [0, 1, 2] + [3, 3, 3, 3, 4, 4, 4, 4] + [7, 8]
    assert pos[2].tolist() == [0, 1, 2] + [3, 4, 5, 6] * 2 + [7, 8]
    assert delta == 9 - 13
    p2, d2 = mrope_position_ids(torch.tensor([1, 2, 3]), None, 1000)
    assert p2.tolist() == [[0, 1, 2]] * 3 and d2 == 0


@pytest.mark.parametrize("family", ["qwen2_vl", "qwen2_5_vl"])
def test_vlm_matches_hf(family):
    tr = pytest.importorskip("transformers")
    torch.manual_seed(0)
    if family == "qwen2_vl":
        if not hasattr(tr, "Qwen2VLForConditionalGeneration"):
            pytest.skip("transformers without Qwen2-VL")
        hcfg = tr.Qwen2VLConfig(**TEXT, **IDS, vision_config=dict(depth=2, embed_dim=64, num_heads=4, mlp_ratio=2, in_chans=3, patch_size=14,
                                                                     temporal_patch_size=2, spatial_merge_size=2, hidden_size=256))
        hf = tr.Qwen2VLForConditionalGeneration(hcfg)
    else:
        if not hasattr(tr, "Qwen2_5_VLForConditionalGeneration"):
            pytest.skip("transformers without Qwen2.5-VL")
        hcfg = tr.Qwen2_5_VLConfig(**TEXT, **IDS, vision_config=dict(depth=2, hidden_size=64, intermediate_size=96, num_heads=4, in_chans=3,
                                                                       patch_size=14, temporal_patch_size=2, spatial_merge_size=2,
                                                                       out_hidden_size=256, window_size=56, fullatt_block_indexes=[1]))
        hf = tr.Qwen2_5_VLForConditionalGeneration(hcfg)
    hf = hf.float().eval()
    with tempfile.TemporaryDirectory() as d:
        hf.save_pretrained(d, safe_serialization=True)
        mc = ModelConfig.from_pretrained(d)
        assert mc.is_vlm and mc.mrope_section == [8, 12, 12] and mc.image_token_id == 1000
        m = build_model(mc, dtype=torch.float32, device="cpu", seed=0)
        hf_io.load_model_hf(m, d)
        # and back: our HF export has the same tensors
        with tempfile.TemporaryDirectory() as d2:
            hf_io.save_model_hf(m, d2)
            back = dict(hf_io.iter_safetensors(d2))
            ref_sd = hf.state_dict()
            assert any(k.startswith("visual.") for k in back)
            for k, v in back.items():
                cands = [k, "model." + k, k.replace("model.", "model.language_model.", 1)]
                hit = next((c for c in cands if c in ref_sd), None)
                assert hit is not None, k
                assert torch.equal(ref_sd[hit], v), k
    m.eval()
    px, grid = preprocess_images(_images(), m.vcfg, min_pixels=28 * 28, max_pixels=28 * 28 * 36)
    nt = num_image_tokens(grid)
    seq = [5, 6, 1002] + [1000] * nt[0] + [7, 8, 1002] + [1000] * nt[1] + [9, 10, 11]
    ids = torch.tensor(seq)
    with torch.no_grad():
        pos3, _, where = m.packed_mrope(ids, [0, len(seq)], grid)
        assert where.tolist() == (ids == 1000).nonzero().view(-1).tolist()
        kw = dict(input_ids=ids[None], pixel_values=px, image_grid_thw=grid, attention_mask=torch.ones(1, len(seq), dtype=torch.long),
                  position_ids=pos3[:, None, :])
        try:
            ref = hf(**kw, mm_token_type_ids=(ids == 1000).long()[None]).logits[0]
        except TypeError:
            ref = hf(**kw).logits[0]
        pb = PackedBatch(torch.tensor([0, len(seq)], dtype=torch.int32), torch.arange(len(seq)), len(seq), len(seq))
        out = m.logits(m.forward_hidden(ids, pb, mm={"pixel_values": px, "image_grid_thw": grid}))
    assert (out - ref).abs().max().item() < 1e-4
    # the tower alone, two images in one call (frames / windows never attend across images)
    with torch.no_grad():
        both = m.visual(px, grid)
        first = m.visual(px[: int(grid[0].prod())], grid[:1])
    assert torch.allclose(both[: nt[0]], first, atol=1e-5)


def _vlm_batch(mc, vcfg):
    unit = vcfg.patch_size * vcfg.spatial_merge_size
    px, grid = preprocess_images(_images(), vcfg, min_pixels=unit * unit, max_pixels=unit * unit * 16)
    nt = num_image_tokens(grid)
    rows, mm = [], []
    g = torch.Generator().manual_seed(0)
    for i in range(4):
        if i < 2:
            a = int(grid[:i].prod(-1).sum())
            b = a + int(grid[i].prod())
            seq = [5, 1002] + [1000] * nt[i] + torch.randint(3, 900, (10 + i,), generator=g).tolist()
            mm.append({"pixel_values": px[a:b], "image_grid_thw": grid[i:i + 1]})
        else:
            seq = torch.randint(3, 900, (20 + i,), generator=g).tolist()
            mm.append(None)
        rows.append(seq)
    L = max(len(r) for r in rows)
    ids = torch.zeros(4, L, dtype=torch.long)
    am = torch.zeros(4, L, dtype=torch.bool)
    for i, r in enumerate(rows):
        ids[i, :len(r)] = torch.tensor(r)
        am[i, :len(r)] = True
    lm = am.clone().int()
    lm[:, :8] = 0
    lm[torch.arange(4), am.sum(1) - 1] = 0
    lm = lm * (ids != 1000)
    return dict(input_ids=ids, attention_mask=am, loss_mask=lm, multi_modal_input=mm)


@pytest.mark.parametrize("name", ["tiny-qwen2.5-vl", "tiny-qwen3-vl"])
def test_train_engine_steps_a_vlm_and_tower_gets_gradients(name):
    from areal_b200.api.cli_args import MicroBatchSpec, OptimizerConfig, TrainEngineConfig
    from areal_b200.engine.train_engine import B200TrainEngine

    mc = preset(name)
    eng = B200TrainEngine(TrainEngineConfig(init_from_scratch=True, dtype="float32", optimizer=OptimizerConfig(lr=1e-2),
                                            mb_spec=MicroBatchSpec(max_tokens_per_mb=64)))
    eng.create_process_group()
    eng.initialize(model_config=mc, seed=3)
    batch = _vlm_batch(mc, eng.model.vcfg)

    def loss_fn(logp, ent, mb):
        m = mb["loss_mask"].bool()
        return -(logp * m).sum() / m.sum().clamp(min=1)

    before = eng.model.visual.blocks[0].attn.qkv.weight.detach().clone()
    losses = [eng.train_batch(batch, loss_fn, lambda mb: mb["loss_mask"].count_nonzero())["loss"] for _ in range(4)]
    assert losses[-1] < losses[0]
    assert not torch.equal(before, eng.model.visual.blocks[0].attn.qkv.weight.detach())
    if eng.model.vcfg.deepstack_visual_indexes:           # the deep-stack mergers train too
        assert eng.model.visual.deepstack_merger_list[0].linear_fc1.weight.main_grad is not None
    lp = eng.forward_batch(batch)
    assert lp.shape == batch["input_ids"].shape and torch.isfinite(lp).all()
    eng.destroy()


@pytest.mark.parametrize("name", ["tiny-qwen2-vl", "tiny-qwen3-vl"])
def test_vision_rlvr_workflow_rollout_cpu(name):
    from areal_b200.api.cli_args import GenerationHyperparameters, InferenceEngineConfig, NativeInferConfig
    from areal_b200.engine.infer_engine import NativeInferenceEngine
    from areal_b200.rollout.workflows.vision_rlvr import VisionRLVRWorkflow, expand_image_placeholders

    assert expand_image_placeholders([1, 1000, 2, 1000], [2, 3], 1000) == [1, 1000, 1000, 2, 1000, 1000, 1000]
    mc = preset(name)
    eng = NativeInferenceEngine(InferenceEngineConfig(), NativeInferConfig(max_running_requests=4, context_length=256), model_config=mc)
    eng.initialize(device="cpu", start_executor=False)
    try:
        seen = {}

        def reward(prompt, completion, prompt_ids, completion_ids, **kw):
            seen["n_prompt"] = len(prompt_ids)
            return float(len(completion_ids))

        from PIL import Image

        pil = Image.fromarray(_images()[0])
        wf = VisionRLVRWorkflow(reward, GenerationHyperparameters(n_samples=2, max_new_tokens=5, max_tokens=200, greedy=True), vision_config=eng.model.vcfg,
                                image_token_id=mc.image_token_id, reward_in_process=True, min_pixels=32 * 32, max_pixels=32 * 32 * 16)
        out = asyncio.run(wf.arun_episode(eng, {"input_ids": [5, 6, 1002, 1000, 7], "images": [pil]}))
        assert out["input_ids"].shape[0] == 2 and len(out["multi_modal_input"]) == 2
        grid = out["multi_modal_input"][0]["image_grid_thw"]
        n_img = num_image_tokens(grid)[0]
        assert seen["n_prompt"] == 4 + n_img and (out["input_ids"][0] == 1000).sum() == n_img
        assert out["rewards"].tolist() == [5.0, 5.0]
        # greedy samples of the same prompt agree, and differ from the text-only continuation
        assert torch.equal(out["input_ids"][0], out["input_ids"][1])
    finally:
        eng.destroy()


def test_qwen3_vl_matches_hf():
    """Qwen3-VL: learned position table resampled to the patch grid, tanh-GELU tower, deep-stack
    features added after the first decoder layers, interleaved M-RoPE."""
    tr = pytest.importorskip("transformers")
    if not hasattr(tr, "Qwen3VLForConditionalGeneration"):
        pytest.skip("transformers without Qwen3-VL")
    torch.manual_seed(0)
    text = dict(vocab_size=1024, hidden_size=256, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
                intermediate_size=512, max_position_embeddings=4096, rms_norm_eps=1e-6,
                rope_parameters=dict(rope_type="default", rope_theta=1e4, mrope_section=[12, 10, 10], mrope_interleaved=True))
    vis = dict(depth=3, hidden_size=64, num_heads=4, intermediate_size=128, in_channels=3, patch_size=16, temporal_patch_size=2,
               spatial_merge_size=2, out_hidden_size=256, num_position_embeddings=64, deepstack_visual_indexes=[0, 2])
    hf = tr.Qwen3VLForConditionalGeneration(tr.Qwen3VLConfig(text_config=text, vision_config=vis, tie_word_embeddings=False, **IDS)).float().eval()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if p.dim() == 1:
                p.add_(torch.randn_like(p) * 0.1)
    with tempfile.TemporaryDirectory() as d:
        hf.save_pretrained(d, safe_serialization=True)
        mc = ModelConfig.from_pretrained(d)
        assert mc.is_vlm and mc.mrope_interleaved and mc.qk_norm and mc.vision_config().deepstack_visual_indexes == [0, 2]
        m = build_model(mc, dtype=torch.float32, device="cpu", seed=0)
        hf_io.load_model_hf(m, d)
        with tempfile.TemporaryDirectory() as d2:
            hf_io.save_model_hf(m, d2)
            mc.save_pretrained(d2)
            back = tr.Qwen3VLForConditionalGeneration.from_pretrained(d2, torch_dtype=torch.float32)
            ref_sd = hf.state_dict()
            for k, v in back.state_dict().items():
                assert torch.equal(ref_sd[k], v), k
    m.eval()
    px, grid = preprocess_images(_images(), m.vcfg, min_pixels=32 * 32, max_pixels=32 * 32 * 30)
    nt = num_image_tokens(grid)
    seq = [5, 6, 1002] + [1000] * nt[0] + [7, 8, 1002] + [1000] * nt[1] + [9, 10, 11]
    ids = torch.tensor(seq)
    with torch.no_grad():
        pos3, _, where = m.packed_mrope(ids, [0, len(seq)], grid)
        kw = dict(input_ids=ids[None], pixel_values=px, image_grid_thw=grid, attention_mask=torch.ones(1, len(seq), dtype=torch.long),
                  position_ids=pos3[:, None, :])
        try:
            ref = hf(**kw, mm_token_type_ids=(ids == 1000).long()[None]).logits[0]
        except TypeError:
            ref = hf(**kw).logits[0]
        pb = PackedBatch(torch.tensor([0, len(seq)], dtype=torch.int32), torch.arange(len(seq)), len(seq), len(seq))
        out = m.logits(m.forward_hidden(ids, pb, mm={"pixel_values": px, "image_grid_thw": grid}))
        # text only: the three streams coincide
        t_ids = torch.tensor([5, 6, 7, 8, 9, 10])
        ref_t = hf(input_ids=t_ids[None]).logits[0]
        out_t = m.logits(m(t_ids, torch.tensor([0, 6], dtype=torch.int32), max_seqlen=6))
    assert (out - ref).abs().max().item() < 1e-4, (out - ref).abs().max().item()
    assert (out_t - ref_t).abs().max().item() < 1e-4
