"""RLVR for vision-language models: like :class:`RLVRWorkflow`, but every prompt carries
images. The prompt's image placeholders are expanded to one token per merged patch, the
pictures travel to the inference engine with the request, and every trajectory keeps its
``multi_modal_input`` (patches + grid) so the trainer can re-run the tower.

Reference: ``areal/workflow/vision_rlvr.py`` (processor call :60-82, ``image_data`` on the
request :88-95, ``multi_modal_input`` in the result :120-133).
"""
from __future__ import annotations

import asyncio
import uuid
from typing import Any, Callable, Optional

import torch

from ...api.cli_args import GenerationHyperparameters
from ...api.io_struct import ModelRequest
from ...models.vision import VisionConfig, num_image_tokens, preprocess_images
from ...utils import data as D
from ...utils import stats_tracker
from ...utils.image import load_image
from .. import workflow_context as wctx
from .rlvr import RLVRWorkflow, default_get_input_ids


def expand_image_placeholders(input_ids: list[int], counts: list[int], image_token_id: int) -> list[int]:
    """Replaces the i-th single image placeholder by ``counts[i]`` copies (a prompt that is
    already expanded is returned unchanged)."""
    n_single = sum(1 for t in input_ids if t == image_token_id)
    if n_single == sum(counts):
        return list(input_ids)
    if n_single != len(counts):
        raise ValueError(f"{n_single} image placeholders for {len(counts)} images")
    out, k = [], 0
    for t in input_ids:
        if t == image_token_id:
            out += [image_token_id] * counts[k]
            k += 1
        else:
            out.append(t)
    return out


class VisionRLVRWorkflow(RLVRWorkflow):
    def __init__(self, reward_fn: Callable[..., float], gconfig: GenerationHyperparameters, tokenizer=None, processor=None,
                 vision_config: Optional[VisionConfig] = None, image_token_id: int = 151655, enable_thinking: bool = False,
                 get_input_ids_fn: Callable = default_get_input_ids, reward_in_process: bool = False, reward_timeout: float = 15.0,
                 min_pixels: int = 56 * 56, max_pixels: int = 14 * 14 * 4 * 1280):
        super().__init__(reward_fn, gconfig, tokenizer, enable_thinking, get_input_ids_fn, reward_in_process, reward_timeout)
        self.processor = processor
        self.vcfg = vision_config or VisionConfig()
        self.image_token_id = image_token_id
        self.min_pixels, self.max_pixels = min_pixels, max_pixels

    def _process(self, data: dict[str, Any]):
        images = [load_image(im) for im in (data.get("images") or [])]
        if self.processor is not None and "messages" in data:
            # an HF processor does tokenisation, placeholder expansion and patching in one call
            text = self.processor.apply_chat_template(data["messages"], tokenize=False, add_generation_prompt=True)
            enc = self.processor(images=images or None, text=text, padding=False, return_tensors="pt")
            ids = enc["input_ids"][0].tolist()
            return ids, enc.get("pixel_values"), enc.get("image_grid_thw"), images
        ids = self.get_input_ids_fn(data, self.tokenizer, self.enable_thinking)
        if not images:
            return ids, None, None, images
        px, grid = preprocess_images(images, self.vcfg, self.min_pixels, self.max_pixels)
        ids = expand_image_placeholders(ids, num_image_tokens(grid, self.vcfg.spatial_merge_size), self.image_token_id)
        return ids, px, grid, images

    async def _one_vision_sample(self, engine, ids, px, grid, images, data, gconfig):
        meta = {} if px is None else {"pixel_values": px, "image_grid_thw": grid}
        req = ModelRequest(rid=uuid.uuid4().hex, input_ids=ids, gconfig=gconfig, tokenizer=self.tokenizer,
                           image_data=images or None, metadata=meta)
        resp = await engine.agenerate(req)
        prompt_str = completion_str = None
        if self.tokenizer is not None:
            prompt_str = self.tokenizer.decode(ids)
            completion_str = self.tokenizer.decode(resp.output_tokens)
        reward = await self._reward(prompt_str, completion_str, resp.input_tokens, resp.output_tokens, data)
        stats_tracker.get(wctx.stat_scope()).scalar(reward=reward, gen_len=len(resp.output_tokens))
        seq = resp.input_tokens + resp.output_tokens
        n_in, n_out = resp.input_len, resp.output_len
        out = dict(
            input_ids=torch.tensor(seq, dtype=torch.int32).unsqueeze(0),
            loss_mask=torch.tensor([0] * n_in + [1] * n_out, dtype=torch.int32).unsqueeze(0),
            logprobs=torch.tensor([0.0] * n_in + resp.output_logprobs, dtype=torch.float32).unsqueeze(0),
            versions=torch.tensor([-1] * n_in + resp.output_versions, dtype=torch.int32).unsqueeze(0),
            turn_ids=torch.tensor([-1] * n_in + [0] * n_out, dtype=torch.int32).unsqueeze(0),
            attention_mask=torch.ones(1, len(seq), dtype=torch.bool),
            rewards=torch.tensor([float(reward)], dtype=torch.float32),
        )
        out["multi_modal_input"] = [None if px is None else {"pixel_values": px, "image_grid_thw": grid}]
        return out

    async def arun_episode(self, engine, data: dict[str, Any]) -> Optional[dict[str, Any]]:
        ids, px, grid, images = self._process(data)
        n = max(1, self.gconfig.n_samples)
        g1 = self.gconfig.new(n_samples=1)
        data = {k: v for k, v in data.items() if k != "images"}
        samples = await asyncio.gather(*[self._one_vision_sample(engine, ids, px, grid, images, data, g1) for _ in range(n)])
        return D.concat_padded_tensors(list(samples))
