"""Datasets keyed by ``(path, type)`` (reference: ``areal/dataset/__init__.py``
``get_custom_dataset``): synthetic arithmetic / random-token sets for offline experiments,
and loaders for gsm8k-style JSON/parquet files on disk."""
from __future__ import annotations

import json
import os
import random
from typing import Sequence, Any, Callable, Optional

import torch
from torch.utils.data import Dataset


VALID_DATASETS = ["gsm8k", "clevr_count_70k", "geometry3k", "virl39k", "hh-rlhf", "torl_data", "synthetic/arithmetic", "synthetic/random_tokens",
                  "synthetic/countdown", "synthetic/count_shapes"]


class CharTokenizer:
    """Character-level tokenizer over ``0-9 + = space`` plus pad / eos (ids stable)."""

    def __init__(self):
        self.chars = list("0123456789+= ")
        self.pad_token_id = len(self.chars)
        self.eos_token_id = len(self.chars) + 1
        self.vocab_size = len(self.chars) + 2
        self._idx = {c: i for i, c in enumerate(self.chars)}

    def encode(self, text: str) -> list[int]:
        return [self._idx[c] for c in text if c in self._idx]

    def decode(self, ids) -> str:
        out = []
        for i in ids:
            i = int(i)
            if i == self.eos_token_id:
                break
            if 0 <= i < len(self.chars):
                out.append(self.chars[i])
        return "".join(out)

    def save_pretrained(self, path: str):
        os.makedirs(path, exist_ok=True)
        with open(os.path.join(path, "char_tokenizer.json"), "w") as f:
            json.dump({"chars": self.chars}, f)


class ArithmeticDataset(Dataset):
    """Seeded prompts ``'a+b='`` with a, b uniform in 0..99, char-level tokens left-padded with
    spaces to ``pad_to`` tokens; the answer is kept for the reward function."""

    def __init__(self, size: int = 1024, seed: int = 1, pad_to: int = 16, max_operand: int = 99):
        rng = random.Random(seed)
        self.tok = CharTokenizer()
        self.items = []
        for _ in range(size):
            a, b = rng.randint(0, max_operand), rng.randint(0, max_operand)
            text = f"{a}+{b}="
            text = " " * max(0, pad_to - len(text)) + text
            self.items.append(dict(input_ids=self.tok.encode(text), answer=a + b, prompt=text))

    def __len__(self):
        return len(self.items)

    def __getitem__(self, i):
        return self.items[i]


def arithmetic_reward_fn(prompt, completion, prompt_ids, completion_ids, answer=None, **kwargs) -> float:
    tok = CharTokenizer()
    text = completion if completion is not None else tok.decode(completion_ids)
    text = text.strip()
    digits = ""
    for ch in text:
        if ch.isdigit():
            digits += ch
        else:
            break
    try:
        return 1.0 if digits and int(digits) == int(answer) else 0.0
    except (TypeError, ValueError):
        return 0.0


class RandomTokenDataset(Dataset):
    """Uniform-random prompt token ids with forced response lengths drawn from a log-normal
    (forced-length benchmarks); rewards are Bernoulli from the seed.

    ``n_samples > 0``: every item carries ``max_new_tokens_per_sample`` -- one independent draw
    per sample of the prompt's group (the samples of a group then finish at different times, as
    they do with real generations). ``n_samples = 0``: one draw per prompt (``max_new_tokens``),
    shared by the whole group."""

    def __init__(self, size: int, prompt_len: int, vocab_size: int, seed: int = 1, median_len: int = 1024,
                 max_len: int = 4096, sigma: float = 0.6, min_len: int = 16, n_samples: int = 0):
        g = torch.Generator().manual_seed(seed)
        self.prompts = torch.randint(0, vocab_size, (size, prompt_len), generator=g, dtype=torch.int32)
        z = torch.randn(size, max(1, n_samples), generator=g)
        lens = (median_len * torch.exp(sigma * z)).clamp(min_len, max_len).long()
        self.per_sample = n_samples > 0
        self.lens = lens.tolist()
        self.rewards = (torch.rand(size, generator=g) < 0.5).float().tolist()

    def __len__(self):
        return self.prompts.shape[0]

    def __getitem__(self, i):
        item = dict(input_ids=self.prompts[i].tolist(), reward=self.rewards[i], idx=i)
        if self.per_sample:
            item["max_new_tokens_per_sample"] = list(self.lens[i])
        else:
            item["max_new_tokens"] = self.lens[i][0]
        return item


def bernoulli_reward_fn(prompt, completion, prompt_ids, completion_ids, reward=0.0, idx=0, **kwargs) -> float:
    """Bernoulli(0.5) reward that is deterministic in (prompt index, sampled completion), so
    the samples of one group differ and group-normalised advantages are non-zero."""
    import zlib

    h = zlib.crc32(bytes(int(t) & 0xFF for t in completion_ids[:64])) ^ (int(idx) * 2654435761 & 0xFFFFFFFF)
    return float((h >> 7) & 1)


def small_id_fraction_reward_fn(prompt, completion, prompt_ids, completion_ids, threshold: int = 10, **kwargs) -> float:
    """Shaped synthetic reward a random-init model can climb within a few steps: the fraction
    of generated token ids below ``threshold``."""
    return sum(1 for t in completion_ids if t < threshold) / max(1, len(completion_ids))


class CountdownDataset(Dataset):
    """Procedural Countdown problems (offline stand-in for the reference's ``examples/countdown``
    data): ``numbers`` and a reachable ``target``; items carry a ``prompt`` / ``messages`` pair."""

    def __init__(self, size: int = 4096, seed: int = 1, n_numbers: int = 3, max_number: int = 50, tokenizer=None):
        self.size, self.seed, self.n, self.max_number, self.tokenizer = size, seed, n_numbers, max_number, tokenizer

    def __len__(self):
        return self.size

    def __getitem__(self, i):
        rng = random.Random(self.seed * 7919 + i)
        nums = [rng.randint(1, self.max_number) for _ in range(self.n)]
        val = nums[0]
        for x in nums[1:]:
            op = rng.choice("+-*")
            val = val + x if op == "+" else (val - x if op == "-" else val * x)
        q = (f"Using the numbers {nums}, create an equation that equals {val}. Use each number exactly once with + - * /. "
             "Put the equation inside <answer> </answer>.")
        item = dict(prompt=q, messages=[{"role": "user", "content": q}], numbers=nums, target=val, idx=i)
        if self.tokenizer is not None:
            item["input_ids"] = list(self.tokenizer.encode(q))
        return item


class CountShapesDataset(Dataset):
    """Procedural vision-language task (offline stand-in for clevr_count_70k): a picture with
    ``k`` bright squares on a dark canvas; the question asks for ``k``. Items carry ``images``
    (PIL), ``input_ids`` (``[bos, vision_start, image, question tokens...]``) and ``answer``."""

    def __init__(self, size: int = 1024, seed: int = 1, image_size: int = 112, max_shapes: int = 6, image_token_id: int = 1000,
                 vision_start_token_id: int = 1002, question_ids: Sequence[int] = (11, 12, 13)):
        self.size, self.seed, self.image_size, self.max_shapes = size, seed, image_size, max_shapes
        self.prefix = [5, vision_start_token_id, image_token_id] + list(question_ids)

    def __len__(self):
        return self.size

    def __getitem__(self, i):
        import numpy as np
        from PIL import Image

        rng = np.random.default_rng(self.seed * 1000003 + i)
        k = int(rng.integers(1, self.max_shapes + 1))
        S = self.image_size
        img = np.full((S, S, 3), 16, dtype=np.uint8)
        cell = S // 4
        for c in rng.choice(16, size=k, replace=False):
            y, x = (c // 4) * cell + cell // 4, (c % 4) * cell + cell // 4
            img[y:y + cell // 2, x:x + cell // 2] = rng.integers(160, 255, 3)
        return dict(images=[Image.fromarray(img)], input_ids=list(self.prefix), answer=k, idx=i)


def count_shapes_reward_fn(prompt, completion, prompt_ids, completion_ids, answer=None, **kwargs) -> float:
    """1 when the first generated token id equals ``20 + answer`` (digit tokens of the toy vocabulary)."""
    return float(bool(completion_ids) and int(completion_ids[0]) == 20 + int(answer))


def _record_images(r: dict) -> list:
    """Images of a record in the layouts of geometry3k / clevr_count (``images`` as a list of
    ``{"bytes": ...}`` / bytes / paths, or a single ``image``)."""
    from ..utils.image import load_image

    raw = r.get("images")
    if raw is None and r.get("image") is not None:
        raw = [r["image"]]
    out = []
    for im in raw or []:
        if isinstance(im, dict):
            im = im.get("bytes") or im.get("path")
        if isinstance(im, str) and os.path.exists(im):
            from PIL import Image

            out.append(Image.open(im).convert("RGB"))
        else:
            out.append(load_image(im))
    return out


def _load_records(path: str) -> list[dict]:
    if os.path.isdir(path):
        files = sorted(os.path.join(path, f) for f in os.listdir(path) if f.endswith((".jsonl", ".json", ".parquet")))
    else:
        files = [path]
    recs: list[dict] = []
    for fn in files:
        if fn.endswith(".jsonl"):
            with open(fn) as f:
                recs += [json.loads(l) for l in f if l.strip()]
        elif fn.endswith(".json"):
            with open(fn) as f:
                d = json.load(f)
            recs += d if isinstance(d, list) else [d]
        elif fn.endswith(".parquet"):
            import pyarrow.parquet as pq

            recs += pq.read_table(fn).to_pylist()
    return recs


class RecordDataset(Dataset):
    def __init__(self, records: list[dict], transform: Optional[Callable[[dict], dict]] = None):
        self.records, self.transform = records, transform

    def __len__(self):
        return len(self.records)

    def __getitem__(self, i):
        r = self.records[i]
        return self.transform(r) if self.transform else r


def get_custom_dataset(path: str, type: str = "rl", split: str = "train", tokenizer=None, max_length: Optional[int] = None,
                       **kwargs) -> Dataset:
    """Resolves a dataset by path / type. Built-ins: ``synthetic/arithmetic``,
    ``synthetic/random_tokens``; any local json/jsonl/parquet file or directory with
    gsm8k-style (``question``/``answer``) or chat (``messages``) or preference
    (``chosen``/``rejected``) records."""
    if path.startswith("synthetic/arithmetic"):
        return ArithmeticDataset(size=kwargs.get("size", 4096), seed=kwargs.get("seed", 1))
    if path.startswith("synthetic/random_tokens"):
        return RandomTokenDataset(kwargs.get("size", 4096), kwargs.get("prompt_len", 512), kwargs.get("vocab_size", 151936),
                                  seed=kwargs.get("seed", 1), median_len=kwargs.get("median_len", 1024),
                                  max_len=kwargs.get("max_len", 4096))
    if path.startswith("synthetic/countdown"):
        return CountdownDataset(size=kwargs.get("size", 4096), seed=kwargs.get("seed", 1), n_numbers=kwargs.get("n_numbers", 3),
                                tokenizer=tokenizer)
    if path.startswith("synthetic/count_shapes"):
        return CountShapesDataset(size=kwargs.get("size", 1024), seed=kwargs.get("seed", 1), image_size=kwargs.get("image_size", 112),
                                  image_token_id=kwargs.get("image_token_id", 1000),
                                  vision_start_token_id=kwargs.get("vision_start_token_id", 1002))
    if not os.path.exists(path):
        raise FileNotFoundError(f"dataset '{path}' not found locally (no network access to fetch it)")
    recs = _load_records(os.path.join(path, split) if os.path.isdir(os.path.join(path, split)) else path)

    def rl_transform(r):
        q = r.get("question") or r.get("prompt") or r.get("problem")
        out = dict(r)
        out["messages"] = r.get("messages") or [{"role": "user", "content": q}]
        if tokenizer is not None:
            out["input_ids"] = list(tokenizer.apply_chat_template(out["messages"], tokenize=True, add_generation_prompt=True))
        return out

    def sft_transform(r):
        q = r.get("question") or r.get("prompt") or ""
        a = r.get("answer") or r.get("response") or ""
        p_ids = tokenizer.encode(q)
        a_ids = tokenizer.encode(a) + [tokenizer.eos_token_id]
        ids = (p_ids + a_ids)[:max_length] if max_length else p_ids + a_ids
        mask = ([0] * len(p_ids) + [1] * len(a_ids))[: len(ids)]
        return dict(input_ids=ids, loss_mask=mask)

    def rw_transform(r):
        return dict(chosen_ids=tokenizer.encode(r["chosen"])[:max_length], rejected_ids=tokenizer.encode(r["rejected"])[:max_length])

    def vl_rl_transform(r):
        # geometry3k / clevr_count style: question text + pictures; the chat template gets one image slot per picture
        q = r.get("problem") or r.get("question") or r.get("prompt") or ""
        images = _record_images(r)
        content = [{"type": "image"} for _ in images] + [{"type": "text", "text": q.replace("<image>", "")}]
        out = {k: v for k, v in r.items() if k not in ("images", "image")}
        out["messages"] = [{"role": "user", "content": content}]
        out["images"] = images
        return out

    def torl_transform(r):
        # torl_data / verl-style records: ``prompt`` is a message list, the answer sits in ``reward_model.ground_truth``
        msgs = r.get("prompt") if isinstance(r.get("prompt"), list) else [{"role": "user", "content": str(r.get("prompt") or r.get("question") or "")}]
        rm = r.get("reward_model") or {}
        out = {k: v for k, v in r.items() if k not in ("prompt",)}
        out["messages"] = list(msgs)
        out["answer"] = rm.get("ground_truth", r.get("answer"))
        if tokenizer is not None:
            out["input_ids"] = list(tokenizer.apply_chat_template(out["messages"], tokenize=True, add_generation_prompt=True))
        return out

    # named sets of the reference keep their conventions: picture sets carry images, torl carries verl-style records
    if type == "rl" and any(n in path for n in ("clevr_count_70k", "geometry3k", "virl39k")):
        type = "vl_rl"
    elif type == "rl" and "torl" in path:
        type = "torl"
    tf = {"rl": rl_transform, "sft": sft_transform, "rw": rw_transform, "dpo": rw_transform, "vl_rl": vl_rl_transform,
          "torl": torl_transform}.get(type)
    ds = RecordDataset(recs, tf if (tokenizer is not None or type in ("rl", "vl_rl", "torl")) else None)
    if max_length and type == "rl" and tokenizer is not None:
        keep = [i for i in range(len(ds)) if len(ds[i]["input_ids"]) <= max_length]
        ds = RecordDataset([recs[i] for i in keep], tf)
    return ds
