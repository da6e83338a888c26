"""Datasets keyed by ``(path, type)`` (reference: ``areal/dataset/__init__.py``
``get_custom_dataset``): synthetic arithmetic / random-token sets for offline experiments,
and loaders for gsm8k-style JSON/parquet files on disk."""
from __future__ import annotations

import json
import os
import random
from typing import Any, Callable, Optional

import torch
from torch.utils.data import Dataset


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
    """Uniform-random prompt token ids with a per-sample response budget drawn from a
    log-normal (forced-length benchmarks); rewards are Bernoulli from the seed."""

    def __init__(self, size: int, prompt_len: int, vocab_size: int, seed: int = 1, median_len: int = 1024,
                 max_len: int = 4096, sigma: float = 0.6, min_len: int = 16):
        g = torch.Generator().manual_seed(seed)
        self.prompts = torch.randint(0, vocab_size, (size, prompt_len), generator=g, dtype=torch.int32)
        z = torch.randn(size, generator=g)
        lens = (median_len * torch.exp(sigma * z)).clamp(min_len, max_len).long()
        self.lens = lens.tolist()
        self.rewards = (torch.rand(size, generator=g) < 0.5).float().tolist()

    def __len__(self):
        return self.prompts.shape[0]

    def __getitem__(self, i):
        return dict(input_ids=self.prompts[i].tolist(), max_new_tokens=self.lens[i], reward=self.rewards[i], idx=i)


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

    tf = {"rl": rl_transform, "sft": sft_transform, "rw": rw_transform, "dpo": rw_transform}.get(type)
    ds = RecordDataset(recs, tf if (tokenizer is not None or type == "rl") else None)
    if max_length and type == "rl" and tokenizer is not None:
        keep = [i for i in range(len(ds)) if len(ds[i]["input_ids"]) <= max_length]
        ds = RecordDataset([recs[i] for i in keep], tf)
    return ds
