"""Tokenizer / processor / config loading helpers (reference: ``areal/utils/hf_utils.py``)."""
from __future__ import annotations

import functools
import json
import os
from typing import Any, Optional


@functools.lru_cache(maxsize=8)
def load_hf_tokenizer(path: str, fast_tokenizer: bool = True, padding_side: Optional[str] = None) -> Any:
    """``AutoTokenizer`` for a local directory; a directory written by ``CharTokenizer`` loads
    as that. The pad token defaults to eos when unset."""
    if os.path.isfile(os.path.join(path, "char_tokenizer.json")):
        from ..dataset import CharTokenizer

        return CharTokenizer()
    import transformers

    kw: dict[str, Any] = {"use_fast": fast_tokenizer, "trust_remote_code": True}
    if padding_side is not None:
        kw["padding_side"] = padding_side
    tok = transformers.AutoTokenizer.from_pretrained(path, **kw)
    if tok.pad_token_id is None:
        tok.pad_token_id = tok.eos_token_id
    return tok


@functools.lru_cache(maxsize=8)
def load_hf_processor_and_tokenizer(path: str, fast_tokenizer: bool = True, padding_side: Optional[str] = None):
    import transformers

    tok = load_hf_tokenizer(path, fast_tokenizer, padding_side)
    try:
        proc = transformers.AutoProcessor.from_pretrained(path, trust_remote_code=True, use_fast=True)
    except Exception:
        proc = None
    return proc, tok


def load_hf_config_dict(path: str) -> dict:
    with open(os.path.join(path, "config.json")) as f:
        return json.load(f)


def is_valid_vision_model(model_type: str) -> bool:
    return model_type in ("qwen2_vl", "qwen2_5_vl", "qwen3_vl", "gemma3")
