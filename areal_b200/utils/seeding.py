"""Deterministic seeding (reference: ``areal/utils/seeding.py``): per-component seeds derived
from a base seed and a key, plus per-request seeds for deterministic sampling."""
from __future__ import annotations

import hashlib
import random

import numpy as np
import torch

_BASE_SEED = None
_KEY = None


def _derive(base: int, key: str) -> int:
    h = hashlib.sha256(f"{base}:{key}".encode()).digest()
    return int.from_bytes(h[:4], "little")


def set_random_seed(base_seed: int, key: str = "") -> int:
    global _BASE_SEED, _KEY
    _BASE_SEED, _KEY = base_seed, key
    seed = _derive(base_seed, key) if key else base_seed
    random.seed(seed)
    np.random.seed(seed % (2 ** 32))
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)
    return seed


def get_seed() -> int:
    if _BASE_SEED is None:
        raise RuntimeError("set_random_seed has not been called")
    return _derive(_BASE_SEED, _KEY) if _KEY else _BASE_SEED


def derive_deterministic_seed(identity: str, request_index: int, base_seed: int | None = None) -> int:
    base = _BASE_SEED if base_seed is None else base_seed
    return _derive(base or 0, f"{identity}#{request_index}") & 0x7FFFFFFF
