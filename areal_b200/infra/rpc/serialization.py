"""JSON-safe serialization of RPC payloads: tensors and numpy arrays (base64 of the raw
bytes + dtype + shape), dataclasses (import path + fields), enums, bytes, tuples/sets and
nested containers. Plays the role of the pydantic ``Serialized*`` models of the reference
(``areal/infra/rpc/serialization.py``). Only classes importable from this package (or
builtins / torch / numpy) are re-instantiated on load."""
from __future__ import annotations

import base64
import dataclasses
import enum
import importlib
from typing import Any

import numpy as np
import torch

_T = "__type__"
_ALLOWED_PREFIXES = ("areal_b200.", "tests.", "builtins")


def _cls_path(obj_or_cls) -> str:
    c = obj_or_cls if isinstance(obj_or_cls, type) else type(obj_or_cls)
    return f"{c.__module__}:{c.__qualname__}"


def _load_cls(path: str):
    mod, _, qual = path.partition(":")
    if not mod.startswith(_ALLOWED_PREFIXES):
        raise ValueError(f"refusing to load class from module '{mod}'")
    obj = importlib.import_module(mod)
    for part in qual.split("."):
        obj = getattr(obj, part)
    return obj


def serialize_value(v: Any) -> Any:
    if v is None or isinstance(v, (bool, int, float, str)):
        return v
    if torch.is_tensor(v):
        t = v.detach().cpu().contiguous()
        if t.dtype == torch.bfloat16:
            raw, dt = t.view(torch.int16).numpy().tobytes(), "bfloat16"
        else:
            raw, dt = t.numpy().tobytes(), str(t.dtype).replace("torch.", "")
        return {_T: "tensor", "dtype": dt, "shape": list(t.shape), "data": base64.b64encode(raw).decode()}
    if isinstance(v, np.ndarray):
        return {_T: "ndarray", "dtype": str(v.dtype), "shape": list(v.shape), "data": base64.b64encode(np.ascontiguousarray(v).tobytes()).decode()}
    if isinstance(v, np.generic):
        return v.item()
    if isinstance(v, bytes):
        return {_T: "bytes", "data": base64.b64encode(v).decode()}
    if isinstance(v, enum.Enum):
        return {_T: "enum", "cls": _cls_path(v), "name": v.name}
    if dataclasses.is_dataclass(v) and not isinstance(v, type):
        return {_T: "dataclass", "cls": _cls_path(v),
                "fields": {f.name: serialize_value(getattr(v, f.name)) for f in dataclasses.fields(v)}}
    if isinstance(v, dict):
        if all(isinstance(k, str) for k in v) and _T not in v:
            return {k: serialize_value(x) for k, x in v.items()}
        return {_T: "dict", "items": [[serialize_value(k), serialize_value(x)] for k, x in v.items()]}
    if isinstance(v, tuple):
        return {_T: "tuple", "items": [serialize_value(x) for x in v]}
    if isinstance(v, (set, frozenset)):
        return {_T: "set", "items": [serialize_value(x) for x in v]}
    if isinstance(v, list):
        return [serialize_value(x) for x in v]
    if isinstance(v, type):
        return {_T: "class", "cls": _cls_path(v)}
    raise TypeError(f"cannot serialize object of type {type(v).__name__}")


def deserialize_value(v: Any) -> Any:
    if isinstance(v, list):
        return [deserialize_value(x) for x in v]
    if not isinstance(v, dict):
        return v
    t = v.get(_T)
    if t is None:
        return {k: deserialize_value(x) for k, x in v.items()}
    if t == "tensor":
        raw = base64.b64decode(v["data"])
        if v["dtype"] == "bfloat16":
            return torch.frombuffer(bytearray(raw), dtype=torch.int16).view(torch.bfloat16).reshape(v["shape"]).clone()
        dt = getattr(torch, v["dtype"])
        if not raw:
            return torch.empty(v["shape"], dtype=dt)
        return torch.frombuffer(bytearray(raw), dtype=dt).reshape(v["shape"]).clone()
    if t == "ndarray":
        return np.frombuffer(base64.b64decode(v["data"]), dtype=np.dtype(v["dtype"])).reshape(v["shape"]).copy()
    if t == "bytes":
        return base64.b64decode(v["data"])
    if t == "enum":
        return _load_cls(v["cls"])[v["name"]]
    if t == "dataclass":
        cls = _load_cls(v["cls"])
        fields = {k: deserialize_value(x) for k, x in v["fields"].items()}
        init = {f.name for f in dataclasses.fields(cls) if f.init}
        obj = cls(**{k: x for k, x in fields.items() if k in init})
        for k, x in fields.items():
            if k not in init:
                object.__setattr__(obj, k, x)
        return obj
    if t == "dict":
        return {deserialize_value(k) if not isinstance(k, list) else tuple(deserialize_value(k)): deserialize_value(x)
                for k, x in v["items"]}
    if t == "tuple":
        return tuple(deserialize_value(x) for x in v["items"])
    if t == "set":
        return set(deserialize_value(x) for x in v["items"])
    if t == "class":
        return _load_cls(v["cls"])
    raise ValueError(f"unknown serialized type tag '{t}'")
