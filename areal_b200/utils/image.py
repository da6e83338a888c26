"""Image helpers for vision-language rollouts: PIL <-> bytes / base64, and decoding of whatever
a request carries (PIL image, uint8 array, raw bytes, base64 string or ``data:`` URL).
Reference: ``areal/utils/image.py`` (``image2base64``, padding to a square canvas)."""
from __future__ import annotations

import base64
import io
from typing import Any, Sequence, Union

import numpy as np


def image_to_bytes(image, fmt: str = "PNG") -> bytes:
    buf = io.BytesIO()
    image.convert("RGB").save(buf, format=fmt)
    return buf.getvalue()


def image2base64(images: Union[Any, Sequence[Any]], fmt: str = "PNG") -> list[str]:
    """PIL image(s) -> base64 strings (one per image)."""
    if not isinstance(images, (list, tuple)):
        images = [images]
    return [base64.b64encode(image_to_bytes(im, fmt)).decode("ascii") for im in images]


def load_image(obj):
    """Anything a request may carry -> an RGB PIL image (arrays are passed through)."""
    from PIL import Image

    if isinstance(obj, np.ndarray):
        return obj
    if hasattr(obj, "convert"):
        return obj.convert("RGB")
    if isinstance(obj, str):
        if obj.startswith("data:"):
            obj = obj.split(",", 1)[1]
        obj = base64.b64decode(obj)
    if isinstance(obj, (bytes, bytearray)):
        return Image.open(io.BytesIO(obj)).convert("RGB")
    raise TypeError(f"cannot decode an image from {type(obj).__name__}")


def pad_to_square(image, fill=(127, 127, 127)):
    """Centres the picture on a square canvas of its longer side."""
    from PIL import Image

    w, h = image.size
    if w == h:
        return image
    side = max(w, h)
    canvas = Image.new("RGB", (side, side), fill)
    canvas.paste(image, ((side - w) // 2, (side - h) // 2))
    return canvas
