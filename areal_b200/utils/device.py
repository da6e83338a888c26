"""Device memory logging helpers (reference: ``areal/utils/device.py``)."""
from __future__ import annotations

import torch

from . import logging as alog

logger = alog.getLogger("device")


def memory_stats(device=None) -> dict[str, float]:
    if not torch.cuda.is_available():
        return {"allocated_gb": 0.0, "reserved_gb": 0.0, "free_gb": 0.0, "total_gb": 0.0}
    free, total = torch.cuda.mem_get_info(device)
    return {"allocated_gb": torch.cuda.memory_allocated(device) / 2 ** 30, "reserved_gb": torch.cuda.memory_reserved(device) / 2 ** 30,
            "free_gb": free / 2 ** 30, "total_gb": total / 2 ** 30}


def log_gpu_stats(head: str, rank: int | None = None, device=None) -> dict[str, float]:
    s = memory_stats(device)
    logger.info("%s%s: allocated %.2f GB, reserved %.2f GB, free %.2f of %.2f GB", head, "" if rank is None else f" [rank {rank}]",
                s["allocated_gb"], s["reserved_gb"], s["free_gb"], s["total_gb"])
    return s


def clear_memory():
    import gc

    gc.collect()
    if torch.cuda.is_available():
        torch.cuda.empty_cache()
