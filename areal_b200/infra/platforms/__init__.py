"""Device platform abstraction (reference: ``areal/infra/platforms/*``): communication backend
name, device control, memory queries and NUMA affinity for the CUDA (B200) and CPU platforms.
This framework targets sm_100a only; the CPU platform exists for tests and control processes."""
from __future__ import annotations

import os
from typing import Optional

import torch


class Platform:
    device_type = "cpu"
    communication_backend = "gloo"
    device_control_env_var = ""

    def device_count(self) -> int:
        return 0

    def current_device(self):
        return torch.device("cpu")

    def set_device(self, index: int) -> None:
        pass

    def synchronize(self) -> None:
        pass

    def mem_info(self) -> tuple[int, int]:
        import psutil

        vm = psutil.virtual_memory()
        return vm.available, vm.total

    def set_numa_affinity(self, index: int) -> None:
        pass

    def is_blackwell(self) -> bool:
        return False


class CpuPlatform(Platform):
    pass


class CudaPlatform(Platform):
    device_type = "cuda"
    communication_backend = "nccl"
    device_control_env_var = "CUDA_VISIBLE_DEVICES"

    def device_count(self) -> int:
        return torch.cuda.device_count()

    def current_device(self):
        return torch.device("cuda", torch.cuda.current_device())

    def set_device(self, index: int) -> None:
        torch.cuda.set_device(index)

    def synchronize(self) -> None:
        torch.cuda.synchronize()

    def mem_info(self) -> tuple[int, int]:
        return torch.cuda.mem_get_info()

    def is_blackwell(self) -> bool:
        return torch.cuda.get_device_capability()[0] >= 10

    def set_numa_affinity(self, index: int) -> None:
        """Pins the process to the CPUs NVML reports as local to the GPU (read-only NVML use)."""
        try:
            import pynvml

            pynvml.nvmlInit()
            h = pynvml.nvmlDeviceGetHandleByIndex(index)
            n = (os.cpu_count() or 64 + 63) // 64 + 1
            mask = pynvml.nvmlDeviceGetCpuAffinity(h, n)
            cpus = [i * 64 + b for i, w in enumerate(mask) for b in range(64) if (w >> b) & 1]
            if cpus:
                os.sched_setaffinity(0, cpus)
        except Exception:
            pass


def _detect() -> Platform:
    if torch.cuda.is_available() and os.environ.get("AREAL_FORCE_CPU", "0") != "1":
        return CudaPlatform()
    return CpuPlatform()


current_platform: Platform = _detect()
