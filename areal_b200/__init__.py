"""areal_b200: asynchronous RL training of language models, written for B200 GPUs.

The names a training script usually needs are reachable from here and resolved on first use, so ``import areal_b200``
stays cheap (no torch, no CUDA library load). Reference: the lazy exports of ``areal/__init__.py:7-43``.
"""
from .version import __version__, version_info  # noqa: F401

_LAZY = {
    "PPOTrainer": ".trainer.rl_trainer", "SFTTrainer": ".trainer.sft_trainer", "RWTrainer": ".trainer.rw_trainer", "DPOTrainer": ".trainer.dpo_trainer",
    "TrainController": ".infra.controller.train_controller", "RolloutController": ".infra.controller.rollout_controller",
    "WorkflowExecutor": ".rollout.executor", "StalenessManager": ".rollout.staleness", "current_platform": ".infra.platforms",
    "workflow_context": ".rollout",
}

__all__ = ["__version__", "version_info", *_LAZY]


def __getattr__(name: str):
    mod = _LAZY.get(name)
    if mod is None:
        raise AttributeError(f"module 'areal_b200' has no attribute '{name}'")
    import importlib

    m = importlib.import_module(mod, __name__)
    val = importlib.import_module(mod + ".workflow_context", __name__) if name == "workflow_context" else getattr(m, name)
    globals()[name] = val
    return val


def __dir__():
    return sorted(__all__)
