"""Trainers (lazy exports so that importing one does not pull in the others)."""


def __getattr__(name):
    if name in ("PPOTrainer", "GRPOTrainer"):
        from .rl_trainer import PPOTrainer

        return PPOTrainer
    if name == "SFTTrainer":
        from .sft_trainer import SFTTrainer

        return SFTTrainer
    if name == "RWTrainer":
        from .rw_trainer import RWTrainer

        return RWTrainer
    if name == "DPOTrainer":
        from .dpo_trainer import DPOTrainer

        return DPOTrainer
    raise AttributeError(name)


__all__ = ["PPOTrainer", "GRPOTrainer", "SFTTrainer", "RWTrainer", "DPOTrainer"]
