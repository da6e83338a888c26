from .rollout_callback import RolloutCallback
from .rollout_controller import RolloutController
from .train_controller import TrainController, merge_results, split_batch

__all__ = ["TrainController", "RolloutController", "RolloutCallback", "split_batch", "merge_results"]
