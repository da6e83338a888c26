"""Vision-language GRPO on a procedural counting task (no external files; CPU or one GPU):
each prompt is a picture with k squares, the reward is 1 when the first generated token names k.
The tiny Qwen2-VL-style model (image tower + decoder) is trained end to end: the tower
receives gradients through the image features spliced into the prompt."""
import sys

from areal_b200.api.cli_args import GRPOConfig, load_expr_config
from areal_b200.dataset import count_shapes_reward_fn, get_custom_dataset
from areal_b200.models.config import preset
from areal_b200.rollout.workflows.vision_rlvr import VisionRLVRWorkflow
from areal_b200.trainer import PPOTrainer


def main(argv):
    config, _ = load_expr_config(argv, GRPOConfig)
    mc = preset("tiny-qwen2-vl")
    ds = get_custom_dataset(config.train_dataset.path, size=256, image_size=56, image_token_id=mc.image_token_id,
                            vision_start_token_id=mc.vision_start_token_id)
    wf = VisionRLVRWorkflow(count_shapes_reward_fn, config.gconfig, vision_config=mc.vision_config(), image_token_id=mc.image_token_id,
                            reward_in_process=True, min_pixels=28 * 28, max_pixels=28 * 28 * 4)
    with PPOTrainer(config, ds) as trainer:
        hist = trainer.train(workflow=wf)
    r = [h["ppo_actor/task_reward/avg"] for h in hist]
    print(f"reward: first 3 steps {sum(r[:3]) / 3:.3f} -> last 3 steps {sum(r[-3:]) / 3:.3f}")


if __name__ == "__main__":
    main(sys.argv[1:])
