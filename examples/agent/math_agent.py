"""An agent written against the OpenAI chat-completions interface, trained with GRPO.

The agent only sees ``client.chat.completions.create``; token ids, logprobs and weight
versions are captured by the client, the returned float is the reward of the last call and
is propagated to earlier calls with ``turn_discount``."""
import sys

from areal_b200.api.cli_args import GRPOConfig, load_expr_config
from areal_b200.api.workflow_api import AgentWorkflow
from areal_b200.dataset import get_custom_dataset
from areal_b200.reward import gsm8k_reward_fn
from areal_b200.rollout.workflows.agent import AgentRolloutAdapter
from areal_b200.rollout.workflows.rlvr import GroupedRolloutWorkflow
from areal_b200.trainer import PPOTrainer
from areal_b200.utils.hf_utils import load_hf_tokenizer


class ReflectingMathAgent(AgentWorkflow):
    """Answers, then is asked once to double-check its own answer."""

    def __init__(self, max_tokens: int = 512):
        self.max_tokens = max_tokens

    async def run(self, data, client):
        msgs = list(data["messages"])
        first = await client.chat.completions.create(messages=msgs, max_completion_tokens=self.max_tokens)
        msgs += [{"role": "assistant", "content": first.choices[0].message.content},
                 {"role": "user", "content": "Check your work and give the final answer in \\boxed{}."}]
        second = await client.chat.completions.create(messages=msgs, max_completion_tokens=self.max_tokens)
        return gsm8k_reward_fn(None, second.choices[0].message.content, None, None, answer=data.get("answer"))


def main(argv):
    config, _ = load_expr_config(argv, GRPOConfig)
    tok = load_hf_tokenizer(config.tokenizer_path)
    train = get_custom_dataset(config.train_dataset.path, type="rl", split="train", tokenizer=tok, max_length=config.train_dataset.max_length)
    one = AgentRolloutAdapter(ReflectingMathAgent(), tokenizer=tok, gconfig=config.gconfig, export_style="individual", turn_discount=0.9)
    with PPOTrainer(config, train, tokenizer=tok) as trainer:
        trainer.train(workflow=GroupedRolloutWorkflow.from_gconfig(one, config.gconfig))


if __name__ == "__main__":
    main(sys.argv[1:])
