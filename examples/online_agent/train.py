"""Online training: the trainer serves the current policy on an OpenAI-compatible proxy and learns from whatever
outside users do with it. Nothing here generates prompts; an episode is one session that a user (a chat loop, an agent
framework, a product backend) opened, talked through, scored and closed:

    python examples/online_agent/train.py --config examples/online_agent/config.yaml        # prints the proxy URL
    python examples/online_agent/start_session.py --url http://127.0.0.1:8090 --admin-key <key>   # -> sk-sess-...
    python examples/online_agent/chat.py --url http://127.0.0.1:8090 --key sk-sess-...            # talk to the policy
    python examples/online_agent/set_reward.py --url http://127.0.0.1:8090 --key sk-sess-... --reward 1.0

Every model call of the session is recorded with token ids, log-probs and weight versions; ``set_reward.py`` scores the
last turn (earlier turns get ``turn_discount`` times that) and closes the session, which hands it to the trainer. With
``gconfig.n_samples: 1`` and no reward / advantage normalisation every single outcome keeps its signal.

Reference behaviour: ``examples/hermes`` and ``examples/openclaw`` of the reference project (session scripts around an
externally driven agent) and the online mode of its proxy workflow.
"""
import os
import secrets
import sys

from areal_b200.api.cli_args import GRPOConfig, load_expr_config
from areal_b200.openai.proxy import OpenAIProxyServer
from areal_b200.rollout.workflows.online import OnlineSessionWorkflow
from areal_b200.trainer import PPOTrainer
from areal_b200.utils.hf_utils import load_hf_tokenizer


def placeholders(n: int = 1 << 16):
    """The data loader only paces the loop: one placeholder per awaited session."""
    return [{"episode": i} for i in range(n)]


def main(argv):
    config, _ = load_expr_config(argv, GRPOConfig)
    tok = load_hf_tokenizer(config.tokenizer_path)
    admin = os.environ.get("AREAL_ADMIN_KEY") or "adm-" + secrets.token_hex(8)
    with PPOTrainer(config, placeholders(), tokenizer=tok) as trainer:
        proxy = OpenAIProxyServer(trainer.rollout, tok, config.gconfig, host=os.environ.get("AREAL_PROXY_HOST", "127.0.0.1"),
                                  port=int(os.environ.get("AREAL_PROXY_PORT", "8090")), admin_key=admin).start()
        print(f"proxy: {proxy.base_url[:-3]}   admin key: {admin}", flush=True)
        try:
            trainer.train(workflow=OnlineSessionWorkflow(proxy, turn_discount=0.9, timeout=float(os.environ.get("AREAL_SESSION_TIMEOUT", "3600"))))
        finally:
            proxy.stop()


if __name__ == "__main__":
    main(sys.argv[1:])
