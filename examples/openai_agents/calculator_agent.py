"""Tool-using agent written against the OpenAI *Responses* interface (``client.responses.create`` with
function tools and ``function_call_output`` items), trained with GRPO. The agent loop is what an
application using the OpenAI SDK would write; during training ``client`` is the in-process
recorder, in deployment it can be the stock SDK pointed at the proxy server.

Reference behaviour: ``examples/openai_agents/`` of the reference project (agents-SDK style loops
trained through the OpenAI-compatible client)."""
import ast
import json
import operator
import re
import sys

from areal_b200.api.cli_args import GRPOConfig, load_expr_config
from areal_b200.api.workflow_api import AgentWorkflow
from areal_b200.dataset import ArithmeticDataset
from areal_b200.rollout.workflows.agent import AgentRolloutAdapter
from areal_b200.rollout.workflows.rlvr import GroupedRolloutWorkflow
from areal_b200.trainer import PPOTrainer
from areal_b200.utils.hf_utils import load_hf_tokenizer

CALC_TOOL = {"type": "function", "name": "calculate", "description": "Evaluate an arithmetic expression.",
             "parameters": {"type": "object", "properties": {"expression": {"type": "string"}}, "required": ["expression"]}}
_OPS = {ast.Add: operator.add, ast.Sub: operator.sub, ast.Mult: operator.mul, ast.Div: operator.truediv, ast.USub: operator.neg}


def safe_eval(expr: str) -> float:
    """Arithmetic only: numbers, + - * /, parentheses."""
    def ev(n):
        if isinstance(n, ast.Constant) and isinstance(n.value, (int, float)):
            return n.value
        if isinstance(n, ast.BinOp) and type(n.op) in _OPS:
            return _OPS[type(n.op)](ev(n.left), ev(n.right))
        if isinstance(n, ast.UnaryOp) and type(n.op) in _OPS:
            return _OPS[type(n.op)](ev(n.operand))
        raise ValueError("unsupported expression")
    return ev(ast.parse(expr, mode="eval").body)


class CalculatorAgent(AgentWorkflow):
    def __init__(self, max_turns: int = 3, max_tokens: int = 128):
        self.max_turns, self.max_tokens = max_turns, max_tokens

    async def run(self, data, client):
        items = [{"role": "user", "content": data["question"]}]
        text = ""
        for _ in range(self.max_turns):
            r = await client.responses.create(input=items, instructions="Use the calculator when it helps. End with 'Answer: <number>'.",
                                              tools=[CALC_TOOL], max_output_tokens=self.max_tokens)
            text = r.output_text
            calls = [o for o in r.output if o.get("type") == "function_call"]
            if not calls:
                break
            items.append({"role": "assistant", "content": text})
            for c in calls:
                try:
                    val = str(safe_eval(json.loads(c["arguments"]).get("expression", "")))
                except Exception as e:  # the model sees its own mistake
                    val = f"error: {e}"
                items.append({"type": "function_call_output", "call_id": c["call_id"], "output": val})
        m = re.search(r"Answer:\s*(-?\d+(?:\.\d+)?)", text or "")
        return 1.0 if m and abs(float(m.group(1)) - float(data["answer"])) < 1e-6 else 0.0


def main(argv):
    config, _ = load_expr_config(argv, GRPOConfig)
    tok = load_hf_tokenizer(config.tokenizer_path)
    data = [{"question": "What is " + d["prompt"].strip().rstrip("=") + "?", "answer": d["answer"]} for d in ArithmeticDataset(size=512)]
    one = AgentRolloutAdapter(CalculatorAgent(), tokenizer=tok, gconfig=config.gconfig, export_style="individual", turn_discount=0.9)
    with PPOTrainer(config, data, tokenizer=tok) as trainer:
        trainer.train(workflow=GroupedRolloutWorkflow.from_gconfig(one, config.gconfig))


if __name__ == "__main__":
    main(sys.argv[1:])
