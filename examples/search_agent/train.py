"""Search agent trained with GRPO: the policy may call a ``search`` tool several times before it
answers. The retrieval backend here is an in-memory corpus scored by token overlap, so the
example runs without any service; point ``LocalSearch`` at a real retriever by replacing
``LocalSearch.query``. The agent is plain OpenAI-style code (``tools=`` on chat completions, tool
messages appended to the conversation); every model call is recorded with its token ids,
log-probs and weight versions, and the final reward is shared with earlier turns
(``turn_discount``).

Reference behaviour: ``examples/search_agent/`` of the reference project (multi-turn retrieval agent
with tool calls and a final-answer reward)."""
import json
import re
import sys

from areal_b200.api.cli_args import GRPOConfig, load_expr_config
from areal_b200.api.workflow_api import AgentWorkflow
from areal_b200.rollout.workflows.agent import AgentRolloutAdapter
from areal_b200.rollout.workflows.rlvr import GroupedRolloutWorkflow
from areal_b200.trainer import PPOTrainer
from areal_b200.utils.hf_utils import load_hf_tokenizer

CORPUS = [
    "The Danube flows through ten countries and empties into the Black Sea.",
    "Mount Kosciuszko is the highest mountain of mainland Australia at 2228 metres.",
    "The Treaty of Tordesillas was signed in 1494 by Spain and Portugal.",
    "Tungsten has the highest melting point of all metals, 3422 degrees Celsius.",
    "The Rosetta Stone was found in 1799 and is kept in the British Museum.",
    "Lake Baikal is the deepest lake on Earth with a depth of 1642 metres.",
]
QUESTIONS = [
    ("Into which sea does the Danube empty?", "black sea"),
    ("How high is Mount Kosciuszko in metres?", "2228"),
    ("In which year was the Treaty of Tordesillas signed?", "1494"),
    ("Which metal has the highest melting point?", "tungsten"),
    ("Where is the Rosetta Stone kept?", "british museum"),
    ("How deep is Lake Baikal in metres?", "1642"),
]
SEARCH_TOOL = {"type": "function", "function": {
    "name": "search", "description": "Look up passages that match a query.",
    "parameters": {"type": "object", "properties": {"query": {"type": "string"}}, "required": ["query"]}}}
SYSTEM = ("Answer the question. You may call the search tool first. Put the final answer inside <answer></answer>.")


class LocalSearch:
    def __init__(self, passages=CORPUS, top_k: int = 2):
        self.passages, self.top_k = list(passages), top_k
        self._bags = [set(re.findall(r"\w+", p.lower())) for p in self.passages]

    def query(self, text: str) -> list[str]:
        q = set(re.findall(r"\w+", text.lower()))
        scored = sorted(((len(q & b), i) for i, b in enumerate(self._bags)), reverse=True)
        return [self.passages[i] for s, i in scored[: self.top_k] if s > 0]


def answer_reward(text: str, gold: str) -> float:
    m = re.search(r"<answer>(.*?)</answer>", text or "", re.S | re.I)
    if not m:
        return 0.0
    return 1.0 if gold.lower() in m.group(1).lower() else 0.1          # well-formed but wrong still beats no answer


class SearchAgent(AgentWorkflow):
    def __init__(self, search: LocalSearch = None, max_turns: int = 3, max_tokens: int = 256):
        self.search, self.max_turns, self.max_tokens = search or LocalSearch(), max_turns, max_tokens

    async def run(self, data, client):
        msgs = [{"role": "system", "content": SYSTEM}, {"role": "user", "content": data["question"]}]
        text = ""
        for _ in range(self.max_turns):
            out = await client.chat.completions.create(messages=msgs, tools=[SEARCH_TOOL], max_completion_tokens=self.max_tokens)
            m = out.choices[0].message
            text = m.content or ""
            if not m.tool_calls:
                break
            msgs.append({"role": "assistant", "content": text, "tool_calls": [t.to_dict() if hasattr(t, "to_dict") else t for t in m.tool_calls]})
            for call in m.tool_calls:
                try:
                    q = json.loads(call.function.arguments).get("query", "")
                except (ValueError, AttributeError):
                    q = ""
                msgs.append({"role": "tool", "tool_call_id": call.id, "content": "\n".join(self.search.query(q)) or "no result"})
        return answer_reward(text, data["answer"])


def dataset(repeat: int = 32):
    return [{"question": q, "answer": a} for _ in range(repeat) for q, a in QUESTIONS]


def main(argv):
    config, _ = load_expr_config(argv, GRPOConfig)
    tok = load_hf_tokenizer(config.tokenizer_path)
    one = AgentRolloutAdapter(SearchAgent(), tokenizer=tok, gconfig=config.gconfig, export_style="individual", turn_discount=0.9)
    with PPOTrainer(config, dataset(), tokenizer=tok) as trainer:
        trainer.train(workflow=GroupedRolloutWorkflow.from_gconfig(one, config.gconfig))


if __name__ == "__main__":
    main(sys.argv[1:])
