"""Tensor-parallel rollout replica on 2 gloo ranks: the leader takes requests, both ranks run
the engine in lock-step; outputs must equal a single-rank engine with the same weights. Also
covers a weight update from full tensors and pause / continue. Prints INFER_TP_OK per rank."""
import asyncio
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
os.environ["AREAL_FORCE_CPU"] = "1"

from areal_b200.api.cli_args import GenerationHyperparameters, InferenceEngineConfig, NativeInferConfig  # noqa: E402
from areal_b200.api.io_struct import ModelRequest, WeightUpdateMeta  # noqa: E402
from areal_b200.engine.infer_engine import NativeInferenceEngine  # noqa: E402
from areal_b200.models.config import preset  # noqa: E402
from areal_b200.models.decoder import build_model  # noqa: E402


def requests(vocab):
    g = torch.Generator().manual_seed(5)
    out = []
    for i in range(6):
        ids = torch.randint(3, vocab, (5 + 3 * i,), generator=g).tolist()
        gc = GenerationHyperparameters(max_new_tokens=6 + i, max_tokens=128, greedy=(i % 2 == 0), temperature=0.8, ignore_eos=True, seed=100 + i)
        out.append(ModelRequest(rid=f"r{i}", input_ids=ids, gconfig=gc))
    return out


async def run_all(eng, reqs):
    return await asyncio.gather(*[eng.agenerate(r) for r in reqs])


def main():
    dist.init_process_group("gloo")
    rank = dist.get_rank()
    mc = preset("tiny-qwen3")                     # 4 query heads, 2 kv heads: splits over 2 ranks
    eng = NativeInferenceEngine(InferenceEngineConfig(), NativeInferConfig(max_running_requests=4, context_length=128), model_config=mc,
                                tp_group=dist.new_group([0, 1]), tp_control_group=dist.new_group([0, 1]))   # the engine thread's own groups
    eng.initialize(device="cpu", seed=7, start_executor=False)
    assert eng.tp_size == 2 and eng.model_config.num_heads == 2 and eng.full_model_config.num_heads == 4
    results = {}
    if rank == 0:
        ref = NativeInferenceEngine(InferenceEngineConfig(), NativeInferConfig(max_running_requests=4, context_length=128), model_config=mc)
        ref.initialize(device="cpu", seed=7, start_executor=False)
        want = asyncio.run(run_all(ref, requests(mc.vocab_size)))
        got = asyncio.run(run_all(eng, requests(mc.vocab_size)))
        for w, g_ in zip(want, got):
            assert w.output_tokens == g_.output_tokens, (w.output_tokens, g_.output_tokens)
            assert max(abs(a - b) for a, b in zip(w.output_logprobs, g_.output_logprobs)) < 1e-4
        results["first"] = [g_.output_tokens for g_ in got]
    else:
        try:
            asyncio.run(eng.agenerate(requests(mc.vocab_size)[0]))
            raise AssertionError("a follower accepted a request")
        except RuntimeError:
            pass
    dist.barrier()
    # ---- weight update: every rank receives the FULL tensors and keeps its slice
    new = build_model(mc, dtype=torch.float32, device="cpu", seed=99)
    eng.pause_generation()
    eng.update_weights_from_tensors({n: p.detach() for n, p in new.named_parameters()}, WeightUpdateMeta(type="disk", version=4))
    eng.continue_generation()
    assert eng.get_version() == 4
    dist.barrier()
    if rank == 0:
        ref.update_weights_from_tensors({n: p.detach() for n, p in new.named_parameters()}, WeightUpdateMeta(type="disk", version=4))
        want = asyncio.run(run_all(ref, requests(mc.vocab_size)))
        got = asyncio.run(run_all(eng, requests(mc.vocab_size)))
        for w, g_ in zip(want, got):
            assert w.output_tokens == g_.output_tokens and set(g_.output_versions) == {4}
        assert [g_.output_tokens for g_ in got] != results["first"]
        ref.destroy()
    dist.barrier()
    eng.destroy()                                  # stop is exchanged: both loops leave together
    assert eng._thread is None
    print("INFER_TP_OK", flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
