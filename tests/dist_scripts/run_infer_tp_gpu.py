"""Tensor-parallel rollout replica on 2 GPUs: the fused path (partial sums exchanged from the GEMM
epilogue over peer memory, reduced inside the norm kernel, decode steps graph captured) against the
library path (NCCL all-reduce, eager decode steps). Greedy tokens must be identical, log-probs
equal to rounding, and the decode time per step of both paths is printed (device-timed on the
leader around the whole generation, host work included: this is what a rollout sees).

    python -m torch.distributed.run --nproc-per-node 2 tests/dist_scripts/run_infer_tp_gpu.py [--model qwen3-8b --batch 64 --new 64]

Prints ``INFER_TP_GPU_OK`` per rank and one JSON line with the timings on the leader.
"""
import argparse
import asyncio
import json
import os
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from areal_b200.api.cli_args import GenerationHyperparameters, InferenceEngineConfig, NativeInferConfig  # noqa: E402
from areal_b200.api.io_struct import ModelRequest  # noqa: E402
from areal_b200.engine.infer_engine import NativeInferenceEngine  # noqa: E402
from areal_b200.models.config import preset  # noqa: E402
from areal_b200.ops import lib as oplib  # noqa: E402


def requests(vocab, batch, prompt_len, new):
    g = torch.Generator().manual_seed(5)
    out = []
    for i in range(batch):
        ids = torch.randint(3, vocab, (prompt_len + (i % 7),), generator=g).tolist()
        gc = GenerationHyperparameters(max_new_tokens=new, max_tokens=prompt_len + new + 16, greedy=True, ignore_eos=True, seed=100 + i)
        out.append(ModelRequest(rid=f"r{i}", input_ids=ids, gconfig=gc))
    return out


async def run_all(eng, reqs):
    return await asyncio.gather(*[eng.agenerate(r) for r in reqs])


def run_engine(fused: bool, mc, args, tp_group, ctl_group, main_group, rank):
    os.environ["AREAL_TP_FUSED"] = "1" if fused else "0"
    ic = NativeInferConfig(max_running_requests=max(8, args.batch), context_length=args.prompt + args.new + 64, page_size=64,
                           max_prefill_tokens=8192, mem_fraction_static=0.5)
    eng = NativeInferenceEngine(InferenceEngineConfig(), ic, model_config=mc, tp_group=tp_group, tp_control_group=ctl_group)
    eng.initialize(device=torch.device("cuda", torch.cuda.current_device()), seed=7, start_executor=False)
    assert (eng.tp_exchange is not None) == fused and eng.icfg.use_cuda_graph == fused
    out, secs = None, 0.0
    if rank == 0:
        asyncio.run(run_all(eng, requests(mc.vocab_size, args.batch, args.prompt, 8)))      # warm-up: graphs captured
        torch.cuda.synchronize()
        steps0 = eng.stats["decode_steps"]
        t0 = time.perf_counter()
        out = asyncio.run(run_all(eng, requests(mc.vocab_size, args.batch, args.prompt, args.new)))
        torch.cuda.synchronize()
        secs = time.perf_counter() - t0
        steps = eng.stats["decode_steps"] - steps0
        secs = secs / max(1, steps)
    dist.barrier(group=main_group)       # never the engine thread's control group: that thread uses it all the time
    eng.destroy()
    err = oplib.kernel_error()
    assert err == 0, f"kernel error word = {err}"
    torch.cuda.empty_cache()
    return out, secs


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="tiny-qwen3")
    ap.add_argument("--batch", type=int, default=6)
    ap.add_argument("--prompt", type=int, default=40)
    ap.add_argument("--new", type=int, default=24)
    args = ap.parse_args()
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    dist.init_process_group("nccl")
    rank = dist.get_rank()
    mc = preset(args.model)
    import faulthandler

    faulthandler.dump_traceback_later(420, exit=True)      # a stuck run prints its stacks and leaves
    tp_group = dist.new_group([0, 1])
    ctl_group = dist.new_group([0, 1], backend="gloo")      # the engine threads' control exchange
    main_group = dist.new_group([0, 1], backend="gloo")     # this script's own barriers
    want, ms_lib = run_engine(False, mc, args, tp_group, ctl_group, main_group, rank)
    got, ms_fused = run_engine(True, mc, args, tp_group, ctl_group, main_group, rank)
    if rank == 0:
        print(json.dumps({"kernel": "tp2_decode_step (engine, host included)", "model": args.model, "batch": args.batch,
                          "prompt": args.prompt, "new": args.new, "ms_per_step_nccl_eager": round(ms_lib * 1e3, 3),
                          "ms_per_step_fused_graph": round(ms_fused * 1e3, 3),
                          "speedup": round(ms_lib / max(ms_fused, 1e-9), 3)}), flush=True)
        same = sum(w.output_tokens == g_.output_tokens for w, g_ in zip(want, got))
        print(f"identical greedy sequences: {same} of {len(want)}", flush=True)
        for w, g_ in zip(want, got):
            assert w.output_tokens == g_.output_tokens, (w.output_tokens[:8], g_.output_tokens[:8])
            assert max(abs(a - b) for a, b in zip(w.output_logprobs, g_.output_logprobs)) < 2e-2
    print("INFER_TP_GPU_OK", flush=True)
    dist.barrier(group=main_group)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
