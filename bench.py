"""Headline benchmark: asynchronous GRPO trained tokens/s on the Qwen3-8B architecture.

``python bench.py --gpus N --steps K --warmup W`` runs the flagship async-RL step on N GPUs
of one node (for N > 1 launch under ``python -m torch.distributed.run --nproc-per-node N``):

* N = 1: trainer and rollout engine share the GPU (colocated, concurrent);
* N >= 2: ranks [0, N/2) train (ZeRO over all trainers, Ulysses sequence parallel in groups of up
  to 4), ranks [N/2, N) generate (tensor-parallel replicas of 2 GPUs from N = 4 on), weights travel
  trainer -> rollout over NVLink after every step, re-sharded in flight.

The default workload is BASELINE.json's Qwen3-8B decoupled-PPO shape (``--preset baseline``) with
all lengths scaled by 0.25 so that the 45 steps of a driver run finish inside its time limit on
one GPU; ``--preset baseline`` runs the unscaled shape, ``--preset small`` the short-sequence
workload of earlier measurements.

Synthetic data (uniform-random prompt ids, forced log-normal response lengths, Bernoulli
rewards) and random-init weights, bf16 compute. After W warm-up steps exactly K steps are
timed on the device (CUDA events, barrier + synchronize on both sides, max over ranks); rank 0
prints one JSON line. ``--impl reference`` runs the reference implementation from
``baseline/_ref`` if it is installed, else reports why it is unavailable.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


PRESETS = {
    # BASELINE.json config 3 (Qwen3-8B decoupled PPO): 1,024-token prompts, log-normal responses with
    # median 4,096 capped at 16,384, groups of 16, 32k-token packed micro-batches
    "baseline": dict(prompt_len=1024, median_len=4096, max_len=16384, group_size=16, max_tokens_per_mb=32768, length_scale=1.0),
    # the same shape with every length scaled by --length-scale (default 0.25): what fits the 45 steps of a
    # driver run into its time limit on one GPU (see README "Benchmark workload")
    "driver": dict(prompt_len=1024, median_len=4096, max_len=16384, group_size=16, max_tokens_per_mb=32768, length_scale=0.25),
    # the short-sequence workload of earlier measurements (data-parallel trainers and rollout replicas)
    "small": dict(prompt_len=256, median_len=256, max_len=768, group_size=8, max_tokens_per_mb=0, length_scale=1.0,
                  sp=1, rollout_tp=1, staleness=2, prompts_per_gpu=4.0, prox_logp_method="reuse_train_logp"),
}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", type=str, default="native", choices=["native", "reference"])
    ap.add_argument("--model", type=str, default="qwen3-8b")
    ap.add_argument("--preset", type=str, default="driver", choices=sorted(PRESETS))
    ap.add_argument("--length-scale", type=float, default=None, help="scales prompt / median / cap lengths of the preset")
    ap.add_argument("--prompts-per-gpu", type=float, default=None,
                    help="prompts (groups) per optimizer step per GPU of the job: the global batch grows with N (weak scaling)")
    ap.add_argument("--group-size", type=int, default=None)
    ap.add_argument("--prompt-len", type=int, default=None)
    ap.add_argument("--median-len", type=int, default=None)
    ap.add_argument("--max-len", type=int, default=None)
    ap.add_argument("--max-tokens-per-mb", type=int, default=None, help="packed micro-batch size in tokens (0: from the memory policy)")
    ap.add_argument("--grad-ckpt", type=int, default=-1,
                    help="-1: one memory rule at every N (keep as many layers' activations as the memory left after parameters, "
                         "gradients and optimizer state holds, recompute the rest), 1: recompute every layer, 0: keep everything")
    ap.add_argument("--prox-logp-method", type=str, default=None,
                    help="recompute (decoupled PPO's own forward pass for the proximal log-probs, the reference's default) | "
                         "reuse_train_logp | loglinear")
    ap.add_argument("--staleness", type=int, default=None, help="max_head_offpolicyness")
    ap.add_argument("--train-gpus", type=int, default=0, help="trainer GPUs of an N >= 2 job (default N / 2)")
    ap.add_argument("--sp", type=int, default=0, help="Ulysses sequence-parallel degree of the trainers (default min(4, trainer GPUs))")
    ap.add_argument("--rollout-tp", type=int, default=0, help="tensor-parallel degree of a rollout replica (default 2 with >= 2 rollout GPUs)")
    ap.add_argument("--nccl-steps", type=int, default=-1,
                    help="steps of the same job re-run on the library-collective path (NCCL reduce-scatter / all-gather / "
                         "all-to-all / broadcast instead of the fused kernels) for config.nccl_path_tokens_per_s; "
                         "-1: max(2, steps / 5) when N >= 2, 0: skip")
    ap.add_argument("--retain-kv", type=int, default=1, help="1: requests in flight keep their KV cache across a weight update; "
                    "0: they are interrupted and re-prefilled under the new weights")
    ap.add_argument("--prefix-sharing", type=int, default=1, help="1: the samples of a group share the prompt's KV pages (one prefetch per prompt)")
    args = ap.parse_args()
    pre = dict(PRESETS[args.preset])
    scale = args.length_scale if args.length_scale is not None else pre["length_scale"]
    args.length_scale = scale
    for k in ("prompt_len", "median_len", "max_len"):
        if getattr(args, k) is None:
            setattr(args, k, max(16, int(round(pre[k] * scale / 16)) * 16))
    if args.group_size is None:
        args.group_size = pre["group_size"]
    if args.max_tokens_per_mb is None:
        args.max_tokens_per_mb = pre["max_tokens_per_mb"]
    if args.staleness is None:
        args.staleness = pre.get("staleness", 8)
    if args.prompts_per_gpu is None:
        args.prompts_per_gpu = pre.get("prompts_per_gpu", 2.0)
    if args.prox_logp_method is None:
        args.prox_logp_method = pre.get("prox_logp_method", "recompute")
    if not args.sp and "sp" in pre:
        args.sp = pre["sp"]
    if not args.rollout_tp and "rollout_tp" in pre:
        args.rollout_tp = pre["rollout_tp"]
    return args


class ClockSampler:
    """Samples SM clocks / throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int = 0):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines: list[str] = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200",
                                          "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self._t = threading.Thread(target=self._read, daemon=True)
            self._t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            p = [x.strip() for x in ln.split(",")]
            if len(p) < 9:
                continue
            try:
                sm.append(float(p[1])); mx.append(float(p[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), p[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def run_reference(args):
    """The reference arm: needs the reference package under baseline/_ref plus its serving and
    config dependencies; reports `unavailable` when they cannot be imported."""
    ref = os.path.join(ROOT, "baseline", "_ref")
    why = None
    if not os.path.isdir(os.path.join(ref, "areal")):
        why = ("reference could not be installed offline: its build backend uv_build is not in /opt/wheelhouse "
               "(pip exits with ModuleNotFoundError: uv_build), and its stock GRPO path also needs hydra, omegaconf "
               "and an SGLang server, none of which is installed")
    else:
        sys.path.insert(0, ref)
        missing = []
        for mod in ("hydra", "omegaconf", "sglang"):
            try:
                __import__(mod)
            except Exception:
                missing.append(mod)
        if missing:
            why = ("reference installed but its stock GRPO path cannot start offline: missing " + ", ".join(missing) +
                   " (config loader needs hydra/omegaconf, rollout needs an SGLang server; none is in the wheelhouse)")
    if why is None:
        why = "reference stock path needs SGLang/vLLM server processes that are not runnable in this image"
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


def main():
    args = parse_args()
    if args.impl == "reference":
        return run_reference(args)
    import faulthandler

    # decode-path switches of the kernel library, read once per process at first use: programmatic
    # dependent launch between the kernels of a captured decode step and split-K for the
    # decode-sized projections (measured +4.7% tokens/s on one GPU with both on)
    os.environ.setdefault("AB2_PDL", "1")
    os.environ.setdefault("AB2_DECODE_SPLITK", "1")
    # no step of this benchmark reduces through NVLink multicast (the fused kernels use plain peer loads and
    # stores unless AREAL_NVLS_REDUCE=1), so no buffer is bound to a multicast object: a rank that ends early
    # then cannot disturb its peers' GPUs through one
    if os.environ.get("AREAL_NVLS_REDUCE", "0") != "1":
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")

    import torch
    import torch.distributed as dist

    from areal_b200.infra.bench_driver import run_async_grpo_bench

    # a rank that stops making progress prints every thread's stack and exits instead of
    # holding the other ranks (and the GPUs) until an outer limit
    # (default: shortly before the 870 s a benchmark run is given, so that a stall leaves stacks behind, not just a kill)
    wd = float(os.environ.get("AREAL_BENCH_WATCHDOG_S", "850") or 0)
    if wd > 0:
        faulthandler.dump_traceback_later(wd, exit=True)

    try:
        result = run_async_grpo_bench(args, ClockSampler)
    except BaseException as e:
        # the innermost cause goes out as the LAST stderr line and as a JSON line, so a failure
        # deep inside an engine thread stays readable from the tail of a log
        import traceback

        traceback.print_exc()
        root = e
        while root.__cause__ is not None or (root.__context__ is not None and not root.__suppress_context__):
            root = root.__cause__ or root.__context__
        msg = f"{type(root).__name__}: {root}"
        if int(os.environ.get("RANK", "0")) == 0:
            print(json.dumps({"impl": "native", "error": msg[:2000]}))
        sys.stdout.flush()
        print(f"bench failed, root cause: {msg[:4000]}", file=sys.stderr, flush=True)
        os._exit(1)
    if result is not None:
        print(json.dumps(result))
    return 0


if __name__ == "__main__":
    sys.exit(main())
