"""Multi-GPU tests: each spawns a torchrun job on 2 GPUs and checks its exit code
(skipped when fewer GPUs are visible)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.multi_gpu]
HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


def _torchrun(script, nproc, port, extra=(), timeout=400, env=None):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), script, *extra]
    e = dict(os.environ)
    e.update(env or {})
    r = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=timeout, env=e)
    if r.returncode != 0:
        sys.stderr.write(r.stdout[-4000:] + r.stderr[-6000:])
    return r


def _need(n):
    if not torch.cuda.is_available() or torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")


def test_fused_zero_step_matches_nccl_path():
    _need(2)
    r = _torchrun(os.path.join(HERE, "dist_scripts", "run_fused_zero.py"), 2, 29711)
    assert r.returncode == 0
    assert "identical_across_ranks True" in r.stdout


def test_split_async_grpo_two_gpus():
    """1 trainer + 1 rollout rank, tiny model, weights pushed peer to peer."""
    _need(2)
    r = _torchrun(os.path.join(ROOT, "bench.py"), 2, 29721,
                  extra=["--gpus", "2", "--model", "tiny-qwen3", "--steps", "2", "--warmup", "2", "--prompt-len", "64",
                         "--median-len", "64", "--max-len", "128"])
    assert r.returncode == 0
    assert '"metric"' in r.stdout


def test_fused_tp_gemm_collectives_two_gpus():
    """all-gather->GEMM and GEMM->reduce-scatter kernels (peer TMA loads / peer reductions)
    against fp32 math on gathered operands."""
    _need(2)
    r = _torchrun(os.path.join(HERE, "dist_scripts", "run_tp_fused.py"), 2, 29731, timeout=300, env={"NCCL_NVLS_ENABLE": "0"})
    assert r.returncode == 0
    assert r.stdout.count("TP_FUSED_OK") == 2


def test_fused_ulysses_projections_two_gpus():
    """QKV projection + seq->heads scatter and heads->seq gather + output projection, each one
    kernel over peer memory, against fp32 math on gathered operands."""
    _need(2)
    r = _torchrun(os.path.join(HERE, "dist_scripts", "run_ulysses_fused.py"), 2, 29751, timeout=300, env={"NCCL_NVLS_ENABLE": "0"})
    assert r.returncode == 0
    assert r.stdout.count("ULYSSES_FUSED_OK") == 2


def test_sequence_parallel_engine_fused_projections_two_gpus():
    """Train engine with sp=2: attention blocks on the fused projection + exchange kernels
    against the same engine on NCCL all-to-alls (loss, gradient norm, weights after two steps)."""
    _need(2)
    r = _torchrun(os.path.join(HERE, "dist_scripts", "run_engine_sp_fused.py"), 2, 29761, timeout=300, env={"NCCL_NVLS_ENABLE": "0"})
    assert r.returncode == 0
    assert r.stdout.count("ENGINE_SP_FUSED_OK") == 2


def test_fused_ep_dispatch_combine_two_gpus():
    """Expert-parallel dispatch and combine as one peer-memory kernel each, against the NCCL
    all-to-all dispatcher on the same model and tokens (hidden states, loss, all gradients)."""
    _need(2)
    r = _torchrun(os.path.join(HERE, "dist_scripts", "run_ep_fused.py"), 2, 29771, timeout=300, env={"NCCL_NVLS_ENABLE": "0"})
    assert r.returncode == 0
    assert r.stdout.count("EP_FUSED_OK") == 2


def test_engine_expert_parallel_fused_dispatch_two_gpus():
    """``native:d2e2`` train engine in bf16: three optimizer steps through the fused dispatch / combine
    kernels give the gradient norms of the NCCL all-to-all path."""
    _need(2)
    r = _torchrun(os.path.join(HERE, "dist_scripts", "run_engine_ep_gpu.py"), 2, 29781, timeout=300, env={"NCCL_NVLS_ENABLE": "0"})
    assert r.returncode == 0
    assert r.stdout.count("ENGINE_EP_GPU_OK") == 2


def test_engine_pipeline_zero_bubble_matches_1f1b_two_gpus():
    """``native:d1p2`` train engine in bf16: the split-backward ZBH1 schedule reproduces the gradient
    norms of plain 1F1B over three optimizer steps."""
    _need(2)
    r = _torchrun(os.path.join(HERE, "dist_scripts", "run_engine_pp_gpu.py"), 2, 29791, timeout=300, env={"NCCL_NVLS_ENABLE": "0"})
    assert r.returncode == 0
    assert r.stdout.count("ENGINE_PP_GPU_OK") == 2


def test_engine_tensor_parallel_sequence_parallel_fused_two_gpus():
    """``native:d1t2`` train engine in bf16 with the residual stream split by rows: fused gather->GEMM /
    GEMM->reduce-scatter kernels and their NCCL form reproduce losses and gradient norms of all-reduce tensor
    parallelism over three optimizer steps."""
    _need(2)
    r = _torchrun(os.path.join(HERE, "dist_scripts", "run_engine_tp_sp_gpu.py"), 2, 29793, timeout=300, env={"NCCL_NVLS_ENABLE": "0"})
    assert r.returncode == 0
    assert r.stdout.count("ENGINE_TP_SP_GPU_OK") == 2


def test_vocab_parallel_head_partials_over_peer_memory_two_gpus():
    """Vocabulary-parallel log-probs and entropy on 2 GPUs against the fp32 full-softmax oracle, with the per-row
    partials gathered by NCCL and by peer stores + flag barrier (``PartialsExchange``): both forms give the same bits."""
    _need(2)
    r = _torchrun(os.path.join(HERE, "dist_scripts", "run_vocab_parallel.py"), 2, 29795, timeout=300, env={"NCCL_NVLS_ENABLE": "0"})
    assert r.returncode == 0
    assert r.stdout.count("VP_OK") == 2 and r.stdout.count("VP_PEER_OK") == 2


def test_engine_layouts_sharded_hybrid_tp_vlm_tp_two_gpus():
    """Sharded parameters (ZeRO-3 on NCCL broadcasts / reductions), a tensor-parallel linear-attention model and a
    vision-language model with a tensor-parallel language model on 2 GPUs in bf16: gradient norms and the three-step
    update follow a single-rank engine with replicated parameters."""
    _need(2)
    r = _torchrun(os.path.join(HERE, "dist_scripts", "run_engine_layouts_gpu.py"), 2, 29797, timeout=300, env={"NCCL_NVLS_ENABLE": "0"})
    assert r.returncode == 0
    assert r.stdout.count("ENGINE_LAYOUTS_GPU_OK") == 2


def test_engine_layouts_expert_tensor_pipeline_four_gpus():
    """Whole and sliced experts under tensor-parallel attention (``native:d2t2e2``, ``native:(attn:d2t2|ffn:e2t2)``) and
    tensor / expert parallelism inside pipeline stages (``native:d1p2t2``, ``native:d2p2e2``) on 4 GPUs in bf16: gradient
    norms and the three-step update follow a single-rank engine."""
    _need(4)
    r = _torchrun(os.path.join(HERE, "dist_scripts", "run_engine_layouts_gpu.py"), 4, 29799, timeout=300,
                  env={"NCCL_NVLS_ENABLE": "0", "LAYOUTS": "ep-tp,ep-etp,pp-tp,pp-ep"})
    assert r.returncode == 0
    assert r.stdout.count("ENGINE_LAYOUTS_GPU_OK") == 4
