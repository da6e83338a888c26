"""Tensor parallelism: shard layout helpers and 2-rank gloo parity run."""
import os
import subprocess
import sys

import pytest
import torch

from areal_b200.models.config import preset
from areal_b200.parallel import tp as TP

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_local_config_and_shard_roundtrip():
    cfg = preset("tiny-qwen3")
    l2 = TP.local_config(cfg, 2)
    assert l2.num_heads == cfg.num_heads // 2 and l2.num_kv_heads == cfg.num_kv_heads // 2 and l2.intermediate_size == cfg.intermediate_size // 2
    assert TP.local_config(cfg, 1) is cfg
    D = cfg.head_dim
    qkv = torch.arange((cfg.num_heads + 2 * cfg.num_kv_heads) * D * 8, dtype=torch.float32).view(-1, 8)
    parts = [TP.shard_tensor(cfg, "layers.0.self_attn.qkv_proj", qkv, 2, r) for r in range(2)]
    assert parts[0].shape[0] == qkv.shape[0] // 2
    # rank 0 holds the first half of the q heads, k heads and v heads
    assert torch.equal(parts[0][: cfg.num_heads * D // 2], qkv[: cfg.num_heads * D // 2])
    assert torch.equal(TP.unshard_tensors(cfg, "layers.0.self_attn.qkv_proj", parts), qkv)
    gu = torch.randn(2 * cfg.intermediate_size, 16)
    parts = [TP.shard_tensor(cfg, "layers.0.mlp.gate_up_proj", gu, 2, r) for r in range(2)]
    assert torch.equal(TP.unshard_tensors(cfg, "layers.0.mlp.gate_up_proj", parts), gu)
    dn = torch.randn(16, cfg.intermediate_size)
    parts = [TP.shard_tensor(cfg, "layers.0.mlp.down_proj", dn, 2, r) for r in range(2)]
    assert parts[0].shape == (16, cfg.intermediate_size // 2) and torch.equal(TP.unshard_tensors(cfg, "x.down_proj", parts), dn)
    norm = torch.randn(cfg.hidden_size)
    assert TP.shard_tensor(cfg, "layers.0.input_layernorm", norm, 2, 1) is norm or torch.equal(TP.shard_tensor(cfg, "layers.0.input_layernorm", norm, 2, 1), norm)


def test_tensor_parallel_matches_unsharded_model_gloo():
    env = dict(os.environ, OMP_NUM_THREADS="1", AREAL_FORCE_CPU="1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
                        "--master-port", "29871", os.path.join(ROOT, "tests", "dist_scripts", "run_tp.py")], cwd=ROOT, env=env,
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("TP_OK") == 2


@pytest.mark.parametrize("seq_par,model", [("0", "tiny-qwen3"), ("1", "tiny-qwen3"), ("0", "tiny-qwen3.5"), ("0", "tiny-qwen3.5-moe")])
def test_train_engine_dp2_tp2_matches_single_rank(tmp_path, seq_par, model):
    """``seq_par`` = 1: the residual stream is split by rows over the tensor-parallel group as well (gather -> product,
    product -> reduce-scatter around attention and MLP; norms and LM head on local rows; outputs gathered for the loss).
    ``tiny-qwen3.5``: linear-attention (gated delta rule) and gated full-attention layers sliced by heads."""
    env = dict(os.environ, OMP_NUM_THREADS="1", AREAL_FORCE_CPU="1", TP_SAVE_DIR=str(tmp_path / "hf"), AREAL_TEST_TP_SP=seq_par, AREAL_TEST_MODEL=model)
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=4", "--master-addr", "127.0.0.1",
                        "--master-port", "29873", os.path.join(ROOT, "tests", "dist_scripts", "run_engine_tp.py")], cwd=ROOT, env=env,
                       capture_output=True, text=True, timeout=400)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("ENGINE_TP_OK") == 4


def test_vocab_parallel_lm_head_matches_full_softmax():
    env = dict(os.environ, OMP_NUM_THREADS="1", AREAL_FORCE_CPU="1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
                        "--master-port", "29877", os.path.join(ROOT, "tests", "dist_scripts", "run_vocab_parallel.py")], cwd=ROOT, env=env,
                       capture_output=True, text=True, timeout=200)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("VP_OK") == 2


def test_sequence_parallel_tp_linear_pair_gloo():
    env = dict(os.environ, OMP_NUM_THREADS="1", AREAL_FORCE_CPU="1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
                        "--master-port", "29879", os.path.join(ROOT, "tests", "dist_scripts", "run_tp_sp.py")], cwd=ROOT, env=env,
                       capture_output=True, text=True, timeout=200)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("TP_SP_OK") == 2


def test_tensor_parallel_rollout_replica_gloo():
    """Inference engine with tp=2 (leader + follower in lock-step) against a single-rank engine:
    identical tokens and log-probs, weight update from full tensors, joint shutdown."""
    env = dict(os.environ, OMP_NUM_THREADS="1", AREAL_FORCE_CPU="1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
                        "127.0.0.1", "--master-port", "29981", os.path.join(ROOT, "tests", "dist_scripts", "run_infer_tp.py")], cwd=ROOT,
                       env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("INFER_TP_OK") == 2


def test_sequence_level_loss_under_ulysses_equals_single_rank():
    """GSPO (sequence-level importance ratios need whole sequences) with two Ulysses ranks: the
    per-token outputs are gathered over the group before the loss, so the gradient norm and the
    parameter update equal the single-rank run."""
    env = dict(os.environ, OMP_NUM_THREADS="1", AREAL_FORCE_CPU="1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
                        "127.0.0.1", "--master-port", "29983", os.path.join(ROOT, "tests", "dist_scripts", "run_sp_gspo.py")], cwd=ROOT,
                       env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("SP_GSPO_OK") == 2


@pytest.mark.parametrize("world", [2, 3])
def test_zigzag_context_parallel_engine_matches_single_rank(world):
    """The engine with ``fsdp.context_parallel=zigzag``: sequence chunks per rank, blockwise attention against the
    gathered keys / values, outputs restored to the packed order before the (sequence-level) loss. Three ranks show
    that no head count has to divide (the tiny model has 4 query and 2 key / value heads)."""
    env = dict(os.environ, OMP_NUM_THREADS="1", AREAL_FORCE_CPU="1", AREAL_TEST_CP_MODE="zigzag")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
                        "127.0.0.1", "--master-port", str(29985 + world), os.path.join(ROOT, "tests", "dist_scripts", "run_sp_gspo.py")],
                       cwd=ROOT, env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("SP_GSPO_OK") == world


def test_hybrid_linear_attention_stack_under_ulysses_matches_single_rank():
    """Gated-delta-rule layers under sequence parallelism: local rows -> (all rows, local heads) in front of the causal
    convolution and the recurrence, back afterwards; the gated full-attention layer uses the same exchange. Update and
    gradient norm of a sequence-level loss equal the single-rank run."""
    env = dict(os.environ, OMP_NUM_THREADS="1", AREAL_FORCE_CPU="1", AREAL_TEST_MODEL="tiny-qwen3.5")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
                        "127.0.0.1", "--master-port", "29991", os.path.join(ROOT, "tests", "dist_scripts", "run_sp_gspo.py")],
                       cwd=ROOT, env=env, capture_output=True, text=True, timeout=400)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("SP_GSPO_OK") == 2


def test_vision_language_model_under_ulysses_matches_single_rank():
    """Qwen2.5-VL and Qwen3-VL (deep-stack features) with the tokens of a micro-batch split over two ranks: image
    features and per-token rotary tables are made for the whole micro-batch and cut to the local rows; losses, gradient
    norms, the update and forward-only log-probs equal the single-rank engine."""
    env = dict(os.environ, OMP_NUM_THREADS="1", AREAL_FORCE_CPU="1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
                        "127.0.0.1", "--master-port", "29993", os.path.join(ROOT, "tests", "dist_scripts", "run_vlm_sp.py")],
                       cwd=ROOT, env=env, capture_output=True, text=True, timeout=500)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("VLM_SP_OK") == 2


def test_vision_language_model_with_tensor_parallel_language_model():
    """Qwen2.5-VL and Qwen3-VL with the language model sliced over two ranks and the image tower whole on both (its
    parameters count once in the global norm): losses, gradient norms, gathered weights after two steps and
    forward-only log-probs equal the single-rank engine."""
    env = dict(os.environ, OMP_NUM_THREADS="1", AREAL_FORCE_CPU="1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
                        "127.0.0.1", "--master-port", "29995", os.path.join(ROOT, "tests", "dist_scripts", "run_vlm_tp.py")],
                       cwd=ROOT, env=env, capture_output=True, text=True, timeout=500)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("VLM_TP_OK") == 2
