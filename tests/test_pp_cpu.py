"""Pipeline parallelism over gloo ranks on CPU."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("stages,port", [(2, 29881), (3, 29883)])
def test_pipeline_matches_unsplit_model(stages, port):
    env = dict(os.environ, OMP_NUM_THREADS="1", AREAL_FORCE_CPU="1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={stages}", "--master-addr",
                        "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests", "dist_scripts", "run_pp.py")], cwd=ROOT,
                       env=env, capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("PP_OK") == stages


def test_expert_parallel_matches_unsplit_moe():
    env = dict(os.environ, OMP_NUM_THREADS="1", AREAL_FORCE_CPU="1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
                        "127.0.0.1", "--master-port", "29887", os.path.join(ROOT, "tests", "dist_scripts", "run_ep.py")], cwd=ROOT,
                       env=env, capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("EP_OK") == 2


@pytest.mark.parametrize("ranks,port", [(2, 29917), (4, 29919)])
def test_zigzag_context_parallel_attention(ranks, port):
    """Zig-zag split / gather round trip and attention against gathered K/V (forward + gradients)."""
    env = dict(os.environ, OMP_NUM_THREADS="1", AREAL_FORCE_CPU="1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={ranks}", "--master-addr",
                        "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests", "dist_scripts", "run_cp.py")], cwd=ROOT,
                       env=env, capture_output=True, text=True, timeout=180)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("CP_OK") == ranks


def test_train_engine_pipeline_x_data_parallel(tmp_path):
    """dp2 x pp2 engine (ZeRO inside each stage, 1F1B over micro-batches) against one rank:
    gradient norms, weights after two steps, forward-only outputs on every stage, HF export /
    reload, complete weight dictionary; untied and tied embeddings."""
    env = dict(os.environ, OMP_NUM_THREADS="1", AREAL_FORCE_CPU="1", PP_SAVE_DIR=str(tmp_path))
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=4", "--master-addr",
                        "127.0.0.1", "--master-port", "29931", os.path.join(ROOT, "tests", "dist_scripts", "run_engine_pp.py")], cwd=ROOT,
                       env=env, capture_output=True, text=True, timeout=400)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("ENGINE_PP_OK") == 4


@pytest.mark.parametrize("ranks,port", [(2, 29941), (4, 29943)])
def test_train_engine_expert_parallel(tmp_path, ranks, port):
    """d{N}e2 engine on a tiny MoE model (dense parameters sharded over all ranks, experts over the
    replicas of the same experts, one global norm) against one rank; HF export / reload, sharded
    recovery checkpoint with both optimizers."""
    env = dict(os.environ, OMP_NUM_THREADS="1", AREAL_FORCE_CPU="1", EP_SAVE_DIR=str(tmp_path))
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={ranks}", "--master-addr",
                        "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests", "dist_scripts", "run_engine_ep.py")], cwd=ROOT,
                       env=env, capture_output=True, text=True, timeout=400)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("ENGINE_EP_OK") == ranks
