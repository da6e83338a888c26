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
