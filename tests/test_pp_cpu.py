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


def test_train_engine_data_pipeline_tensor_parallel_8_ranks(tmp_path):
    """``native:d2p2t2``: two replicas x two stages x two tensor-parallel slices per stage against one rank (tied
    embedding: its last-stage copy and the slices' replicated parameters each count once in the global norm)."""
    env = dict(os.environ, OMP_NUM_THREADS="1", AREAL_FORCE_CPU="1", PP_SAVE_DIR=str(tmp_path), PP_LAYOUT="native:d2p2t2")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=8", "--master-addr",
                        "127.0.0.1", "--master-port", "29933", os.path.join(ROOT, "tests", "dist_scripts", "run_engine_pp.py")], cwd=ROOT,
                       env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("ENGINE_PP_OK") == 8


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


@pytest.mark.parametrize("backend,port,model", [("native:d2t2e2", 29945, "tiny-qwen3-moe"), ("native:(attn:d2t2|ffn:e2t2)", 29947, "tiny-qwen3-moe"),
                                                ("native:d2t2e2", 29949, "tiny-qwen3.5-moe"), ("native:(attn:d2t2|ffn:e2t2)", 29951, "tiny-qwen3.5-moe")])
def test_train_engine_expert_parallel_with_tensor_parallel_attention(tmp_path, backend, port, model):
    """Hybrid attention / expert layouts on 4 ranks against one rank: tensor-parallel attention with whole experts
    spread over data x tensor ranks (each TP rank routes its share of the tokens), and experts sliced over the TP group
    and spread over the data ranks. Weights after two steps, the global gradient norm, HF export / reload.
    ``tiny-qwen3.5-moe``: linear-attention layers and a sigmoid-gated shared expert (sliced with the experts, or whole on
    each rank's row share)."""
    env = dict(os.environ, OMP_NUM_THREADS="1", AREAL_FORCE_CPU="1", EP_SAVE_DIR=str(tmp_path), EP_TP_BACKEND=backend, EP_TP_MODEL=model)
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=4", "--master-addr",
                        "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests", "dist_scripts", "run_engine_ep_tp.py")], cwd=ROOT,
                       env=env, capture_output=True, text=True, timeout=400)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("ENGINE_EP_TP_OK") == 4


def test_deferred_weight_gradients_match_plain_backward():
    """Split backward used by the ZBH1 schedule: with a queue installed, ``linear`` / ``grouped_linear``
    backward yields input gradients only; flushing the queue adds exactly the weight gradients."""
    import torch

    from areal_b200.ops import functional as OF

    torch.manual_seed(0)
    x = torch.randn(7, 8, requires_grad=True)
    w1, w2 = torch.nn.Parameter(torch.randn(6, 8)), torch.nn.Parameter(torch.randn(3, 5, 6))
    counts = [2, 0, 5]

    def loss():
        return OF.grouped_linear(torch.relu(OF.linear(x, w1)), w2, counts).square().sum()

    loss().backward()
    ref = [t.grad.clone() for t in (x, w1, w2)]
    for t in (x, w1, w2):
        t.grad = None
    OF.SPLIT_BACKWARD = True
    try:
        y = loss()
        with OF.deferred_wgrad() as q:
            y.backward()
        assert w1.grad is None and w2.grad is None and len(q) == 2
        assert torch.allclose(x.grad, ref[0], atol=1e-5)
        OF.flush_wgrad(q)
    finally:
        OF.SPLIT_BACKWARD = False
    assert torch.allclose(w1.grad, ref[1], atol=1e-4) and torch.allclose(w2.grad, ref[2], atol=1e-4)
    # with main_grad buffers (flat-shard training) the products accumulate there
    w1.grad = None
    w1.main_grad = torch.zeros(6, 8)
    OF.SPLIT_BACKWARD = True
    try:
        with OF.deferred_wgrad() as q:
            loss().backward()
        OF.flush_wgrad(q)
    finally:
        OF.SPLIT_BACKWARD = False
    assert w1.grad is None and torch.allclose(w1.main_grad, ref[1], atol=1e-4)
    # a weight that is a VIEW of a parameter (one expert of a stack, the per-expert loop of the CPU path): its gradient
    # has to reach the parameter through autograd, so it is computed at once instead of waiting in the queue
    w3 = torch.nn.Parameter(torch.randn(3, 5, 8))
    xs = torch.randn(4, 8)
    OF.linear(xs, w3[1]).square().sum().backward()
    want = w3.grad.clone()
    w3.grad = None
    OF.SPLIT_BACKWARD = True
    try:
        with OF.deferred_wgrad() as q:
            OF.linear(xs, w3[1]).square().sum().backward()
        assert len(q) == 0
    finally:
        OF.SPLIT_BACKWARD = False
    assert torch.allclose(w3.grad, want, atol=1e-5) and w3.grad[0].abs().max() == 0


@pytest.mark.parametrize("P,M", [(2, 4), (4, 8), (4, 5), (8, 16)])
def test_zbv_timetable_is_complete_and_respects_dependencies(P, M):
    """V placement + greedy order: every forward and backward of every (micro-batch, stage) runs exactly once, on the
    rank that owns the stage, after its input arrived; at most 2 P chunk activations are alive on a rank unless the
    bound had to be lifted; the table is no longer than the interleaved 1F1B one for the same problem."""
    from areal_b200.parallel.pp import build_timetable, owner_of, stage_of

    V, S = 2, 2 * P
    assert [owner_of(s, P, "v") for s in (0, P - 1, P, S - 1)] == [(0, 0), (P - 1, 0), (P - 1, 1), (0, 1)]
    assert all(owner_of(stage_of(r, v, P, "v"), P, "v") == (r, v) for r in range(P) for v in range(V))
    table = build_timetable(P, V, M, "ZBV", False, "v")
    done, have, alive, peak = {}, set(), [0] * P, 0
    for tick, (row, delivered) in enumerate(table):
        for (src, dst, kind, mb, s) in delivered:
            assert owner_of(s, P, "v")[0] == dst
            have.add((kind, mb, s))
        for r, op in enumerate(row):
            if op is None:
                continue
            kind, mb, v = op
            s = stage_of(r, v, P, "v")
            assert (kind, mb, s) not in done
            if kind == "F":
                assert s == 0 or ("act", mb, s) in have
                alive[r] += 1
            else:
                assert ("F", mb, s) in done and (s == S - 1 or ("grad", mb, s) in have)
                alive[r] -= 1
            done[(kind, mb, s)] = tick
            peak = max(peak, alive[r])
    assert len(done) == 2 * M * S and all(a == 0 for a in alive)
    assert peak <= 2 * P + 1
    if M % P == 0:
        loop = build_timetable(P, V, M, "Interleaved1F1B", False, "loop")
        assert len(table) <= len(loop) + P
