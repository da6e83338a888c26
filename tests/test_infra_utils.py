"""name_resolve backends, ports, seeding, distributed lock, timing controls."""
import os
import threading
import time

import pytest
import torch

from areal_b200.utils import name_resolve, network, seeding
from areal_b200.utils.lock import DistributedLock
from areal_b200.utils.timeutil import EpochStepTimeFreqCtl, FrequencyControl, ValueScheduler


@pytest.mark.parametrize("kind", ["memory", "nfs"])
def test_name_resolve_backends(tmp_path, kind):
    repo = name_resolve.reconfigure(type=kind, record_root=str(tmp_path))
    name_resolve.clear_subtree("a")
    name_resolve.add("a/b/c", "1")
    with pytest.raises(name_resolve.NameEntryExistsError):
        name_resolve.add("a/b/c", "2")
    name_resolve.add("a/b/c", "3", replace=True)
    name_resolve.add("a/b/d", "4")
    assert name_resolve.get("a/b/c") == "3"
    assert sorted(name_resolve.get_subtree("a/b")) == ["3", "4"]
    assert len(name_resolve.find_subtree("a")) == 2
    with pytest.raises(name_resolve.NameEntryNotFoundError):
        name_resolve.get("a/zzz")
    threading.Timer(0.1, lambda: name_resolve.add("a/late", "x")).start()
    assert name_resolve.wait("a/late", timeout=3) == "x"
    with pytest.raises(TimeoutError):
        name_resolve.wait("a/never", timeout=0.2)
    fired = threading.Event()
    name_resolve.watch_names("a/b/d", fired.set, poll_frequency=0.02)
    time.sleep(0.1)
    name_resolve.delete("a/b/d")
    assert fired.wait(2)
    sub = name_resolve.add_subentry("a/servers", "h:1")
    assert name_resolve.get(sub) == "h:1"
    repo.reset()
    with pytest.raises(ValueError, match="unknown name_resolve backend"):
        name_resolve.reconfigure(type="zookeeper")
    name_resolve.reconfigure(type="memory")


def test_ports_and_seeds():
    ps = network.find_free_ports(3)
    assert len(set(ps)) == 3 and all(network.is_port_free(p) for p in ps)
    a = seeding.set_random_seed(1, "trainer0")
    b = seeding.set_random_seed(1, "rollout0")
    assert a != b and seeding.set_random_seed(1, "trainer0") == a
    assert seeding.derive_deterministic_seed("rid", 0, 5) != seeding.derive_deterministic_seed("rid", 1, 5)


def test_distributed_lock(tmp_path):
    l1 = DistributedLock("x/y", root=str(tmp_path))
    l2 = DistributedLock("x/y", root=str(tmp_path))
    assert l1.acquire(timeout=1)
    assert not l2.acquire(timeout=0.1)
    l2.release()                       # a non-owner cannot release
    assert not l2.acquire(timeout=0.1)
    l1.release()
    with l2:
        assert not l1.acquire(timeout=0.05)
    stale = DistributedLock("z", root=str(tmp_path), ttl=0.05)
    assert stale.acquire(timeout=1)
    time.sleep(0.1)
    assert DistributedLock("z", root=str(tmp_path), ttl=0.05).acquire(timeout=1)


def test_frequency_controls_and_schedules():
    f = FrequencyControl(frequency_steps=3)
    assert [f.check() for _ in range(6)] == [False, False, True, False, False, True]
    e = EpochStepTimeFreqCtl(freq_epoch=1, freq_step=None, freq_sec=None)
    assert not e.check(epochs=0, steps=1) and e.check(epochs=1, steps=1)
    sd = e.state_dict()
    e2 = EpochStepTimeFreqCtl(freq_epoch=1)
    e2.load_state_dict(sd)
    assert ValueScheduler("linear", 1.0, 10, 0.0).get(5) == pytest.approx(0.5)
    assert ValueScheduler("cosine", 1.0, 10, 0.0).get(10) == pytest.approx(0.0, abs=1e-9)


def test_async_checkpoint_writer_and_saver_async_mode(tmp_path):
    import threading
    import time as _time

    import torch as _torch

    from areal_b200.api.cli_args import SaverConfig
    from areal_b200.models import hf_io
    from areal_b200.models.config import preset
    from areal_b200.models.decoder import build_model
    from areal_b200.utils.async_checkpoint import AsyncCheckpointWriter
    from areal_b200.utils.saver import Saver

    w = AsyncCheckpointWriter(max_pinned_gb=0.001)
    t = _torch.arange(10.0)
    gate, seen = threading.Event(), {}

    def write(host):
        gate.wait(5)
        seen.update({n: x.clone() for n, x in host})
    w.save([("a", t)], write, "p")
    t.zero_()                                   # the source may change right after staging
    assert w.busy
    gate.set()
    w.wait()
    assert _torch.equal(seen["a"], _torch.arange(10.0)) and not w.busy
    w.save([("a", t)], lambda host: (_ for _ in ()).throw(IOError("disk full")), "p")
    try:
        w.wait()
        raise AssertionError("expected the writer's error")
    except RuntimeError as e:
        assert "failed" in str(e)

    class Eng:
        device = _torch.device("cpu")
        local_index = 0

        def __init__(self):
            self.model = build_model(preset("tiny-qwen2"), dtype=_torch.float32, device="cpu", seed=1)
    eng = Eng()
    sv = Saver(SaverConfig(fileroot=str(tmp_path), experiment_name="e", trial_name="t", freq_steps=1, mode="async"))
    path = sv.save(eng, 0, 0, 0)
    sv.maybe_wait_for_staging()
    sv.wait()
    m2 = build_model(preset("tiny-qwen2"), dtype=_torch.float32, device="cpu", seed=2)
    hf_io.load_model_hf(m2, path)
    a, b = dict(eng.model.named_parameters()), dict(m2.named_parameters())
    assert all(_torch.equal(a[k], b[k]) for k in a)


def test_delta_weight_transfer_exact_and_predicted():
    import torch as _torch

    from areal_b200.wsync.delta import DeltaPusher, changed_blocks, predict_changed_blocks

    _torch.manual_seed(0)
    n, blk = 10_000, 256
    master = _torch.randn(n) * 0.05
    old = master.to(_torch.bfloat16)
    m, v = _torch.randn(n) * 1e-3, _torch.rand(n) * 1e-6 + 1e-8
    lr, b1, b2, eps, wd, step = 1e-7, 0.9, 0.95, 1e-8, 0.0, 10
    m[:512] *= 50000                                          # a region with large updates
    upd = lr * ((m / (1 - b1 ** step)) / ((v / (1 - b2 ** step)).sqrt() + eps) + wd * master)
    new_master = master - upd
    new = new_master.to(_torch.bfloat16)
    exact = changed_blocks(new, old, blk)
    assert exact[:2].all() and exact.float().mean() < 0.9
    pred = predict_changed_blocks(new_master, m, v, lr, b1, b2, eps, wd, step, blk, safety=2.0)
    assert bool((pred | ~exact).all()), "prediction must be a superset of the exact set"
    # pusher: the receiver ends up identical while only changed runs travel
    dst = _torch.zeros(n, dtype=_torch.bfloat16)
    src = old.clone()
    copies = []

    def copy(off, ln):
        copies.append((off, ln))
        dst[off:off + ln] = src[off:off + ln]
    p = DeltaPusher(src, copy, block=blk)
    assert p.push() == 1.0 and _torch.equal(dst, src)
    src.copy_(new)
    frac = p.push()
    assert _torch.equal(dst, src) and 0 < frac < 1.0 and abs(frac - exact.float().mean().item()) < 0.05
    assert p.push() == 0.0 and len(copies) < 2 + exact.sum().item() + 1


def test_stateful_dataloader_resumes_and_partitions():
    from areal_b200.utils.dataloader import StatefulDataLoader, create_dataloader

    data = list(range(103))
    loaders = [create_dataloader(data, 8, rank=r, world_size=2, seed=3) for r in range(2)]
    assert all(len(l) == 51 // 4 for l in loaders)
    e0 = [list(l) for l in loaders]
    seen = [x for b in e0[0] for x in b] + [x for b in e0[1] for x in b]
    assert len(seen) == len(set(seen)) == 2 * 12 * 4                     # ranks see disjoint samples
    e1 = [x for b in loaders[0] for x in b]
    assert e1 != [x for b in e0[0] for x in b]                           # next epoch: another permutation
    # resume in the middle of an epoch
    a = StatefulDataLoader(data, 5, seed=1)
    it = iter(a)
    first = [next(it) for _ in range(7)]
    sd = a.state_dict()
    rest = list(it)
    b = StatefulDataLoader(data, 5, seed=1)
    b.load_state_dict(sd)
    assert list(b) == rest and sd["served"] == 7
    assert first + rest == list(StatefulDataLoader(data, 5, seed=1))
    # a finished epoch resumes at the start of the next one
    c = StatefulDataLoader(data, 5, seed=1)
    list(c)
    d = StatefulDataLoader(data, 5, seed=1)
    d.load_state_dict(c.state_dict())
    assert d.epoch == 1 and list(d) == list(c)
    # without drop_last every rank still gets the same number of batches
    u = [StatefulDataLoader(data, 4, drop_last=False, rank=r, world_size=3, seed=0) for r in range(3)]
    assert len({len(list(x)) for x in u}) == 1


def test_slurm_and_ray_launcher_plans(tmp_path, capsys):
    from areal_b200.api.cli_args import ClusterSpecConfig, GRPOConfig
    from areal_b200.infra.launcher import ray as ray_launcher
    from areal_b200.infra.launcher import slurm as slurm_launcher

    cfg = GRPOConfig(experiment_name="e", trial_name="t", allocation_mode="native:d2+d12", cluster=ClusterSpecConfig(fileroot=str(tmp_path), n_nodes=2))
    jobs = slurm_launcher.plan_jobs("train.py", ["--config", "c.yaml"], cfg, gpus_per_node=8)
    assert [j["name"] for j in jobs] == ["llm_server", "trainer"]
    assert jobs[0]["nodes"] == 1 and jobs[0]["gpus_per_node"] == 2 and jobs[1]["nodes"] == 2 and jobs[1]["gpus_per_node"] == 8
    assert "--nnodes=2 --nproc-per-node=8" in jobs[1]["command"] and "train.py --config c.yaml" in jobs[1]["command"]
    assert slurm_launcher.launch("train.py", ["--config", "c.yaml"], cfg, dry_run=True) == 0
    out = capsys.readouterr().out
    assert out.count("#SBATCH --job-name=e_t:") == 2 and "--gres=gpu:8" in out and "srun" in out
    tasks = ray_launcher.plan_tasks(cfg)
    assert [t["role"] for t in tasks].count("server") == 2 and [t["role"] for t in tasks].count("trainer") == 12
    assert tasks[-1]["rank"] == 11 and tasks[-1]["world"] == 12

    # the Ray launcher against a stand-in module: servers are cancelled when the trainers return
    calls = {"run": [], "cancel": 0}

    class _Handle:
        def __init__(self, fn, opts):
            self.fn, self.opts = fn, opts

        def options(self, **kw):
            return _Handle(self.fn, kw)

        def remote(self, *a):
            calls["run"].append((self.opts.get("name"), a[0]))
            return ("future", self.opts.get("name"))

    class _Ray:
        def is_initialized(self):
            return True

        def remote(self, fn):
            return _Handle(fn, {})

        def get(self, futs):
            return [0 for _ in futs]

        def cancel(self, f, force=False):
            calls["cancel"] += 1

    assert ray_launcher.launch("train.py", [], cfg, ray_module=_Ray()) == 0
    assert calls["cancel"] == 2 and sum(1 for n, _ in calls["run"] if n.startswith("trainer_")) == 12


# --------------------------------------------------------------------------- name_resolve: etcd and Ray backends
class _FakeEtcd:
    """The five JSON-gateway routes of etcd v3 that the backend uses, with lease expiry."""

    def __init__(self):
        import base64
        import http.server
        import json
        import threading
        import time

        kv, leases, lock = {}, {}, threading.Lock()
        self.kv, self.leases, self.keepalives = kv, leases, []
        outer = self

        class H(http.server.BaseHTTPRequestHandler):
            def log_message(self, *a):
                pass

            def do_POST(self):
                body = json.loads(self.rfile.read(int(self.headers["Content-Length"])) or b"{}")
                dec = lambda s: base64.b64decode(s).decode("latin-1")
                enc = lambda s: base64.b64encode(s.encode("latin-1")).decode()
                out = {}
                with lock:
                    now = time.monotonic()
                    for k in [k for k, (_, lid) in kv.items() if lid and leases.get(lid, 0) < now]:
                        del kv[k]                                   # lease ran out
                    if self.path == "/v3/kv/put":
                        kv[dec(body["key"])] = (dec(body["value"]), body.get("lease"))
                    elif self.path == "/v3/kv/range":
                        k, end = dec(body["key"]), dec(body["range_end"]) if "range_end" in body else None
                        hits = [x for x in sorted(kv) if (x == k if end is None else k <= x < end)]
                        out = {"kvs": [{"key": enc(x), "value": enc(kv[x][0])} for x in hits], "count": str(len(hits))}
                    elif self.path == "/v3/kv/deleterange":
                        k, end = dec(body["key"]), dec(body["range_end"]) if "range_end" in body else None
                        hits = [x for x in list(kv) if (x == k if end is None else k <= x < end)]
                        for x in hits:
                            del kv[x]
                        out = {"deleted": str(len(hits))}
                    elif self.path == "/v3/lease/grant":
                        lid = str(len(leases) + 1000)
                        leases[lid] = now + int(body["TTL"])
                        out = {"ID": lid, "TTL": str(body["TTL"])}
                    elif self.path == "/v3/lease/keepalive":
                        leases[body["ID"]] = now + 2
                        outer.keepalives.append(body["ID"])
                        out = {"result": {"ID": body["ID"]}}
                data = json.dumps(out).encode()
                self.send_response(200)
                self.send_header("Content-Length", str(len(data)))
                self.end_headers()
                self.wfile.write(data)

        self.server = http.server.ThreadingHTTPServer(("127.0.0.1", 0), H)
        self.addr = f"127.0.0.1:{self.server.server_address[1]}"
        threading.Thread(target=self.server.serve_forever, daemon=True).start()

    def close(self):
        self.server.shutdown()


def test_etcd_name_resolve_backend_against_a_fake_gateway():
    import time

    from areal_b200.utils import name_resolve as nr

    etcd = _FakeEtcd()
    try:
        repo = nr.Etcd3NameRecordRepository(etcd.addr)
        repo.add("exp/t0/workers/0", "10.0.0.1:7000")
        repo.add("exp/t0/workers/1", "10.0.0.2:7000")
        repo.add("exp/t0/worker", "not-in-subtree")
        with pytest.raises(nr.NameEntryExistsError):
            repo.add("exp/t0/workers/0", "other")
        repo.add("exp/t0/workers/0", "10.0.0.9:7000", replace=True)
        assert repo.get("exp/t0/workers/0") == "10.0.0.9:7000"
        assert repo.get_subtree("exp/t0/workers") == ["10.0.0.9:7000", "10.0.0.2:7000"]
        assert repo.find_subtree("exp/t0/workers") == ["exp/t0/workers/0", "exp/t0/workers/1"]
        assert repo.wait("exp/t0/workers/1", timeout=1) == "10.0.0.2:7000"
        with pytest.raises(nr.NameEntryNotFoundError):
            repo.get("exp/t0/nobody")
        repo.delete("exp/t0/workers/1")
        with pytest.raises(nr.NameEntryNotFoundError):
            repo.delete("exp/t0/workers/1")
        # an entry with a TTL stays alive only while its lease is renewed
        repo.add("exp/t0/alive", "x", keepalive_ttl=1)
        time.sleep(1.6)
        assert repo.get("exp/t0/alive") == "x" and etcd.keepalives
        repo.clear_subtree("exp/t0")
        assert repo.find_subtree("exp/t0") == []
        # the module-level selector
        assert isinstance(nr.reconfigure(type="etcd3", addr=etcd.addr), nr.Etcd3NameRecordRepository)
        nr.add("a/b", "1")
        assert nr.get("a/b") == "1"
        nr.reset()
        with pytest.raises(nr.NameEntryNotFoundError):
            nr.get("a/b")
    finally:
        nr.reconfigure(type="memory")
        etcd.close()


def test_ray_name_resolve_backend_against_a_fake_ray():
    import types

    from areal_b200.utils import name_resolve as nr

    class _Ref:
        def __init__(self, v):
            self.v = v

    class _Handle:
        def __init__(self, obj):
            self._obj = obj

        def __getattr__(self, name):
            fn = getattr(self._obj, name)
            return types.SimpleNamespace(remote=lambda *a: _Ref(fn(*a)))

    actors = {}

    def remote(cls):
        def options(name=None, **kw):
            def make():
                if name not in actors:
                    actors[name] = _Handle(cls())
                return actors[name]
            return types.SimpleNamespace(remote=make)
        return types.SimpleNamespace(options=options)

    def get_actor(name):
        if name not in actors:
            raise ValueError("no such actor")
        return actors[name]

    fake = types.SimpleNamespace(is_initialized=lambda: True, init=lambda **kw: None, remote=remote, get_actor=get_actor,
                                 get=lambda ref: ref.v)
    a = nr.RayNameRecordRepository("kv", ray_module=fake)
    b = nr.RayNameRecordRepository("kv", ray_module=fake)          # a second process finds the same actor
    a.add("job/servers/0", "h0:1")
    b.add("job/servers/1", "h1:1")
    assert a.get_subtree("job/servers") == ["h0:1", "h1:1"] and b.get("job/servers/0") == "h0:1"
    with pytest.raises(nr.NameEntryExistsError):
        b.add("job/servers/0", "dup")
    a.reset()
    with pytest.raises(nr.NameEntryNotFoundError):
        b.get("job/servers/0")
    b.clear_subtree("job")
    assert b.find_subtree("job") == []


def test_perf_tracer_merges_a_profiler_trace_and_profiles_listed_steps(tmp_path):
    """Kernel-level events of a PyTorch-profiler trace land in the rank's trace: shifted onto the
    tracer's clock, attributed to the rank, on virtual (negative) thread ids with names; a
    ``profile_scope`` runs the profiler only on the listed steps."""
    import json

    from areal_b200.api.cli_args import PerfTracerConfig
    from areal_b200.utils.perf_tracer import PerfTracer

    cfg = PerfTracerConfig(experiment_name="e", trial_name="t", fileroot=str(tmp_path), enabled=True, profile_steps=[2])
    tr = PerfTracer(cfg, rank=3, role="trainer")
    fake = {"traceEvents": [
        {"ph": "M", "name": "thread_name", "pid": 0, "tid": 7, "args": {"name": "stream 7"}},
        {"ph": "M", "name": "process_name", "pid": 0, "tid": 0, "args": {"name": "python"}},
        {"ph": "X", "name": "ab2::gemm_bf16_kernel", "cat": "kernel", "pid": 0, "tid": 7, "ts": 5_000_100.0, "dur": 40.0},
        {"ph": "X", "name": "aten::mm", "cat": "cpu_op", "pid": 1234, "tid": 99, "ts": 5_000_000.0, "dur": 60.0},
        {"ph": "X", "name": "internal", "cat": "x", "pid": "Spans", "tid": 1, "ts": 5_000_000.0, "dur": 1.0}]}
    n = tr.merge_profiler_trace(fake, base_us=1000.0)
    assert n == 2
    evs = {e["name"]: e for e in tr._events if e.get("ph") == "X"}
    assert evs["aten::mm"]["ts"] == 1000.0 and evs["ab2::gemm_bf16_kernel"]["ts"] == 1100.0
    assert all(e["pid"] == 3 and e["tid"] < 0 for e in evs.values())
    names = {e["tid"]: e["args"]["name"] for e in tr._events if e.get("ph") == "M"}
    assert names[evs["ab2::gemm_bf16_kernel"]["tid"]] == "stream 7"
    # profile_scope: a plain scope on step 1, profiler events merged on step 2
    tr.set_step(1)
    with tr.profile_scope("update"):
        torch.ones(8).sum()
    before = len(tr._events)
    tr.set_step(2)
    with tr.profile_scope("update"):
        (torch.ones(64, 64) @ torch.ones(64, 64)).sum()
    added = tr._events[before:]
    assert any(e.get("args", {}).get("profiled") for e in added if e.get("name") == "update")
    assert any("mm" in str(e.get("name")) or "matmul" in str(e.get("name")) for e in added)
    tr.save(force=True)
    lines = [json.loads(l) for l in open(os.path.join(tr._out_dir(), "traces-r3.jsonl"))]
    assert len(lines) >= len(added)


def test_memory_profiler_is_inert_without_cuda_and_respects_its_step_list(tmp_path):
    from areal_b200.api.cli_args import MemoryProfilerConfig
    from areal_b200.utils.memory_profiler import MemoryProfiler

    mp = MemoryProfiler(MemoryProfilerConfig(enabled=True, profile_steps=[3], max_entries=1000), rank=0)
    assert mp.wants(3) and not mp.wants(2)
    if not torch.cuda.is_available():
        assert mp.start(3) is False and mp.stop(str(tmp_path)) is None
    assert MemoryProfiler(MemoryProfilerConfig(enabled=False, profile_steps=[3])).wants(3) is False


def test_bench_activation_policy_shrinks_the_micro_batch_before_it_recomputes():
    from areal_b200.infra.bench_driver import kept_layers_for, plan_activation_policy

    # Qwen3-8B trainer rank of the 4-GPU layout: 68.7 GB free, 16384 tokens per rank asked for
    assert kept_layers_for(68.7, 16384, 36, 4096) == 8
    assert plan_activation_policy(68.7, 16384, 36, 4096, 4096) == (4096, 36)
    # 8-GPU layout: more room, still 4096 per rank (8192 would keep 29 of 36)
    assert plan_activation_policy(99.5, 8192, 36, 4096, 4096) == (4096, 36)
    # a lone trainer holding all optimizer state: the floor (longest sequence) stops the shrinking, the rest is recomputed
    t, keep = plan_activation_policy(30.0, 29696, 36, 4096, 5120)
    assert t == 7424 and 0 < keep < 8
    # plenty of memory: nothing changes
    assert plan_activation_policy(150.0, 8192, 36, 4096, 4096) == (8192, 36)
    # no memory at all: floor and full recompute
    assert plan_activation_policy(10.0, 8192, 36, 4096, 4096) == (4096, 0)


def test_version_info_experiment_metadata_and_chained_schedule(tmp_path):
    import areal_b200
    from areal_b200.infra.utils.exp_metadata import load_experiment_metadata, save_experiment_metadata
    from areal_b200.utils.timeutil import ChainedValueScheduler, ValueScheduler

    v = areal_b200.version_info
    assert areal_b200.__version__ == v.version and v.full_version_with_dirty_description.startswith(v.version)
    assert (v.commit == "unknown") == (v.full_version == v.version)
    p = save_experiment_metadata(str(tmp_path), "exp", "t0", {"allocation_mode": "d4"})
    m = load_experiment_metadata(str(tmp_path), "exp", "t0")
    assert p.endswith("version.json") and m["commit_id"] == v.commit and m["allocation_mode"] == "d4" and m["trial_name"] == "t0"
    assert load_experiment_metadata(str(tmp_path), "exp", "other") is None
    # warm-up 0 -> 1 over 10 steps, then cosine 1 -> 0.1 over 90, then whatever the last part ends at
    sch = ChainedValueScheduler([ValueScheduler("linear", 0.0, 10, 1.0), ValueScheduler("cosine", 1.0, 90, 0.1)])
    assert sch.total_iters == 100 and sch.init_value == 0.0 and abs(sch.final_value - 0.1) < 1e-12
    assert sch.get(0) == 0.0 and abs(sch.get(5) - 0.5) < 1e-12 and sch.get(10) == 1.0 and abs(sch.get(55) - 0.55) < 1e-9 and abs(sch.get(1000) - 0.1) < 1e-12
    import pytest

    with pytest.raises(ValueError):
        ChainedValueScheduler([])
    # the package's public names resolve lazily
    assert areal_b200.StalenessManager.__name__ == "StalenessManager" and "PPOTrainer" in dir(areal_b200)
    with pytest.raises(AttributeError):
        areal_b200.no_such_name


def test_launcher_helpers_validate_wait_and_run_the_post_exit_hook(tmp_path):
    import threading
    import time

    import pytest

    from areal_b200.api.cli_args import BaseExperimentConfig, GRPOConfig
    from areal_b200.infra.utils.launcher import (JobException, JobInfo, JobState, run_post_exit_hook, validate_config_for_launcher,
                                                 wait_llm_server_addrs)
    from areal_b200.utils import name_resolve, names

    assert JobState.RUNNING.active() and JobState.PENDING.active() and not any(s.active() for s in (JobState.COMPLETED, JobState.FAILED, JobState.CANCELLED))
    assert "FAILED" in str(JobException("run", "trainer", "node3", JobState.FAILED)) and JobInfo("x", JobState.PENDING).slurm_id is None
    # an RL layout on a config without actor / rollout sections, and a layout larger than the cluster
    base = BaseExperimentConfig(allocation_mode="native:d2+d2")
    base.cluster.fileroot = str(tmp_path / "root")
    with pytest.raises(RuntimeError, match="`actor` is required"):
        validate_config_for_launcher(base)
    g = GRPOConfig(allocation_mode="native:d4+d8")
    g.cluster.fileroot = str(tmp_path / "root")
    with pytest.raises(ValueError, match="needs 12 GPUs"):
        validate_config_for_launcher(g)
    g.allocation_mode = "native:d4+d4"
    validate_config_for_launcher(g)
    validate_config_for_launcher(g, n_gpus_available=0)              # CPU launch: no device count to hold against
    # servers announce themselves; the wait returns once enough have
    name_resolve.reconfigure(type="memory")
    key = names.gen_servers("e", "t")
    threading.Timer(0.3, lambda: [name_resolve.add_subentry(key, a) for a in ("h:1", "h:2")]).start()
    t0 = time.time()
    assert sorted(wait_llm_server_addrs("e", "t", 2, timeout=10, poll=0.05)) == ["h:1", "h:2"] and time.time() - t0 >= 0.25
    with pytest.raises(TimeoutError, match="found 2"):
        wait_llm_server_addrs("e", "t", 3, timeout=0.2, poll=0.05)
    # the hook: a shell command that sees LOG_DIR, a failing one, a module:function, none
    out = tmp_path / "hook.txt"
    g.experiment_name, g.trial_name = "e", "t"
    g.post_exit_hook = f'echo "$LOG_DIR" > {out}'
    assert run_post_exit_hook(g) == 0 and out.read_text().strip().endswith(os.path.join("e", "t"))
    g.post_exit_hook = "exit 7"
    assert run_post_exit_hook(g) == 7
    g.post_exit_hook = "sleep 5"
    assert run_post_exit_hook(g, timeout=0.2) == -1
    g.post_exit_hook = "os:getcwd"
    assert run_post_exit_hook(g) == -1                                # getcwd(config) raises: logged, not propagated
    g.post_exit_hook = "builtins:repr"
    assert run_post_exit_hook(g) == 0
    g.post_exit_hook = None
    assert run_post_exit_hook(g) is None


@pytest.mark.parametrize("reservation,exclusive,present,absent", [
    (None, False, [], ["--reservation", "--exclusive"]), ("shanghai", False, ["#SBATCH --reservation=shanghai"], ["--exclusive"]),
    (None, True, ["#SBATCH --exclusive"], ["--reservation"]), ("r1", True, ["#SBATCH --reservation=r1", "#SBATCH --exclusive"], [])])
def test_sbatch_script_reservation_exclusive_and_container_kinds(reservation, exclusive, present, absent):
    from areal_b200.api.cli_args import SchedulingSpec
    from areal_b200.infra.scheduler.slurm import render_sbatch_script

    spec = SchedulingSpec()
    assert spec.reservation is None and spec.exclusive is False
    txt = render_sbatch_script("j", 2, 1, 4, 8, "/tmp/j.log", "echo hi", reservation=reservation, exclusive=exclusive)
    assert all(p in txt for p in present) and not any(a in txt for a in absent)
    # extra srun arguments and the two container styles
    t2 = render_sbatch_script("j", 1, 1, 4, 8, "/tmp/j.log", "python x.py", container_image="/img.sif", container_mounts="/data:/data",
                              srun_additional_args="--mpi=pmix --label", container_type="apptainer")
    line = [l for l in t2.splitlines() if l.startswith("srun")][0]
    assert "--mpi=pmix --label" in line and "apptainer exec --nv --bind /data:/data /img.sif" in line and "--container-image" not in line
    t3 = render_sbatch_script("j", 1, 1, 4, 8, "/tmp/j.log", "python x.py", container_image="nvcr.io/x:1", container_mounts="/data:/data", container_type="pyxis")
    assert "--container-image=nvcr.io/x:1 --container-mounts=/data:/data" in t3 and "apptainer" not in t3


def test_hostport_helpers_handle_ipv6():
    from areal_b200.utils.network import format_hostport, gethostip_any, is_ipv6_literal, split_hostport

    assert format_hostport("node3", 80) == "node3:80" and format_hostport("10.0.0.1", 80) == "10.0.0.1:80"
    assert format_hostport("fe80::1", 8000) == "[fe80::1]:8000" and format_hostport("[fe80::1]", 8000) == "[fe80::1]:8000"
    assert split_hostport("node3:80") == ("node3", 80) and split_hostport("[fe80::1%eth0]:9") == ("fe80::1%eth0", 9)
    assert split_hostport("2001:db8::5:7000") == ("2001:db8::5", 7000)            # unbracketed, as some launchers write it
    assert split_hostport(format_hostport("::1", 1234)) == ("::1", 1234)
    for bad in ("node3", ":80", "[fe80::1]80", "[nonsense]:80", "1.2.3.4:99999", "zz::zz:80", "[fe80::1"):
        with pytest.raises(ValueError):
            split_hostport(bad)
    assert is_ipv6_literal("::1") and is_ipv6_literal("[::1]") and not is_ipv6_literal("127.0.0.1") and not is_ipv6_literal("host")
    ip = gethostip_any()
    assert isinstance(ip, str) and ip
