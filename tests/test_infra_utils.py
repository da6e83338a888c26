"""name_resolve backends, ports, seeding, distributed lock, timing controls."""
import threading
import time

import pytest

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
    with pytest.raises(RuntimeError):
        name_resolve.reconfigure(type="etcd3")
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
