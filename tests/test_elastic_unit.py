"""Elastic pieces in isolation: the driver with a mocked rendezvous, fixed
host lists and in-thread fake workers; host manager bookkeeping; TorchState /
ElasticSampler semantics in a single process. Mirrors
test/single/test_elastic_driver.py and test/single/test_torch_elastic.py."""
import time
from unittest import mock

import pytest
import torch

from horovod_b200.common.elastic import HostUpdateResult
from horovod_b200.runner.elastic import driver as driver_mod
from horovod_b200.runner.elastic.discovery import FixedHosts, HostManager
from horovod_b200.runner.elastic.driver import ElasticDriver
from parallel_utils import run_parallel


@pytest.fixture(autouse=True)
def fast(monkeypatch):
    monkeypatch.setattr(driver_mod, "DISCOVER_HOSTS_FREQUENCY_SECS", 0.01)


def test_rank_and_size_assignment_and_results():
    driver = ElasticDriver(mock.Mock(), FixedHosts({"host-1": 2, "host-2": 2}), min_np=2,
                           max_np=4)
    driver.wait_for_available_slots(min_np=2)
    seen = {}

    def worker(slot_info, events):
        updated = driver.get_slot_info(slot_info.hostname, slot_info.local_rank)
        seen[slot_info.rank] = (slot_info, updated)
        return 0, time.time()

    driver.start(np=2, create_worker_fn=worker)
    res = driver.get_results().worker_results
    driver.stop()
    assert len(res) == 4 and all(code == 0 for code, _ in res.values())
    assert sorted(seen) == [0, 1, 2, 3]
    for rank, (slot, updated) in seen.items():
        assert updated.size == 4 and updated.rank == rank
        assert updated.local_size == 2 and updated.cross_size == 2


def test_host_added_triggers_new_round_with_stable_ranks():
    disc = FixedHosts({"host-1": 2})
    driver = ElasticDriver(mock.Mock(), disc, min_np=2, max_np=4)
    driver.wait_for_available_slots(min_np=2)
    final = {}

    def worker(slot_info, events):
        if slot_info.hostname == "host-1":
            if slot_info.rank == 0:
                disc.set({"host-1": 2, "host-2": 2})
            driver.wait_for_available_slots(4)
            # surviving workers re-rendezvous; the round they complete starts
            # the workers of the new host
            driver.record_ready(slot_info.hostname, slot_info.local_rank)
        final[(slot_info.hostname, slot_info.local_rank)] = driver.get_slot_info(
            slot_info.hostname, slot_info.local_rank)
        return 0, time.time()

    driver.start(np=2, create_worker_fn=worker)
    res = driver.get_results().worker_results
    driver.stop()
    assert len(res) == 4
    assert all(info.size == 4 for info in final.values())
    # old host keeps the low ranks (rank 0 holds the state to broadcast)
    assert final[("host-1", 0)].rank == 0 and final[("host-1", 1)].rank == 1
    assert {final[("host-2", 0)].rank, final[("host-2", 1)].rank} == {2, 3}


def test_failed_host_is_blacklisted_and_job_continues():
    driver = ElasticDriver(mock.Mock(), FixedHosts({"host-1": 2, "host-2": 2}), min_np=2,
                           max_np=4)
    driver.wait_for_available_slots(min_np=4)
    attempts = {}

    def worker(slot_info, events):
        key = (slot_info.hostname, slot_info.local_rank)
        attempts[key] = attempts.get(key, 0) + 1
        if slot_info.hostname == "host-2":
            return 1, time.time()
        # survivors notice the failure and come back for a new round
        driver.record_ready(slot_info.hostname, slot_info.local_rank)
        info = driver.get_slot_info(slot_info.hostname, slot_info.local_rank)
        assert info.size == 2
        return 0, time.time()

    driver.start(np=4, create_worker_fn=worker)
    res = driver.get_results()
    driver.stop()
    assert res.error_message is None
    assert driver.host_manager.is_blacklisted("host-2")
    assert not driver.host_manager.is_blacklisted("host-1")
    assert attempts[("host-2", 0)] == 1  # never restarted on the bad host


def test_all_workers_failing_stops_the_job():
    driver = ElasticDriver(mock.Mock(), FixedHosts({"host-1": 2}), min_np=2, max_np=2)
    driver.wait_for_available_slots(min_np=2)
    driver.start(np=2, create_worker_fn=lambda s, e: (1, time.time()))
    res = driver.get_results()
    driver.stop()
    assert res.error_message is not None
    assert all(code == 1 for code, _ in res.worker_results.values())


def test_wait_for_slots_times_out():
    driver = ElasticDriver(mock.Mock(), FixedHosts({"host-1": 1}), min_np=2, max_np=2,
                           timeout=0.3)
    with pytest.raises(TimeoutError):
        driver.wait_for_available_slots(min_np=2)
    driver.stop()


def test_host_manager_update_results_and_order():
    disc = FixedHosts({"a": 2})
    hm = HostManager(disc)
    assert hm.update_available_hosts() == HostUpdateResult.added
    assert hm.update_available_hosts() == HostUpdateResult.no_update
    disc.set({"a": 2, "b": 2})
    assert hm.update_available_hosts() == HostUpdateResult.added
    disc.set({"b": 2, "c": 1})
    assert hm.update_available_hosts() == HostUpdateResult.mixed
    assert hm.current_hosts.host_assignment_order == ["b", "c"]  # survivor first
    hm.blacklist("b")
    assert hm.current_hosts.host_assignment_order == ["c"]
    assert hm.current_hosts.count_available_slots() == 1
    disc.set({"b": 1, "c": 1})
    assert hm.update_available_hosts() == HostUpdateResult.removed


def test_torch_state_commit_restore_and_sampler():
    import horovod_b200.torch as hvd
    hvd.init()
    try:
        model = torch.nn.Linear(3, 2)
        opt = torch.optim.SGD(model.parameters(), lr=0.1, momentum=0.9)
        state = hvd.elastic.TorchState(model=model, optimizer=opt, epoch=3, batch=7)
        w0 = model.weight.detach().clone()
        state.commit()
        with torch.no_grad():
            model.weight.add_(1.0)
        state.epoch, state.batch = 9, 1
        state.restore()
        assert torch.equal(model.weight, w0) and state.epoch == 3 and state.batch == 7
        state.epoch = 4
        state.commit()
        with torch.no_grad():
            model.weight.mul_(0)
        state.restore()
        assert torch.equal(model.weight, w0) and state.epoch == 4
        state.sync()  # size 1: a no-op that must not fail
        called = []
        state.register_reset_callbacks([lambda: called.append(1)])
        state.on_reset()
        assert called == [1]
        # host update raised at commit, with skip_sync only for pure removals
        state.on_hosts_updated(time.time() + 10, HostUpdateResult.removed)
        with pytest.raises(hvd.HostsUpdatedInterrupt) as e:
            state.commit()
        assert e.value.skip_sync

        data = list(range(20))
        sampler = hvd.elastic.ElasticSampler(data, shuffle=False)
        assert list(sampler) == data and len(sampler) == 20
        sampler.record_batch(0, 5)
        sampler.record_batch(1, 5)
        assert sampler.processed_indices == set(range(10))
        sampler.reset()
        assert list(sampler) == list(range(10, 20))
        saved = sampler.state_dict()
        sampler.set_epoch(1)
        assert list(sampler) == data
        sampler.load_state_dict(saved)
        assert list(sampler) == list(range(10, 20))
        shuffled = hvd.elastic.ElasticSampler(data, shuffle=True, seed=3)
        a = list(shuffled)
        assert sorted(a) == data and a != data
        shuffled.set_epoch(1)
        assert list(shuffled) != a
    finally:
        hvd.shutdown()


def _joiner_takes_over_rank0_state(rank, size):
    """What a worker that joins a running job must end up with after
    state.sync(): rank 0's weights, optimizer state, sampler progress and
    attributes, and these as its rollback point too."""
    import horovod_b200.torch as hvd
    hvd.init()
    torch.manual_seed(100 + rank)                     # every rank starts from other weights
    model = torch.nn.Linear(6, 3)
    opt = torch.optim.SGD(model.parameters(), lr=0.1, momentum=0.9)
    data = torch.utils.data.TensorDataset(torch.arange(40.0).view(40, 1))
    sampler = hvd.elastic.ElasticSampler(data, shuffle=False)
    state = hvd.elastic.TorchState(model, opt, sampler=sampler, epoch=0, batch=0)
    if rank == 0:                                     # the old-timer has trained and committed
        model(torch.ones(2, 6)).sum().backward()
        opt.step()
        list(iter(sampler))
        sampler.record_batch(0, 8)
        state.epoch, state.batch = 3, 1
        state.save()                                  # commit() without its collective check
    state.sync()
    flat = torch.cat([p.detach().reshape(-1) for p in model.parameters()])
    momentum = torch.cat([opt.state[p]["momentum_buffer"].reshape(-1) for p in model.parameters()])
    everyone = hvd.allgather(torch.cat([flat, momentum]).unsqueeze(0), name="joiner.check")
    same = bool((everyone == everyone[0]).all())
    progress = (state.epoch, state.batch, len(sampler.processed_indices), len(sampler))
    # a rollback returns to the synchronised state, not to the pre-join one
    with torch.no_grad():
        for p in model.parameters():
            p.add_(1.0)
    state.epoch = 9
    state.restore()
    after = torch.cat([p.detach().reshape(-1) for p in model.parameters()])
    rolled_back = bool(torch.equal(after, flat)) and state.epoch == 3 and \
        len(sampler.processed_indices) == 8
    hvd.shutdown()
    return same, progress, rolled_back


def test_a_joining_worker_takes_over_rank0_state_on_sync():
    for same, progress, rolled_back in run_parallel(_joiner_takes_over_rank0_state, np=2,
                                                    timeout=90):
        assert same and rolled_back
        assert progress == (3, 1, 8, 16)              # 32 samples left for 2 ranks
