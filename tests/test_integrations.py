"""Cluster integrations without their frameworks installed: the Ray
coordinator's rank arithmetic and rendezvous, Ray host discovery against a
stand-in ``ray`` module, the Spark rank arithmetic and the filesystem store
(parity: test/single/test_ray.py coordinator tests, test/utils/spark_common,
test/integration/test_spark.py store tests)."""
import os
import sys
import types

import pytest


def test_ray_coordinator_rank_layout_and_rendezvous():
    from horovod_b200.ray import Coordinator
    c = Coordinator()
    # 2 nodes with 2 ranks, 1 node with 1 rank, registered out of node order
    for hostname, node, rank in (("h1", "n1", 0), ("h2", "n2", 1), ("h1", "n1", 2),
                                 ("h3", "n3", 3), ("h2", "n2", 4)):
        c.register(hostname, node, rank)
    assert c.world_size == 5 and c.hostnames == {"h1", "h2", "h3"}
    assert c.node_id_string == "n1:2,n2:2,n3:1"
    info = c.finalize_registration()
    assert info[0] == {"HOROVOD_RANK": 0, "HOROVOD_SIZE": 5, "HOROVOD_LOCAL_RANK": 0,
                       "HOROVOD_LOCAL_SIZE": 2, "HOROVOD_CROSS_RANK": 0, "HOROVOD_CROSS_SIZE": 3}
    assert info[2]["HOROVOD_LOCAL_RANK"] == 1 and info[2]["HOROVOD_CROSS_SIZE"] == 2
    assert info[4]["HOROVOD_CROSS_RANK"] == 1 and info[4]["HOROVOD_LOCAL_RANK"] == 1
    assert info[3]["HOROVOD_CROSS_RANK"] == 2 and info[3]["HOROVOD_LOCAL_SIZE"] == 1
    env = c.establish_rendezvous("127.0.0.1")
    try:
        assert env["HOROVOD_GLOO_RENDEZVOUS_ADDR"] == "127.0.0.1"
        assert int(env["HOROVOD_GLOO_RENDEZVOUS_PORT"]) > 0
        assert env["HOROVOD_CONTROLLER"] == "gloo"
    finally:
        c.shutdown()


def test_ray_executor_argument_checks_and_missing_ray():
    from horovod_b200.ray import RayExecutor
    with pytest.raises(ValueError):
        RayExecutor()
    with pytest.raises(ValueError):
        RayExecutor(num_workers=2, num_hosts=1)
    with pytest.raises(ValueError):
        RayExecutor(num_workers=2, gpus_per_worker=1)
    ex = RayExecutor(num_hosts=2, num_workers_per_host=4, use_gpu=True)
    assert ex.num_workers == 8 and ex.gpus_per_worker == 1
    if "ray" not in sys.modules:
        try:
            import ray  # noqa: F401
        except ImportError:
            with pytest.raises(ImportError, match="ray"):
                ex.start()


def test_ray_host_discovery_counts_slots(monkeypatch):
    from horovod_b200.ray import RayHostDiscovery
    fake = types.ModuleType("ray")
    fake.nodes = lambda: [
        {"alive": True, "NodeManagerAddress": "10.0.0.1", "Resources": {"CPU": 16, "GPU": 8}},
        {"alive": True, "NodeManagerAddress": "10.0.0.2", "Resources": {"CPU": 4, "GPU": 8}},
        {"alive": False, "NodeManagerAddress": "10.0.0.3", "Resources": {"CPU": 16, "GPU": 8}},
        {"alive": True, "NodeManagerAddress": "10.0.0.4", "Resources": {"CPU": 16}},
    ]
    monkeypatch.setitem(sys.modules, "ray", fake)
    assert RayHostDiscovery(use_gpu=True, cpus_per_slot=2, gpus_per_slot=1) \
        .find_available_hosts_and_slots() == {"10.0.0.1": 8, "10.0.0.2": 2}
    assert RayHostDiscovery(use_gpu=False, cpus_per_slot=4) \
        .find_available_hosts_and_slots() == {"10.0.0.1": 4, "10.0.0.2": 1, "10.0.0.4": 4}


def test_spark_rank_coordinates_and_missing_pyspark():
    from horovod_b200.spark.runner import _coordinates, run
    hosts = ["a", "b", "a", "c", "b", "a"]
    assert _coordinates(hosts, 0) == (0, 3, 0, 3)
    assert _coordinates(hosts, 2) == (1, 3, 0, 2)
    assert _coordinates(hosts, 4) == (1, 2, 1, 2)
    assert _coordinates(hosts, 5) == (2, 3, 0, 1)
    assert _coordinates(hosts, 3) == (0, 1, 2, 3)
    try:
        import pyspark  # noqa: F401
    except ImportError:
        with pytest.raises(ImportError, match="pyspark"):
            run(lambda: 0, num_proc=2)


def test_filesystem_store_layout_and_sync(tmp_path):
    from horovod_b200.spark import LocalStore, Store
    store = Store.create(str(tmp_path / "store"))
    assert isinstance(store, LocalStore) and os.path.isdir(store.prefix_path)
    assert store.get_train_data_path().endswith("intermediate_train_data")
    assert store.get_val_data_path(3).endswith("intermediate_val_data.3")
    run_id = "run_001"
    assert store.get_checkpoint_path(run_id) == os.path.join(store.get_run_path(run_id), "checkpoint")
    assert store.get_logs_path(run_id).endswith(os.path.join(run_id, "logs"))
    assert not store.exists(store.get_checkpoint_path(run_id))
    with store.get_local_output_dir_fn(run_id)() as local:
        with open(os.path.join(local, "checkpoint"), "wb") as f:
            f.write(b"weights")
        os.makedirs(os.path.join(local, "logs"))
        with open(os.path.join(local, "logs", "events.txt"), "w") as f:
            f.write("step 1")
        store.sync_fn(run_id)(local)
    assert not os.path.exists(local)
    assert store.read(store.get_checkpoint_path(run_id)) == b"weights"
    assert store.exists(os.path.join(store.get_logs_path(run_id), "events.txt"))
    remote = store.to_remote(run_id, None)
    assert remote.checkpoint_path == store.get_checkpoint_path(run_id) and callable(remote.sync)
    os.makedirs(store.get_train_data_path())
    assert not store.is_parquet_dataset(store.get_train_data_path())
    open(os.path.join(store.get_train_data_path(), "part-0.parquet"), "w").close()
    assert store.is_parquet_dataset(store.get_train_data_path())
    quiet = LocalStore(str(tmp_path / "q"), save_runs=False)
    assert quiet.get_checkpoint_path("r") is None and not quiet.saving_runs()
    with pytest.raises(ValueError):
        Store.create("hdfs://namenode/path")
