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
    with pytest.raises(RuntimeError, match="(?i)hdfs"):  # no Hadoop client on this machine
        Store.create("hdfs://namenode/path")
    with pytest.raises(ValueError):
        Store.create("gs://bucket/path")


def test_ray_placement_plans():
    from horovod_b200.ray import plan_colocated, plan_packed
    p = plan_packed(3, cpus_per_worker=2, gpus_per_worker=1)
    assert p.strategy == "PACK" and p.bundles == [{"CPU": 2, "GPU": 1}] * 3
    assert p.bundle_of_rank == [0, 1, 2] and p.num_workers == 3
    c = plan_colocated(2, 4, cpus_per_worker=1, gpus_per_worker=1)
    assert c.strategy == "STRICT_SPREAD" and c.bundles == [{"CPU": 4, "GPU": 4}] * 2
    assert c.bundle_of_rank == [0, 0, 0, 0, 1, 1, 1, 1]
    assert plan_packed(1).bundles == [{"CPU": 1}]  # no GPU key without GPUs
    with pytest.raises(ValueError):
        plan_colocated(0, 2)


class _FakeRef:
    def __init__(self, value=None, error=None):
        self.value, self.error = value, error


def _fake_ray(node_ids, nodes=None):
    """A stand-in ``ray`` module that runs actor methods and tasks in this
    process: enough to drive the executors' orchestration. Actor r reports
    node_ids[r]; placement requests and task options are recorded."""
    ray = types.ModuleType("ray")
    ray.calls = {"options": [], "groups": [], "removed": 0, "killed": 0, "tasks": []}
    state = {"next_actor": 0}

    class Method:
        def __init__(self, bound):
            self.bound = bound

        def remote(self, *a, **kw):
            try:
                return _FakeRef(self.bound(*a, **kw))
            except Exception as e:  # surfaces at ray.get, as in Ray
                return _FakeRef(error=e)

    class Actor:
        def __init__(self, obj, index):
            self._obj, self._index = obj, index

        def __getattr__(self, name):
            if name == "node_id":
                return Method(lambda: node_ids[self._index])
            return Method(getattr(self._obj, name))

    class RemoteClass:
        def __init__(self, cls):
            self.cls = cls

        def options(self, **opts):
            ray.calls["options"].append(opts)
            return self

        def remote(self, *a, **kw):
            index = state["next_actor"]
            state["next_actor"] += 1
            return Actor(self.cls(*a, **kw), index)

    class RemoteFunction:
        def __init__(self, fn):
            self.fn = fn

        def options(self, **opts):
            ray.calls["tasks"].append(opts)
            return self

        def remote(self, *a, **kw):
            return Method(self.fn).remote(*a, **kw)

    def remote(target):
        return RemoteClass(target) if isinstance(target, type) else RemoteFunction(target)

    def get(refs):
        def one(r):
            if r.error is not None:
                raise r.error
            return r.value
        return [one(r) for r in refs] if isinstance(refs, list) else one(refs)

    ray.remote = remote
    ray.get = get
    ray.wait = lambda refs, timeout=None: (list(refs), [])
    ray.kill = lambda actor: ray.calls.__setitem__("killed", ray.calls["killed"] + 1)
    ray.cancel = lambda ref, force=False: None
    ray.nodes = lambda: nodes or []
    ray.available_resources = lambda: {}
    util = types.ModuleType("ray.util")
    util.get_node_ip_address = lambda: "127.0.0.1"

    class Group:
        def ready(self):
            return _FakeRef(True)

    def placement_group(bundles, strategy="PACK"):
        ray.calls["groups"].append((bundles, strategy))
        return Group()

    def remove_placement_group(group):
        ray.calls["removed"] += 1

    util.placement_group = placement_group
    util.remove_placement_group = remove_placement_group
    ray.util = util
    return ray, util


def test_ray_executor_orchestration_with_a_stand_in_ray(monkeypatch):
    """start() reserves the placement group, creates one actor per rank in its
    bundle, hands every rank its coordinates and the rendezvous address;
    run()/execute() reach every actor; shutdown() releases everything."""
    from horovod_b200.ray import RayExecutor
    ray, util = _fake_ray(["n0", "n0", "n1", "n1"])
    monkeypatch.setitem(sys.modules, "ray", ray)
    monkeypatch.setitem(sys.modules, "ray.util", util)
    saved = dict(os.environ)
    ex = RayExecutor(num_hosts=2, num_workers_per_host=2, use_gpu=True)
    try:
        class Exe:
            def __init__(self, base):
                self.base = base
        ex.start(executable_cls=Exe, executable_args=[10], extra_env_vars={"MY_FLAG": "1"})
        assert ray.calls["groups"] == [([{"CPU": 2, "GPU": 2}] * 2, "STRICT_SPREAD")]
        assert [o["placement_group_bundle_index"] for o in ray.calls["options"]] == [0, 0, 1, 1]
        assert all(o["num_gpus"] == 1 and o["num_cpus"] == 1 for o in ray.calls["options"])
        # The stand-in runs every actor in this process, so the environment
        # seen afterwards is that of the last rank.
        env = ex.run(lambda: dict(os.environ))[3]
        assert (env["HOROVOD_RANK"], env["HOROVOD_SIZE"], env["HOROVOD_LOCAL_RANK"],
                env["HOROVOD_LOCAL_SIZE"], env["HOROVOD_CROSS_RANK"],
                env["HOROVOD_CROSS_SIZE"]) == ("3", "4", "1", "2", "1", "2")
        assert env["MY_FLAG"] == "1" and env["HOROVOD_GLOO_RENDEZVOUS_ADDR"] == "127.0.0.1"
        assert ex.execute(lambda exe: exe.base + 1) == [11] * 4
        assert ex.execute_single(lambda exe: exe.base) == 10
        assert ex.run(lambda a, b=0: a + b, args=[1], kwargs={"b": 2}) == [3] * 4
    finally:
        ex.shutdown()
        os.environ.clear()
        os.environ.update(saved)
    assert ray.calls["killed"] == 4 and ray.calls["removed"] == 1 and ex.coordinator is None


def test_elastic_ray_executor_runs_a_round_with_a_stand_in_ray(monkeypatch):
    """The elastic executor discovers the cluster's slots, starts one task per
    slot pinned to its node with that slot's coordinates, and returns the
    workers' values by rank."""
    from horovod_b200.ray import ElasticRayExecutor
    nodes = [{"alive": True, "NodeManagerAddress": "10.0.0.1", "Resources": {"CPU": 4, "GPU": 2}},
             {"alive": True, "NodeManagerAddress": "10.0.0.2", "Resources": {"CPU": 4, "GPU": 2}}]
    ray, util = _fake_ray([], nodes)
    monkeypatch.setitem(sys.modules, "ray", ray)
    monkeypatch.setitem(sys.modules, "ray.util", util)
    saved = dict(os.environ)
    try:
        with pytest.raises(ValueError):
            ElasticRayExecutor(ElasticRayExecutor.create_settings(), gpus_per_slot=1)
        settings = ElasticRayExecutor.create_settings(min_np=4, max_np=4, elastic_timeout=20,
                                                      verbose=0)
        ex = ElasticRayExecutor(settings, use_gpu=True, cpus_per_slot=2,
                                env_vars={"MY_FLAG": "1"})
        ex.start(advertise_ip="127.0.0.1")

        def worker():
            return (int(os.environ["HOROVOD_RANK"]), os.environ["HOROVOD_HOSTNAME"],
                    os.environ["HOROVOD_ELASTIC"], os.environ["MY_FLAG"],
                    os.environ["HOROVOD_SIZE"])
        results = ex.run(worker)
        assert [r[0] for r in results] == [0, 1, 2, 3]
        assert sorted(r[1] for r in results) == ["10.0.0.1"] * 2 + ["10.0.0.2"] * 2
        assert all(r[2:] == ("1", "1", "4") for r in results)
        pinned = sorted(list(t["resources"])[0] for t in ray.calls["tasks"])
        assert pinned == ["node:10.0.0.1"] * 2 + ["node:10.0.0.2"] * 2
        assert all(t["num_gpus"] == 1 and t["num_cpus"] == 2 for t in ray.calls["tasks"])
    finally:
        os.environ.clear()
        os.environ.update(saved)


def test_spark_run_with_a_stand_in_pyspark(monkeypatch):
    """run() starts one barrier task per rank; every task derives its
    coordinates from the hosts gathered through the barrier context, finds the
    rendezvous server of the driver in its environment, and the results come
    back ordered by rank. The stand-in runs the tasks one after the other in
    this process, in reverse partition order."""
    import horovod_b200.spark.task
    from horovod_b200.spark.runner import run
    hosts = ["a", "b", "a", "b"]
    current = {"partition": None}
    pyspark = types.ModuleType("pyspark")

    class BarrierTaskContext:
        @staticmethod
        def get():
            return BarrierTaskContext()

        def allGather(self, message):
            return list(hosts)

        def partitionId(self):
            return current["partition"]

        def resources(self):
            # Spark's resource scheduling: one GPU address per task
            return {"gpu": types.SimpleNamespace(addresses=[str(current["partition"] + 4)])}

    class RDD:
        def __init__(self, n):
            self.n = n
            self.barrier_used = False

        def barrier(self):
            self.barrier_used = True
            return self

        def mapPartitionsWithIndex(self, task):
            self.task = task
            return self

        def collect(self):
            assert self.barrier_used
            out = []
            for index in reversed(range(self.n)):
                current["partition"] = index
                out.extend(self.task(index, iter([index])))
            return out

    class SparkContext:
        _active_spark_context = None
        defaultParallelism = 4

        def range(self, start, numSlices=None):
            return RDD(numSlices)

    pyspark.BarrierTaskContext = BarrierTaskContext
    pyspark.SparkContext = SparkContext
    monkeypatch.setitem(sys.modules, "pyspark", pyspark)
    with pytest.raises(Exception, match="SparkContext"):
        run(lambda: 0, num_proc=2)
    SparkContext._active_spark_context = SparkContext()
    saved = dict(os.environ)
    try:
        def fn(tag):
            e = os.environ
            return (tag, int(e["HOROVOD_RANK"]), int(e["HOROVOD_SIZE"]),
                    int(e["HOROVOD_LOCAL_RANK"]), int(e["HOROVOD_LOCAL_SIZE"]),
                    int(e["HOROVOD_CROSS_RANK"]), int(e["HOROVOD_CROSS_SIZE"]),
                    e["HOROVOD_HOSTNAME"], int(e["HOROVOD_GLOO_RENDEZVOUS_PORT"]) > 0, e["EXTRA"],
                    horovod_b200.spark.task.get_available_devices())
        with pytest.raises(ValueError, match="MPI"):
            run(fn, use_mpi=True)
        results = run(fn, args=("t",), env={"EXTRA": "overridden"}, extra_env={"EXTRA": "x"},
                      use_gloo=True, nics=["eth7"], verbose=0)  # num_proc inferred
        assert os.environ["HOROVOD_GLOO_IFACE"] == "eth7"
    finally:
        os.environ.clear()
        os.environ.update(saved)
    assert results == [("t", 0, 4, 0, 2, 0, 2, "a", True, "x", ["4"]),
                       ("t", 1, 4, 0, 2, 1, 2, "b", True, "x", ["5"]),
                       ("t", 2, 4, 1, 2, 0, 2, "a", True, "x", ["6"]),
                       ("t", 3, 4, 1, 2, 1, 2, "b", True, "x", ["7"])]
    horovod_b200.spark.task.set_resources(None)
    assert horovod_b200.spark.task.get_available_devices() == []


def test_spark_run_gives_up_when_the_tasks_do_not_start(monkeypatch):
    """A cluster without room for num_proc simultaneous tasks never starts the
    barrier stage: run() cancels its job group after start_timeout and says
    what to check."""
    import threading
    from horovod_b200.spark.runner import run
    released = threading.Event()
    cancelled = []
    pyspark = types.ModuleType("pyspark")

    class RDD:
        def barrier(self):
            return self

        def mapPartitionsWithIndex(self, task):
            return self

        def collect(self):
            released.wait(10)  # the scheduler never finds the slots
            raise RuntimeError("job group cancelled")

    class SparkContext:
        _active_spark_context = None
        defaultParallelism = 2

        def range(self, start, numSlices=None):
            return RDD()

        def setJobGroup(self, group, description, interruptOnCancel=False):
            self.group = group

        def cancelJobGroup(self, group):
            cancelled.append(group == self.group)
            released.set()

    pyspark.BarrierTaskContext = object
    pyspark.SparkContext = SparkContext
    SparkContext._active_spark_context = SparkContext()
    monkeypatch.setitem(sys.modules, "pyspark", pyspark)
    monkeypatch.setenv("HOROVOD_SPARK_START_TIMEOUT", "1")
    with pytest.raises(Exception, match="enough resources to run all 2 processes"):
        run(lambda: 0, verbose=0)
    assert cancelled == [True]


def test_spark_run_elastic_with_tasks_as_child_processes(monkeypatch):
    """run_elastic() against a stand-in pyspark whose stage runs every task in
    a forked child process: the tasks register with the coordinator over the
    signed RPC, the elastic driver sees them as slots of one host, hands each a
    slot's environment, and the values the function returned come back ordered
    by rank; afterwards every task is told that the job is over."""
    import multiprocessing as mp
    from horovod_b200.spark import run_elastic
    pyspark = types.ModuleType("pyspark")

    class RDD:
        def __init__(self, n):
            self.n = n

        def mapPartitionsWithIndex(self, task):
            self.task = task
            return self

        def collect(self):
            ctx = mp.get_context("fork")
            procs = [ctx.Process(target=lambda i=i: list(self.task(i, iter([i]))))
                     for i in range(self.n)]
            for p in procs:
                p.start()
            for p in procs:
                p.join(120)
            assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
            return list(range(self.n))

    class SparkContext:
        _active_spark_context = None
        defaultParallelism = 3

        def range(self, start, numSlices=None):
            return RDD(numSlices)

    pyspark.SparkContext = SparkContext
    monkeypatch.setitem(sys.modules, "pyspark", pyspark)
    with pytest.raises(Exception, match="SparkContext"):
        run_elastic(lambda: 0, num_proc=2)
    SparkContext._active_spark_context = SparkContext()
    with pytest.raises(ValueError):
        run_elastic(lambda: 0, num_proc=2, min_np=3, max_np=4)

    def fn(tag):
        e = os.environ
        return (tag, int(e["HOROVOD_RANK"]), int(e["HOROVOD_SIZE"]), e["HOROVOD_ELASTIC"],
                e["EXTRA"], int(e["HOROVOD_GLOO_RENDEZVOUS_PORT"]) > 0)

    results = run_elastic(fn, args=("t",), num_proc=3, min_np=2, max_np=3, env={"EXTRA": "x"},
                          elastic_timeout=30, verbose=0)
    assert results == [("t", r, 3, "1", "x", True) for r in range(3)]


def test_dbfs_and_arrow_filesystem_stores(tmp_path):
    """dbfs:/ paths map onto the local DBFS mount; the same store layout works
    over a pyarrow filesystem (what the HDFS store is built on); hdfs:// URLs
    without a Hadoop client fail with a message that names the cause."""
    from horovod_b200.spark import ArrowFilesystemStore, DBFSLocalStore, HDFSStore, Store
    root = str(tmp_path / "mount")
    store = DBFSLocalStore("dbfs:/ml/exp", root=root)
    assert store.prefix_path == root + "/ml/exp" and os.path.isdir(store.prefix_path)
    assert DBFSLocalStore.matches("dbfs:/x") and DBFSLocalStore.matches("/dbfs/x")
    assert not DBFSLocalStore.matches("/data/x")
    assert store.normalize("dbfs:///a/b") == root + "/a/b"
    assert store.normalize("/dbfs/a/b") == root + "/a/b"
    ckpt = store.get_checkpoint_path("r1")
    assert ckpt == root + "/ml/exp/runs/r1/checkpoint"
    with store.get_local_output_dir_fn("r1")() as local:
        with open(os.path.join(local, "checkpoint"), "wb") as f:
            f.write(b"w")
        store.sync_fn("r1")(local)
    assert store.exists("dbfs:/ml/exp/runs/r1/checkpoint") and store.read(ckpt) == b"w"

    fs = pytest.importorskip("pyarrow.fs")
    base = str(tmp_path / "arrow")
    os.makedirs(base)
    arrow = ArrowFilesystemStore(fs.SubTreeFileSystem(base, fs.LocalFileSystem()), "exp")
    assert os.path.isdir(os.path.join(base, "exp"))
    assert not arrow.exists(arrow.get_checkpoint_path("r2"))
    with arrow.get_local_output_dir_fn("r2")() as local:
        os.makedirs(os.path.join(local, "logs"))
        with open(os.path.join(local, "checkpoint"), "wb") as f:
            f.write(b"weights")
        with open(os.path.join(local, "logs", "e.txt"), "w") as f:
            f.write("step 1")
        arrow.sync_fn("r2")(local)
    assert arrow.read(arrow.get_checkpoint_path("r2")) == b"weights"
    assert arrow.exists(arrow.get_logs_path("r2") + "/e.txt")
    arrow.write_text(arrow.get_train_data_path() + "/part-0.parquet", "")
    assert arrow.is_parquet_dataset(arrow.get_train_data_path())
    assert not arrow.is_parquet_dataset(arrow.get_val_data_path())
    assert callable(arrow.to_remote("r2", None).sync)

    with pytest.raises((RuntimeError, OSError), match="(?i)hdfs"):
        HDFSStore("hdfs://namenode:8020/x")
    with pytest.raises(ValueError):
        Store.create("s3://bucket/x")
    assert isinstance(Store.create("dbfs:/q", root=root), DBFSLocalStore)
