"""Launcher: argument/config/env mapping, host assignment maths, command
builders, process-tree control, RPC services, and end-to-end local runs.
Mirrors the reference's test/single/test_run.py, test_service.py and the
local part of test/integration/test_static_run.py."""
import io
import os
import sys
import threading
import time

import pytest

from horovod_b200.runner import launch, mpi_run, js_run, gloo_run
from horovod_b200.runner.common import config_parser, hosts, network, safe_shell_exec, secret
from horovod_b200.runner.common.settings import Settings
from horovod_b200.runner.util import cache as cache_mod

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_args_map_to_env():
    args = launch.parse_args(
        ["-np", "2", "--fusion-threshold-mb", "10", "--cycle-time-ms", "20",
         "--cache-capacity", "512", "--hierarchical-allreduce", "--hierarchical-allgather",
         "--autotune", "--autotune-log-file", "/tmp/a.csv", "--autotune-warmup-samples", "1",
         "--autotune-steps-per-sample", "5", "--autotune-bayes-opt-max-samples", "10",
         "--autotune-gaussian-process-noise", "0.2", "--timeline-filename", "/tmp/t.json",
         "--timeline-mark-cycles", "--no-stall-check", "--log-level", "INFO",
         "--log-hide-timestamp", "--gpu-backend", "nccl", "python", "train.py"])
    env = config_parser.set_env_from_args({}, args)
    assert env["HOROVOD_FUSION_THRESHOLD"] == str(10 * 1024 * 1024)
    assert env["HOROVOD_CYCLE_TIME"] == "20.0"
    assert env["HOROVOD_CACHE_CAPACITY"] == "512"
    assert env["HOROVOD_HIERARCHICAL_ALLREDUCE"] == "1"
    assert env["HOROVOD_HIERARCHICAL_ALLGATHER"] == "1"
    assert env["HOROVOD_AUTOTUNE"] == "1" and env["HOROVOD_AUTOTUNE_LOG"] == "/tmp/a.csv"
    assert env["HOROVOD_AUTOTUNE_WARMUP_SAMPLES"] == "1"
    assert env["HOROVOD_AUTOTUNE_STEPS_PER_SAMPLE"] == "5"
    assert env["HOROVOD_AUTOTUNE_BAYES_OPT_MAX_SAMPLES"] == "10"
    assert env["HOROVOD_AUTOTUNE_GAUSSIAN_PROCESS_NOISE"] == "0.2"
    assert env["HOROVOD_TIMELINE"] == "/tmp/t.json" and env["HOROVOD_TIMELINE_MARK_CYCLES"] == "1"
    assert env["HOROVOD_STALL_CHECK_DISABLE"] == "1"
    assert env["HOROVOD_LOG_LEVEL"] == "INFO" and env["HOROVOD_LOG_HIDE_TIME"] == "1"
    assert env["HOROVOD_GPU_BACKEND"] == "nccl"
    assert args.command == ["python", "train.py"]
    # the spellings of the timestamp and timeout options
    args = launch.parse_args(["-np", "2", "--gloo-timeout-seconds", "7",
                              "--log-without-timestamp", "--prefix-output-with-timestamp",
                              "python", "train.py"])
    env = config_parser.set_env_from_args({}, args)
    assert env["HOROVOD_GLOO_TIMEOUT_SECONDS"] == "7" and env["HOROVOD_LOG_HIDE_TIME"] == "1"
    assert args.prefix_output_with_timestamp
    args = launch.parse_args(["-np", "2", "--log-with-timestamp", "-prefix-timestamp",
                              "python", "train.py"])
    assert "HOROVOD_LOG_HIDE_TIME" not in config_parser.set_env_from_args({}, args)
    assert args.prefix_output_with_timestamp
    # library options (horovod/runner/launch.py:423-431)
    args = launch.parse_args(["-np", "2", "--mpi-threads-disable", "python", "train.py"])
    assert config_parser.set_env_from_args({}, args)["HOROVOD_MPI_THREADS_DISABLE"] == "1"
    args = launch.parse_args(["-np", "2", "--no-mpi-threads-disable", "python", "train.py"])
    assert "HOROVOD_MPI_THREADS_DISABLE" not in config_parser.set_env_from_args({}, args)


def test_config_file_loses_to_explicit_flags(tmp_path):
    cfg = tmp_path / "c.yaml"
    cfg.write_text("""
params:
  fusion_threshold_mb: 32
  cycle_time_ms: 7
  cache_capacity: 99
autotune:
  enabled: true
  warmup_samples: 2
timeline:
  filename: /tmp/from_cfg.json
stall_check:
  enabled: false
  warning_time_seconds: 5
logging:
  level: DEBUG
""")
    args = launch.parse_args(["-np", "2", "--config-file", str(cfg),
                              "--fusion-threshold-mb", "64", "x"])
    assert args.fusion_threshold_mb == 64      # flag wins
    assert args.cycle_time_ms == 7 and args.cache_capacity == 99
    assert args.autotune and args.autotune_warmup_samples == 2
    assert args.timeline_filename == "/tmp/from_cfg.json"
    assert args.no_stall_check and args.stall_check_warning_time_seconds == 5
    assert args.log_level == "DEBUG"
    with pytest.raises(ValueError):
        launch.parse_args(["-np", "2", "--cycle-time-ms", "-1", "x"])


def test_host_assignments():
    alloc = hosts.get_host_assignments(hosts.parse_hosts("a:2,b:3"), 4)
    assert [(s.hostname, s.rank, s.local_rank, s.cross_rank) for s in alloc] == [
        ("a", 0, 0, 0), ("a", 1, 1, 0), ("b", 2, 0, 1), ("b", 3, 1, 1), ("b", 4, 2, 0)]
    assert all(s.size == 5 for s in alloc)
    assert [s.local_size for s in alloc] == [2, 2, 3, 3, 3]
    assert [s.cross_size for s in alloc] == [2, 2, 2, 2, 1]
    capped = hosts.get_host_assignments(hosts.parse_hosts("a:2,b:3"), 2, max_np=3)
    assert len(capped) == 3 and capped[-1].hostname == "b"
    with pytest.raises(ValueError):
        hosts.get_host_assignments(hosts.parse_hosts("a:2"), 3)


def test_hostfile(tmp_path):
    f = tmp_path / "hosts"
    f.write_text("# comment\nnode1 slots=4\nnode2 slots=2\n\nnode3\n")
    assert hosts.parse_host_files(str(f)) == "node1:4,node2:2,node3:1"


def test_mpi_command_line(monkeypatch):
    monkeypatch.setattr(mpi_run, "_get_mpi_implementation", lambda env=None: mpi_run._OMPI_IMPL)
    flags, binding, impl = mpi_run._get_mpi_implementation_flags(False)
    s = Settings(hosts="h1:2,h2:2", num_proc=4, verbose=0, ssh_port=2222,
                 extra_mpi_args="--mca foo bar")
    line = mpi_run.build_mpi_command(s, ["eth0"], {"HOROVOD_FUSION_THRESHOLD": "1", "PATH": "/bin",
                                                   "IGNORED": "x"},
                                     ["python", "train.py"], flags, binding, impl, "10.0.0.1", 1234)
    assert line.startswith("mpirun --allow-run-as-root --tag-output -np 4 -H h1:2,h2:2")
    assert "-bind-to none -map-by slot" in line and "-mca pml ob1" in line
    assert '-mca plm_rsh_args "-p 2222"' in line
    assert "-mca btl_tcp_if_include eth0" in line and "-x NCCL_SOCKET_IFNAME=eth0" in line
    assert "-x HOROVOD_FUSION_THRESHOLD" in line and "IGNORED" not in line
    assert "--mca foo bar" in line
    assert line.endswith("horovod_b200.runner.mpi_worker 10.0.0.1 1234 python train.py")
    monkeypatch.setattr(mpi_run, "_get_mpi_implementation", lambda env=None: mpi_run._MISSING_IMPL)
    with pytest.raises(Exception, match="mpirun"):
        mpi_run.mpi_run(s, None, {}, ["true"])


def test_jsrun_rankfile(tmp_path, monkeypatch):
    monkeypatch.setenv("HOROVOD_LSF_GPUS_PER_HOST", "4")
    monkeypatch.setenv("HOROVOD_LSF_CORES_PER_HOST", "40")
    monkeypatch.setenv("HOROVOD_LSF_THREADS_PER_CORE", "4")
    s = Settings(hosts="n1:4,n2:4", num_proc=6)
    path = js_run.generate_jsrun_rankfile(s, str(tmp_path / "rf"))
    text = open(path).read()
    assert "rank: 0: { hostname: n1; cpu: {0-39} ; gpu: * ; mem: * }" in text
    assert "rank: 5: { hostname: n2; cpu: {40-79} ; gpu: * ; mem: * }" in text
    assert "rank: 6" not in text
    cmd = js_run.build_jsrun_command(s, path, {}, ["python", "t.py"], "1.2.3.4", 99)
    assert cmd.startswith("jsrun --erf_input") and cmd.endswith("1.2.3.4 99 python t.py")


def test_safe_shell_exec_output_and_kill():
    out = io.StringIO()
    code = safe_shell_exec.execute("echo hello; echo oops 1>&2; exit 3", stdout=out, stderr=out,
                                   index=5)
    assert code == 3
    assert "[5]<stdout>:hello" in out.getvalue() and "[5]<stderr>:oops" in out.getvalue()
    # an event kills the whole tree, including grandchildren
    ev = threading.Event()
    marker = "/tmp/hvd_b200_sse_%d" % os.getpid()
    t0 = time.time()
    threading.Timer(0.5, ev.set).start()
    code = safe_shell_exec.execute("(sleep 30; touch %s) & sleep 30" % marker, events=[ev])
    assert time.time() - t0 < 10 and code != 0
    time.sleep(0.3)
    assert not os.path.exists(marker)


def test_rpc_service_roundtrip_and_auth():
    key = secret.make_secret_key()

    class Echo(network.BasicService):
        def _handle(self, req, client_address):
            if isinstance(req, dict):
                return {"echo": req["v"] * 2}
            return super()._handle(req, client_address)

    svc = Echo("echo service", key)
    try:
        client = network.BasicClient("echo service", svc.addresses(), key, probe_timeout=5)
        results = []
        ts = [threading.Thread(target=lambda i=i: results.append(client._send({"v": i})["echo"]))
              for i in range(8)]
        [t.start() for t in ts]
        [t.join() for t in ts]
        assert sorted(results) == [0, 2, 4, 6, 8, 10, 12, 14]
        with pytest.raises(network.NoValidAddressesFound):
            network.BasicClient("echo service", svc.addresses(), secret.make_secret_key(),
                                probe_timeout=2, attempts=1)
        with pytest.raises(network.NoValidAddressesFound):
            network.BasicClient("other name", svc.addresses(), key, probe_timeout=2, attempts=1)
    finally:
        svc.shutdown()


def test_cache_expiry_and_parameter_change(tmp_path):
    c = cache_mod.Cache(str(tmp_path), 60, ("a",))
    c.put("k", True)
    assert cache_mod.Cache(str(tmp_path), 60, ("a",)).get("k") is True
    assert cache_mod.Cache(str(tmp_path), 60, ("b",)).get("k") is None
    assert cache_mod.Cache(str(tmp_path), 0, ("a",)).get("k") is None


def test_check_build(capsys):
    with pytest.raises(SystemExit):
        launch.parse_args(["--check-build"]) and launch.check_build(False)
    assert "NVLink symmetric-memory kernels" in capsys.readouterr().out


def _env():
    env = os.environ.copy()
    env["PYTHONPATH"] = ROOT + os.pathsep + env.get("PYTHONPATH", "")
    env["OMP_NUM_THREADS"] = "1"
    return env


def test_horovodrun_static_end_to_end(tmp_path):
    script = tmp_path / "train.py"
    script.write_text(
        "import torch, horovod_b200.torch as hvd\n"
        "hvd.init()\n"
        "x = hvd.allreduce(torch.ones(3) * (hvd.rank() + 1), op=hvd.Sum)\n"
        "print('RESULT', hvd.rank(), hvd.size(), hvd.local_rank(), x.tolist())\n"
        "hvd.shutdown()\n")
    outdir = tmp_path / "out"
    import subprocess
    res = subprocess.run([sys.executable, "-m", "horovod_b200.runner.launch", "-np", "3",
                          "--output-filename", str(outdir), sys.executable, str(script)],
                         env=_env(), cwd=ROOT, stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                         text=True, timeout=180)
    assert res.returncode == 0, res.stdout
    for r in range(3):
        text = (outdir / ("rank.%d" % r) / "stdout").read_text()
        assert "RESULT %d 3 %d [6.0, 6.0, 6.0]" % (r, r) in text
    # a failing rank fails the job and names itself
    bad = tmp_path / "bad.py"
    bad.write_text("import os, sys, time\n"
                   "if os.environ['HOROVOD_RANK'] == '1': sys.exit(7)\n"
                   "time.sleep(60)\n")
    res = subprocess.run([sys.executable, "-m", "horovod_b200.runner.launch", "-np", "2",
                          sys.executable, str(bad)], env=_env(), cwd=ROOT,
                         stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=120)
    assert res.returncode == 1
    assert "Process name: 1" in res.stdout and "Exit code: 7" in res.stdout


def _fn(scale):
    import torch
    import horovod_b200.torch as hvd
    hvd.init()
    out = hvd.allreduce(torch.ones(2) * hvd.rank(), op=hvd.Sum).tolist()
    r = hvd.rank()
    hvd.shutdown()
    return r * scale, out


def test_programmatic_run_returns_results_by_rank():
    import horovod_b200
    env = _env()
    # The function is pickled by reference: workers must be able to import
    # this module.
    env["PYTHONPATH"] = os.path.dirname(os.path.abspath(__file__)) + os.pathsep + env["PYTHONPATH"]
    res = horovod_b200.run(_fn, args=(10,), np=2, env=env)
    assert res == [(0, [1.0, 1.0]), (10, [1.0, 1.0])]


def test_nic_discovery_ring_on_loopback():
    """Three task services on this machine register with the driver, probe the
    next one in the ring and report; loopback must be among the common
    interfaces (parity: test/single/test_run.py network/driver-service tests)."""
    import threading
    from horovod_b200.runner.common import secret
    from horovod_b200.runner.driver import driver_service as ds
    key = secret.make_secret_key()
    n = 3
    driver = ds.HorovodRunDriverService(n, key)
    try:
        threads = [threading.Thread(target=ds.task_fn, daemon=True,
                                    args=(i, n, driver.addresses(), key, None, 20, "host%d" % i))
                   for i in range(n)]
        for t in threads:
            t.start()
        common = ds._run_probe(driver, key, n, start_timeout_s=20)
        for t in threads:
            t.join(timeout=10)
        assert "lo" in common
        assert all(not t.is_alive() for t in threads)
        assert sorted(driver.task_host_hash_indices()) == ["host0", "host1", "host2"]
    finally:
        driver.shutdown()
    # a single-host job needs no probing
    assert ds.get_common_interfaces(["localhost"]) == {"lo"}


def test_rpc_rejects_wrong_key():
    from horovod_b200.runner.common import network, secret
    service = network.BasicService("svc", secret.make_secret_key())
    try:
        with pytest.raises(network.NoValidAddressesFound):
            network.BasicClient("svc", service.addresses(), secret.make_secret_key(),
                                probe_timeout=2, attempts=1)
    finally:
        service.shutdown()


def test_lsf_hosts(monkeypatch):
    from horovod_b200.runner.util.lsf import LSFUtils
    monkeypatch.setenv("LSB_JOBID", "1")
    monkeypatch.setenv("LSB_MCPU_HOSTS", "batch1 1 node1 42 node2 42")
    monkeypatch.setenv("CUDA_VISIBLE_DEVICES", "0,1,2,3")
    assert LSFUtils.using_lsf()
    assert LSFUtils.get_compute_hosts() == ["node1", "node2"]
    assert LSFUtils.get_num_processes() == 8


def test_rpc_service_handles_requests_concurrently_and_shuts_down_mid_request():
    """Parity: test/single/test_service.py (concurrent requests, shutdown
    while a request is being served)."""
    from horovod_b200.runner.common import network, secret

    class Sleep:
        def __init__(self, seconds):
            self.seconds = seconds

    class SleepService(network.BasicService):
        def __init__(self, key):
            super().__init__("sleeper", key)
            self.active = 0
            self.max_active = 0
            self._lock = threading.Lock()

        def _handle(self, req, client_address):
            if isinstance(req, Sleep):
                with self._lock:
                    self.active += 1
                    self.max_active = max(self.max_active, self.active)
                time.sleep(req.seconds)
                with self._lock:
                    self.active -= 1
                return network.AckResponse()
            return super()._handle(req, client_address)

    key = secret.make_secret_key()
    service = SleepService(key)
    try:
        client = network.BasicClient("sleeper", {"lo": [("127.0.0.1", service.get_port())]}, key)
        t0 = time.time()
        threads = [threading.Thread(target=client._send, args=(Sleep(0.5),)) for _ in range(4)]
        for t in threads:
            t.start()
        for t in threads:
            t.join(timeout=10)
        elapsed = time.time() - t0
        assert service.max_active >= 2, "requests were serialised"
        assert elapsed < 1.6, elapsed
        # shutdown while a request is in flight: shutdown() returns, the client
        # gets its answer or a connection error, nothing hangs
        result = {}

        def slow():
            try:
                client._send(Sleep(1.0))
                result["outcome"] = "answered"
            except Exception as e:  # noqa: BLE001
                result["outcome"] = type(e).__name__
        t = threading.Thread(target=slow)
        t.start()
        time.sleep(0.2)
        t1 = time.time()
        service.shutdown()
        assert time.time() - t1 < 6
        t.join(timeout=15)
        assert not t.is_alive() and "outcome" in result
    finally:
        try:
            service.shutdown()
        except Exception:  # noqa: BLE001
            pass


def test_safe_shell_exec_kills_the_whole_process_tree_on_event():
    """Parity: test/single/test_run.py safe_shell_exec tests (the shell's
    children must die with it)."""
    import subprocess
    event = threading.Event()
    marker = "hvd_sleep_marker_%d" % os.getpid()
    out = io.StringIO()
    cmd = "bash -c 'echo started; sleep 300 & wait' # %s" % marker
    t = threading.Thread(target=lambda: safe_shell_exec.execute(cmd, stdout=out, events=[event]))
    t0 = time.time()
    t.start()
    time.sleep(1.0)
    event.set()
    t.join(timeout=20)
    assert not t.is_alive() and time.time() - t0 < 15
    assert "started" in out.getvalue()
    time.sleep(0.5)
    ps = subprocess.run(["ps", "-eo", "args"], capture_output=True, text=True).stdout
    assert not [line for line in ps.splitlines() if marker in line and "ps -eo" not in line]


def test_output_filename_writes_per_rank_files(tmp_path):
    """Parity: --output-filename / --prefix-timestamp (runner/gloo_run.py:150-163)."""
    import subprocess
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out_dir = str(tmp_path / "logs")
    env = dict(os.environ, PYTHONPATH=root + os.pathsep + os.environ.get("PYTHONPATH", ""))
    proc = subprocess.run(
        [sys.executable, "-m", "horovod_b200.runner.launch", "-np", "2", "--output-filename",
         out_dir, "--prefix-timestamp", sys.executable, "-c",
         "import horovod_b200.torch as hvd; hvd.init(); print('hello from', hvd.rank())"],
        cwd=root, env=env, capture_output=True, text=True, timeout=120)
    assert proc.returncode == 0, proc.stderr[-1500:]
    for r in range(2):
        text = open(os.path.join(out_dir, "rank.%d" % r, "stdout")).read()
        assert "[%d]<stdout>:hello from %d" % (r, r) in text
        assert text.split("[")[0].strip(), "timestamp prefix missing"
        assert os.path.exists(os.path.join(out_dir, "rank.%d" % r, "stderr"))


def test_small_launcher_utilities(monkeypatch):
    """codec, env, tiny_shell_exec, http_client, util.network / remote /
    streams (parity: horovod/runner/common/util/{codec,env,tiny_shell_exec}.py,
    horovod/runner/http/http_client.py, horovod/runner/util/{network,remote,streams}.py)."""
    import threading
    from horovod_b200.runner.common import codec, env as env_util, tiny_shell_exec
    from horovod_b200.runner.http import http_client
    from horovod_b200.runner.http.http_server import RendezvousServer
    from horovod_b200.runner.util import network, remote, streams

    obj = {"fn": lambda x: x + 1, "n": [1, 2, 3]}
    text = codec.dumps_base64(obj)
    assert isinstance(text, str) and codec.loads_base64(text)["fn"](2) == 3
    assert isinstance(codec.dumps_base64(obj, to_ascii=False), bytes)

    assert env_util.is_exportable("PATH") and not env_util.is_exportable("BASH_FUNC_x%%")
    assert not env_util.is_exportable("_HOROVOD_SECRET_KEY")
    for name in ("HOROVOD_RANK", "HOROVOD_SIZE", "OMPI_COMM_WORLD_RANK", "OMPI_COMM_WORLD_SIZE",
                 "PMI_RANK", "PMI_SIZE", "OMPI_MCA_plm_rsh_agent"):
        monkeypatch.delenv(name, raising=False)
    assert env_util.get_env_rank_and_size() == (0, 1)
    monkeypatch.setenv("OMPI_COMM_WORLD_RANK", "3")
    with pytest.raises(RuntimeError):
        env_util.get_env_rank_and_size()
    monkeypatch.setenv("OMPI_COMM_WORLD_SIZE", "8")
    assert env_util.get_env_rank_and_size() == (3, 8)

    out, code = tiny_shell_exec.execute("echo hello; echo oops 1>&2; exit 3")
    assert code == 3 and "hello" in out and "oops" in out

    server = RendezvousServer(0)
    port = server.start()
    try:
        http_client.put_data_into_kvstore("127.0.0.1", port, "scope", "key", {"a": (1, 2)})
        assert http_client.read_data_from_kvstore("127.0.0.1", port, "scope", "key") == {"a": (1, 2)}
        with pytest.raises(RuntimeError):
            http_client.read_data_from_kvstore("127.0.0.1", port, "scope", "absent")
    finally:
        server.stop()

    assert "127.0.0.1" in network.get_local_host_addresses()
    assert network.filter_local_addresses(["127.0.0.1", "no-such-host.invalid"]) == \
        ["no-such-host.invalid"]
    assert network.resolve_host_address("no-such-host.invalid") is None

    cmd = remote.get_ssh_command("ls", "h1", port=2222, identity_file="/k", timeout_s=5)
    assert cmd.startswith("ssh -o PasswordAuthentication=no") and cmd.endswith(" ls")
    assert " h1 " in cmd and "-p 2222" in cmd and "-i /k" in cmd and "ConnectTimeout=5" in cmd
    monkeypatch.setenv("OMPI_MCA_plm_rsh_agent", env_util.KUBEFLOW_MPI_EXEC)
    assert remote.get_remote_command("ls", "h1") == "/etc/mpi/kubexec.sh h1 ls"

    pipe = streams.Pipe()
    got = []
    reader = threading.Thread(target=lambda: [got.append(pipe.read(3)) for _ in range(3)])
    reader.start()
    pipe.write("abcde")
    pipe.write(b"xy")
    reader.join(10)
    assert got == ["abc", "de", b"xy"]
    pipe.close()
    assert pipe.read() is None
    with pytest.raises(RuntimeError):
        pipe.write("late")


def test_mpi_flavour_queries_and_host_helpers(monkeypatch):
    from horovod_b200.runner import js_run, mpi_run
    banners = {"Open MPI": "mpirun (Open MPI) 4.1.4", "IBM Spectrum MPI": "IBM Spectrum MPI 10.3",
               "MPICH": "HYDRA build details: MPICH 4.0", "Intel": "Intel(R) MPI Library 2021.6"}
    answers = {}
    for key, banner in banners.items():
        monkeypatch.setattr(mpi_run, "_exec", lambda command, banner=banner: (banner, 0))
        answers[key] = (mpi_run.is_open_mpi(), mpi_run.is_spectrum_mpi(), mpi_run.is_mpich(),
                        mpi_run.is_intel_mpi(), mpi_run.mpi_available())
    assert answers == {"Open MPI": (True, False, False, False, True),
                       "IBM Spectrum MPI": (False, True, False, False, True),
                       "MPICH": (False, False, True, False, True),
                       "Intel": (False, False, False, True, True)}
    monkeypatch.setattr(mpi_run, "_exec", lambda command: (None, 1))   # no mpirun on PATH
    assert not mpi_run.mpi_available() and not mpi_run.is_open_mpi()
    assert isinstance(js_run.is_jsrun_installed(), bool)
    assert hosts.parse_hosts_and_slots("a:2,b,c:4") == (["a", "b", "c"], {"a": 2, "b": 1, "c": 4})
