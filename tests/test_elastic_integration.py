"""End-to-end elastic runs with real worker processes on CPU: "localhost" and
"127.0.0.1" act as two hosts of one box (as in the reference's
test/integration/elastic_common.py). Failures are injected on the host side
only: a worker process exits, or the discovery output changes."""
import json
import os
import stat
import sys

import pytest

from horovod_b200.runner import gloo_run
from horovod_b200.runner.common.settings import ElasticSettings
from horovod_b200.runner.common.timeout import Timeout
from horovod_b200.runner.elastic import discovery, driver as driver_mod

HERE = os.path.dirname(os.path.abspath(__file__))
SCRIPT = os.path.join(HERE, "data", "elastic_train.py")


def _settings(disc, np, min_np, max_np, reset_limit=None):
    return ElasticSettings(discovery=disc, min_np=min_np, max_np=max_np, elastic_timeout=60,
                           reset_limit=reset_limit, num_proc=np, verbose=0,
                           start_timeout=Timeout(60, "timed out: {activity}"))


def _env():
    env = os.environ.copy()
    env["PYTHONPATH"] = os.path.dirname(HERE) + os.pathsep + env.get("PYTHONPATH", "")
    env["HOROVOD_GLOO_TIMEOUT_SECONDS"] = "10"
    env["OMP_NUM_THREADS"] = "1"
    return env


def _read(log):
    with open(log) as f:
        return [json.loads(line) for line in f if line.strip()]


@pytest.fixture(autouse=True)
def fast_discovery(monkeypatch):
    monkeypatch.setattr(driver_mod, "DISCOVER_HOSTS_FREQUENCY_SECS", 0.2)


def test_hosts_added_grows_the_job(tmp_path):
    log = str(tmp_path / "log.jsonl")
    # The discovery script offers a second host once two epochs are logged.
    script = tmp_path / "discover.sh"
    script.write_text("#!/bin/bash\necho localhost:2\n"
                      "if [ -f %s ] && [ $(wc -l < %s) -ge 4 ]; then echo 127.0.0.1:2; fi\n"
                      % (log, log))
    script.chmod(script.stat().st_mode | stat.S_IEXEC)
    disc = discovery.HostDiscoveryScript(str(script), slots=2)
    settings = _settings(disc, np=2, min_np=2, max_np=4)
    gloo_run.launch_gloo_elastic([sys.executable, SCRIPT, "--log", log, "--epochs", "8"],
                                 gloo_run._exec_slot, settings, _env(), None)
    rows = _read(log)
    sizes = {r["epoch"]: r["size"] for r in rows}
    assert sizes[0] == 2
    assert sizes[7] == 4, sizes
    # every epoch was completed exactly once per participating rank
    for e in range(8):
        ranks = sorted(r["rank"] for r in rows if r["epoch"] == e)
        assert ranks == list(range(sizes[e])), (e, ranks)


def test_worker_failure_blacklists_host_and_job_continues(tmp_path):
    log = str(tmp_path / "log.jsonl")
    disc = discovery.FixedHosts({"localhost": 2, "127.0.0.1": 2})
    settings = _settings(disc, np=4, min_np=2, max_np=4)
    gloo_run.launch_gloo_elastic(
        [sys.executable, SCRIPT, "--log", log, "--epochs", "5", "--exit-at", "2:127.0.0.1:0"],
        gloo_run._exec_slot, settings, _env(), None)
    rows = _read(log)
    sizes = {}
    for r in rows:
        sizes.setdefault(r["epoch"], set()).add(r["size"])
    assert sizes[0] == {4}
    assert sizes[4] == {2}, sizes
    assert all(r["host"] == "localhost" for r in rows if r["epoch"] == 4)


def test_reset_limit_stops_the_job(tmp_path):
    log = str(tmp_path / "log.jsonl")
    disc = discovery.FixedHosts({"localhost": 2, "127.0.0.1": 2})
    # No reset allowed: the first failure ends the job.
    settings = _settings(disc, np=4, min_np=2, max_np=4, reset_limit=0)
    with pytest.raises(RuntimeError, match="reset limit"):
        gloo_run.launch_gloo_elastic(
            [sys.executable, SCRIPT, "--log", log, "--epochs", "5", "--exit-at",
             "1:127.0.0.1:1"],
            gloo_run._exec_slot, settings, _env(), None)


def test_elastic_mnist_example_takes_on_a_second_host_mid_training(tmp_path, capfd):
    """examples/pytorch_mnist_elastic.py under the elastic driver: a second
    "host" appears some seconds into the run (possibly before rank 0 listens
    for host changes: the driver then tells it as soon as it does); the job
    grows from 1 to 2 ranks at a commit, goes on from there (ElasticSampler
    hands out what is left of the epoch; the new worker takes over rank 0's
    weights) and reports every epoch exactly once."""
    import re
    import time
    example = os.path.join(os.path.dirname(HERE), "examples", "pytorch_mnist_elastic.py")
    script = tmp_path / "discover.sh"
    script.write_text("#!/bin/bash\necho localhost:1\n"
                      "if [ $(( $(date +%%s) - %d )) -ge 9 ]; then echo 127.0.0.1:1; fi\n"
                      % int(time.time()))
    script.chmod(script.stat().st_mode | stat.S_IEXEC)
    disc = discovery.HostDiscoveryScript(str(script), slots=1)
    settings = _settings(disc, np=1, min_np=1, max_np=2)
    gloo_run.launch_gloo_elastic(
        [sys.executable, example, "--epochs", "40", "--samples", "2048", "--batch-size", "32",
         "--batches-per-commit", "4", "--no-cuda"],
        gloo_run._exec_slot, settings, _env(), None)
    out = capfd.readouterr().out
    rows = re.findall(r"epoch (\d+): loss ([0-9.]+) accuracy ([0-9.]+) on (\d) rank\(s\)", out)
    assert [int(r[0]) for r in rows] == list(range(40)), out[-2000:]
    ranks = [int(r[3]) for r in rows]
    assert ranks[-1] == 2 and ranks == sorted(ranks), ranks
    assert float(rows[-1][2]) > 0.9, rows[-1]   # still converges across the change


@pytest.mark.parametrize("dying_rank", [1, 0])
def test_elastic_mnist_example_survives_a_worker_that_dies_mid_epoch(tmp_path, capfd, dying_rank):
    """The same example, with one line added that makes one worker (rank 1, or
    rank 0, the coordinator) exit in the middle of epoch 1 (a host-side failure): the
    survivor's next collective fails, it rolls back to its last commit
    (weights, optimizer, sampler progress, batch counter), re-forms the job
    alone and finishes every epoch exactly once."""
    import re
    example = os.path.join(os.path.dirname(HERE), "examples", "pytorch_mnist_elastic.py")
    source = open(example).read()
    hook = "            optimizer.zero_grad()\n"
    assert source.count(hook) == 1
    marker = str(tmp_path / "died")
    dying = source.replace(hook, hook + (
        "            import os\n"
        "            if state.epoch == 1 and idx == 5 and hvd.rank() == %d and not os.path.exists(%r):\n"
        "                open(%r, 'w').close()\n"
        "                os._exit(1)\n" % (dying_rank, marker, marker)), 1)
    script = tmp_path / "mnist_dying.py"
    script.write_text(dying)
    disc = discovery.FixedHosts({"localhost": 1, "127.0.0.1": 1})
    settings = _settings(disc, np=2, min_np=1, max_np=2)
    gloo_run.launch_gloo_elastic(
        [sys.executable, str(script), "--epochs", "5", "--samples", "2048", "--batch-size", "32",
         "--batches-per-commit", "4", "--no-cuda"],
        gloo_run._exec_slot, settings, _env(), None)
    out = capfd.readouterr().out
    assert os.path.exists(marker)
    rows = re.findall(r"epoch (\d+): loss ([0-9.]+) accuracy ([0-9.]+) on (\d) rank\(s\)", out)
    assert [int(r[0]) for r in rows] == list(range(5)), out[-2000:]
    assert [int(r[3]) for r in rows] == [2, 1, 1, 1, 1]
    assert float(rows[-1][2]) > 0.9, rows[-1]


def test_elastic_mnist_example_gives_up_a_host_that_disappears(tmp_path, capfd):
    """The discovery script stops listing the second "host" some seconds into
    the run: its worker is told that it was removed, the other one goes on
    alone from where the job was (no rollback) and every epoch is reported
    exactly once."""
    import re
    import time
    example = os.path.join(os.path.dirname(HERE), "examples", "pytorch_mnist_elastic.py")
    script = tmp_path / "discover.sh"
    script.write_text("#!/bin/bash\necho localhost:1\n"
                      "if [ $(( $(date +%%s) - %d )) -lt 9 ]; then echo 127.0.0.1:1; fi\n"
                      % int(time.time()))
    script.chmod(script.stat().st_mode | stat.S_IEXEC)
    disc = discovery.HostDiscoveryScript(str(script), slots=1)
    settings = _settings(disc, np=2, min_np=1, max_np=2)
    gloo_run.launch_gloo_elastic(
        [sys.executable, example, "--epochs", "30", "--samples", "2048", "--batch-size", "32",
         "--batches-per-commit", "4", "--no-cuda"],
        gloo_run._exec_slot, settings, _env(), None)
    captured = capfd.readouterr()
    out = captured.out
    # the removed worker says so and leaves without a traceback
    assert "Traceback" not in captured.err, captured.err[-2000:]
    rows = re.findall(r"epoch (\d+): loss ([0-9.]+) accuracy ([0-9.]+) on (\d) rank\(s\)", out)
    assert [int(r[0]) for r in rows] == list(range(30)), out[-2000:]
    ranks = [int(r[3]) for r in rows]
    assert ranks[-1] == 1 and ranks == sorted(ranks, reverse=True), ranks
    assert float(rows[-1][2]) > 0.9, rows[-1]
