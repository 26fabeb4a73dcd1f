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
