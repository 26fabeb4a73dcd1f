"""The clock record of the benchmarks against a stand-in ``nvidia-smi`` (a
script on PATH that prints the CSV lines the real tool prints): parsing,
windows, throttle reasons, and the case where the tool does not exist.
Nothing here touches a GPU or a GPU setting."""
import os
import stat
import time

from horovod_b200.utils.clocks import ClockLog

FAKE = """#!/bin/sh
# args are ignored; prints one sample every 50 ms until terminated
i=0
while [ $i -lt 200 ]; do
  now=$(date +"%Y/%m/%d %H:%M:%S.%3N")
  if [ $i -lt 10 ]; then
    echo "$now, 1965, 1965, 410.5, Not Active, Not Active, Not Active, Not Active"
  else
    echo "$now, 1350, 1965, 998.0, Not Active, Not Active, Not Active, Active"
  fi
  i=$((i+1))
  sleep 0.05
done
"""


def test_clock_log_parses_samples_and_windows(tmp_path, monkeypatch):
    tool = tmp_path / "nvidia-smi"
    tool.write_text(FAKE)
    tool.chmod(tool.stat().st_mode | stat.S_IEXEC)
    monkeypatch.setenv("PATH", str(tmp_path) + os.pathsep + os.environ["PATH"])
    t0 = time.time()
    log = ClockLog(0, period_ms=50)
    try:
        time.sleep(0.35)
        t1 = time.time()
        early = log.window(t0, t1)
        assert early["sm_mhz"] == 1965.0 and early["sm_max_mhz"] == 1965.0
        assert early["reasons"] == [] and early["samples"] >= 3
        time.sleep(0.6)
        t2 = time.time()
        late = log.window(t2 - 0.2, t2)
        assert late["sm_mhz"] == 1350.0 and late["reasons"] == ["sw_power_cap"]
        assert late["power_w"] == 998.0
        # a window shorter than the sampling period falls back to the nearest sample
        assert log.window(t2 - 0.001, t2)["samples"] == 1
    finally:
        log.stop()


def test_clock_log_without_the_tool(tmp_path, monkeypatch):
    monkeypatch.setenv("PATH", str(tmp_path))  # no nvidia-smi anywhere
    log = ClockLog(0)
    out = log.window(0, time.time())
    assert out["sm_mhz"] is None and "unavailable" in out["reasons"][0]
    log.stop()
