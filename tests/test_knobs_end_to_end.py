"""Runtime knobs exercised through real 2-rank CPU jobs: the stall inspector
(warning, then job shutdown), a timeline started from the environment, and
correct results with fusion and the response cache switched off
(parity: test/parallel/test_torch.py + test/integration/test_stall.py)."""
import json
import os
import time

import torch

from parallel_utils import run_parallel


def _stalled_rank(rank, size, shutdown_after):
    os.environ["HOROVOD_STALL_CHECK_TIME_SECONDS"] = "1"
    if shutdown_after:
        os.environ["HOROVOD_STALL_SHUTDOWN_TIME_SECONDS"] = str(shutdown_after)
    import horovod_b200.torch as hvd
    from horovod_b200.common.exceptions import HorovodInternalError
    hvd.init()
    hvd.allreduce(torch.ones(2), name="warm")
    t0 = time.time()
    outcome = None
    try:
        if rank == 1:
            time.sleep(4.0 if not shutdown_after else 7.0)  # the late rank
        out = hvd.allreduce(torch.ones(3), op=hvd.Sum, name="late.tensor")
        outcome = ("ok", out.tolist(), time.time() - t0)
    except HorovodInternalError as e:
        outcome = ("error", str(e), time.time() - t0)
    try:
        hvd.shutdown()
    except Exception:  # noqa: BLE001
        pass
    return outcome


def test_stall_inspector_warns_and_job_continues(capfd):
    out = run_parallel(_stalled_rank, np=2, args=(0,), timeout=120)
    assert out[0][0] == "ok" and out[0][1] == [2.0, 2.0, 2.0], out
    assert out[1][0] == "ok", out
    err = capfd.readouterr().err
    assert "late.tensor" in err and "missing ranks" in err.lower(), err[-800:]


def test_stall_inspector_shuts_the_job_down():
    out = run_parallel(_stalled_rank, np=2, args=(2,), timeout=120)
    # rank 0 waited ~2-4 s, then the coordinator shut the job down; rank 1
    # finds the job gone when it finally arrives
    assert out[0][0] == "error" and out[0][2] < 6.5, out
    assert out[1][0] == "error", out


def _env_timeline(rank, size, path):
    os.environ["HOROVOD_TIMELINE"] = path
    os.environ["HOROVOD_TIMELINE_MARK_CYCLES"] = "1"
    import horovod_b200.torch as hvd
    hvd.init()
    for i in range(3):
        hvd.allreduce(torch.ones(5), name="env.tl")
    hvd.broadcast(torch.ones(2), root_rank=0, name="env.bc")
    hvd.shutdown()
    return True


def test_timeline_from_environment(tmp_path):
    path = str(tmp_path / "timeline.json")
    assert all(run_parallel(_env_timeline, np=2, args=(path,)))
    events = json.load(open(path))
    names = {e.get("name") for e in events}
    assert {"ALLREDUCE", "BROADCAST", "CYCLE_START"} <= names, names
    tensors = {e["args"]["name"] for e in events if e.get("name") == "process_name"}
    assert {"env.tl", "env.bc"} <= tensors


def _no_fusion_no_cache(rank, size, fusion, cache):
    os.environ["HOROVOD_FUSION_THRESHOLD"] = fusion
    os.environ["HOROVOD_CACHE_CAPACITY"] = cache
    import horovod_b200.torch as hvd
    hvd.init()
    ok = True
    for step in range(3):
        hs = [hvd.allreduce_async(torch.full((11 + i,), float(rank + i + step)), op=hvd.Sum,
                                  name="nf.%d" % i) for i in range(12)]
        for i, h in enumerate(hs):
            out = hvd.synchronize(h)
            ok = ok and bool((out == sum(r + i + step for r in range(size))).all())
        g = hvd.grouped_allreduce([torch.full((3,), float(rank)), torch.full((5,), 1.0)],
                                  op=hvd.Average, name="nf.group")
        ok = ok and abs(float(g[0][0]) - (size - 1) / 2.0) < 1e-6 and float(g[1][0]) == 1.0
    hvd.shutdown()
    return ok


def test_results_do_not_depend_on_fusion_or_cache():
    for fusion, cache in (("0", "1024"), (str(64 << 20), "0"), ("0", "0"), ("64", "2")):
        assert all(run_parallel(_no_fusion_no_cache, np=2, args=(fusion, cache))), (fusion, cache)


def _blocking_latency(rank, size, flush):
    """Ten blocking allreduces under a 100 ms cycle time."""
    os.environ["HOROVOD_CYCLE_TIME"] = "100"
    os.environ["HOROVOD_FLUSH_ON_WAIT"] = flush
    import horovod_b200.torch as hvd
    hvd.init()
    hvd.allreduce(torch.ones(2), name="warm")
    t0 = time.time()
    ok = True
    for i in range(10):
        out = hvd.allreduce(torch.full((4,), float(rank + i)), op=hvd.Sum, name="lat.%d" % i)
        ok = ok and out.tolist() == [float(sum(r + i for r in range(size)))] * 4
    # asynchronous ops issued together still travel together (one cycle, fused)
    hs = [hvd.allreduce_async(torch.ones(3) * (rank + 1), op=hvd.Sum, name="lat.async.%d" % i)
          for i in range(20)]
    for h in hs:
        ok = ok and hvd.synchronize(h).tolist() == [float(size * (size + 1) // 2)] * 3
    elapsed = time.time() - t0
    hvd.shutdown()
    return ok, elapsed


def test_a_blocked_caller_does_not_wait_out_the_cycle_time():
    """synchronize() on an op that has not been negotiated yet makes the
    background loop negotiate at once instead of sleeping out its cycle
    (HOROVOD_FLUSH_ON_WAIT, on by default): ten blocking allreduces under a
    100 ms cycle take far less than ten cycles; with the knob off they take
    about one cycle each, as in the reference."""
    fast = run_parallel(_blocking_latency, np=2, args=("1",), timeout=120)
    slow = run_parallel(_blocking_latency, np=2, args=("0",), timeout=120)
    assert all(ok for ok, _ in fast) and all(ok for ok, _ in slow)
    assert max(t for _, t in fast) < 0.5, fast
    assert min(t for _, t in slow) > 0.7, slow
