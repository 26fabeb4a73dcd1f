"""Collective semantics on CPU tensors with 2-4 ranks over the TCP mesh.
Same expectations as the reference's test/parallel/test_torch.py: analytic
results (tensor * size etc.), every dtype and several ranks of tensor,
in-place/async forms, fusion, error paths that must raise on every rank
instead of hanging, join, autograd."""
import itertools
import os

import pytest
import torch

from parallel_utils import run_parallel

DTYPES = [torch.uint8, torch.int8, torch.int16, torch.int32, torch.int64,
          torch.float16, torch.bfloat16, torch.float32, torch.float64]


def _allreduce_family(rank, size):
    import horovod_b200.torch as hvd
    hvd.init()
    for dtype, dim in itertools.product(DTYPES, [1, 2, 3]):
        torch.manual_seed(1234)
        t = torch.randint(0, 5, [7] * dim).to(dtype)
        summed = hvd.allreduce(t, op=hvd.Sum)
        assert torch.equal(summed, (t.double() * size).to(dtype)), (dtype, dim)
        if dtype.is_floating_point:
            avg = hvd.allreduce(t, op=hvd.Average)
            assert torch.allclose(avg.double(), t.double(), atol=1e-2)
    # integer average floors
    t = torch.tensor([rank, rank + 1, 7], dtype=torch.int32)
    avg = hvd.allreduce(t, op=hvd.Average)
    tot = torch.tensor([sum(range(size)), sum(range(1, size + 1)), 7 * size])
    assert torch.equal(avg, torch.div(tot, size, rounding_mode="floor").int())
    # min / max / product
    v = torch.tensor([float(rank + 1), float(-rank)])
    assert hvd.allreduce(v, op=hvd.Min).tolist() == [1.0, float(-(size - 1))]
    assert hvd.allreduce(v, op=hvd.Max).tolist() == [float(size), 0.0]
    prod = 1.0
    for r in range(size):
        prod *= r + 1
    assert hvd.allreduce(v, op=hvd.Product)[0].item() == prod
    # in place + pre/post scale
    x = torch.ones(17) * (rank + 1)
    hvd.allreduce_(x, op=hvd.Sum, prescale_factor=2.0, postscale_factor=0.5)
    assert torch.allclose(x, torch.ones(17) * sum(range(1, size + 1)))
    # async + fusion: many small tensors in flight; poll() must be False at
    # least once (the op really is asynchronous)
    handles, seen_pending = [], False
    tensors = [torch.full((100 + i,), float(i)) for i in range(40)]
    for i, tt in enumerate(tensors):
        handles.append(hvd.allreduce_async(tt, op=hvd.Sum, name="fused.%d" % i))
    for h in handles:
        if not hvd.poll(h):
            seen_pending = True
    outs = [hvd.synchronize(h) for h in handles]
    for i, o in enumerate(outs):
        assert torch.equal(o, tensors[i] * size)
    # grouped
    outs = hvd.grouped_allreduce([torch.ones(3) * rank, torch.ones(5, 2) * 2], op=hvd.Sum)
    assert torch.equal(outs[0], torch.ones(3) * sum(range(size)))
    assert torch.equal(outs[1], torch.ones(5, 2) * 2 * size)
    # fp16 compression round trip
    c = hvd.allreduce(torch.ones(9) * 0.5, op=hvd.Sum, compression=hvd.Compression.fp16)
    assert c.dtype == torch.float32 and torch.allclose(c, torch.ones(9) * 0.5 * size)
    hvd.shutdown()
    return seen_pending


def test_allreduce_family():
    pending = run_parallel(_allreduce_family, np=2)
    assert any(pending)


def _errors(rank, size):
    import horovod_b200.torch as hvd
    from horovod_b200.common.exceptions import HorovodInternalError
    hvd.init()
    # shape mismatch
    with pytest.raises(HorovodInternalError, match="Mismatched ALLREDUCE tensor shapes"):
        hvd.allreduce(torch.ones(10 + rank), name="bad.shape")
    # dtype mismatch
    with pytest.raises(HorovodInternalError, match="Mismatched data types"):
        hvd.allreduce(torch.ones(4, dtype=torch.float32 if rank == 0 else torch.int32),
                      name="bad.dtype")
    # op mismatch
    with pytest.raises(HorovodInternalError, match="Mismatched operations"):
        if rank == 0:
            hvd.allreduce(torch.ones(4), name="bad.op")
        else:
            hvd.allgather(torch.ones(4), name="bad.op")
    # broadcast root mismatch
    with pytest.raises(HorovodInternalError, match="root ranks"):
        hvd.broadcast(torch.ones(4), root_rank=rank, name="bad.root")
    # scale mismatch
    with pytest.raises(HorovodInternalError, match="prescale"):
        hvd.allreduce(torch.ones(4), op=hvd.Sum, prescale_factor=1.0 + rank, name="bad.scale")
    # allgather trailing dim mismatch
    with pytest.raises(HorovodInternalError, match="tensor shapes"):
        hvd.allgather(torch.ones(2, 3 + rank), name="bad.ag")
    # duplicate name while in flight
    a = hvd.allreduce_async(torch.ones(1000), name="dup")
    with pytest.raises(ValueError, match="already pending"):
        hvd.allreduce_async(torch.ones(1000), name="dup")
    hvd.synchronize(a)
    # runtime still healthy afterwards
    assert hvd.allreduce(torch.ones(2), op=hvd.Sum).tolist() == [size, size]
    hvd.shutdown()
    return True


def test_mismatches_raise_on_every_rank():
    assert all(run_parallel(_errors, np=2))


def _gather_bcast_alltoall(rank, size):
    import horovod_b200.torch as hvd
    hvd.init()
    for dtype in DTYPES + [torch.bool]:
        t = (torch.ones(rank + 1, 3) * (rank % 2)).to(dtype)
        g = hvd.allgather(t)
        exp = torch.cat([(torch.ones(r + 1, 3) * (r % 2)).to(dtype) for r in range(size)])
        assert torch.equal(g, exp), dtype
    # several allgathers in flight (fused response)
    hs = [hvd.allgather_async(torch.full((rank + 1, i + 1), float(i)), name="ag.%d" % i)
          for i in range(6)]
    for i, h in enumerate(hs):
        out = hvd.synchronize(h)
        assert out.shape == (sum(range(1, size + 1)), i + 1) and bool((out == i).all())
    for root in range(size):
        t = torch.arange(5.0) * (rank + 1)
        out = hvd.broadcast(t, root_rank=root)
        assert torch.equal(out, torch.arange(5.0) * (root + 1))
        hvd.broadcast_(t, root_rank=root)
        assert torch.equal(t, torch.arange(5.0) * (root + 1))
    # alltoall: even split
    t = torch.arange(size * 2, dtype=torch.float32).view(size * 2, 1) + 100 * rank
    out = hvd.alltoall(t)
    exp = torch.cat([torch.arange(rank * 2, rank * 2 + 2, dtype=torch.float32).view(2, 1)
                     + 100 * r for r in range(size)])
    assert torch.equal(out, exp)
    # uneven split given as tensor; received splits come back
    splits = torch.tensor([p + 1 for p in range(size)], dtype=torch.int32)
    src = torch.cat([torch.full((p + 1,), float(rank * 10 + p)) for p in range(size)])
    out, recv = hvd.alltoall(src, splits=splits)
    assert recv.tolist() == [rank + 1] * size
    assert torch.equal(out, torch.cat([torch.full((rank + 1,), float(r * 10 + rank))
                                       for r in range(size)]))
    # reducescatter, ragged rows
    rows = 2 * size + 1
    full = torch.arange(rows * 2, dtype=torch.float32).view(rows, 2)
    out = hvd.reducescatter(full * (rank + 1), op=hvd.Sum)
    base, extra = divmod(rows, size)
    start = rank * base + min(rank, extra)
    n = base + (1 if rank < extra else 0)
    assert torch.equal(out, full[start:start + n] * sum(range(1, size + 1)))
    avg = hvd.reducescatter(full, op=hvd.Average)
    assert torch.allclose(avg, full[start:start + n])
    # objects
    objs = hvd.allgather_object({"rank": rank, "s": "x" * rank})
    assert [o["rank"] for o in objs] == list(range(size))
    assert hvd.broadcast_object({"a": rank}, root_rank=size - 1) == {"a": size - 1}
    hvd.shutdown()
    return True


def test_allgather_broadcast_alltoall_reducescatter():
    assert all(run_parallel(_gather_bcast_alltoall, np=3))


def _autograd(rank, size):
    import horovod_b200.torch as hvd
    hvd.init()
    x = torch.ones(5, requires_grad=True)
    hvd.allreduce(x, op=hvd.Sum).sum().backward()
    assert torch.equal(x.grad, torch.ones(5) * size)
    x = torch.ones(5, requires_grad=True)
    hvd.allreduce(x, op=hvd.Average).sum().backward()
    assert torch.allclose(x.grad, torch.ones(5))
    t = torch.ones(rank + 1, 2, requires_grad=True)
    g = hvd.allgather(t)
    (g * torch.arange(g.shape[0], dtype=torch.float32).view(-1, 1)).sum().backward()
    off = sum(range(1, rank + 1))
    exp = torch.arange(off, off + rank + 1, dtype=torch.float32).view(-1, 1).expand(-1, 2)
    assert torch.allclose(t.grad, exp)
    b = torch.ones(4, requires_grad=True)
    hvd.broadcast(b, root_rank=0).sum().backward()
    assert torch.allclose(b.grad, torch.ones(4) if rank == 0 else torch.zeros(4))
    a = torch.ones(size * 2, requires_grad=True)
    hvd.alltoall(a).sum().backward()
    assert torch.equal(a.grad, torch.ones(size * 2))
    outs = hvd.grouped_allreduce([torch.ones(3, requires_grad=True) for _ in range(2)],
                                 op=hvd.Sum)
    assert all(o.requires_grad for o in outs)
    r = torch.ones(size * 2, 3, requires_grad=True)
    hvd.reducescatter(r, op=hvd.Sum).sum().backward()
    assert torch.equal(r.grad, torch.ones(size * 2, 3))
    hvd.shutdown()
    return True


def test_autograd_of_collectives():
    assert all(run_parallel(_autograd, np=2))


def _join(rank, size):
    import horovod_b200.torch as hvd
    hvd.init()
    # rank 0 has one batch more than the others; twice, so that the second
    # round goes through the response cache.
    results = []
    for rep in range(2):
        steps = 2 if rank == 0 else 1
        for s in range(steps):
            out = hvd.allreduce(torch.ones(3) * (rank + 1), op=hvd.Average, name="join.grad")
            results.append(out[0].item())
        last = hvd.join()
        assert last >= 0
    # collectives other than allreduce refuse to run against a joined rank
    hvd.shutdown()
    return results


@pytest.mark.parametrize("cache", ["1024", "0"])
def test_join_contributes_zeros(cache):
    out = run_parallel(_join, np=2, env={"HOROVOD_CACHE_CAPACITY": cache})
    # first step: both ranks -> (1+2)/2; second step on rank 0 alone: 1/2
    assert out[0] == [1.5, 0.5, 1.5, 0.5]
    assert out[1] == [1.5, 1.5]


def _reinit_and_timeline(rank, size, path):
    import json
    import horovod_b200.torch as hvd
    hvd.init()
    hvd.start_timeline(path, mark_cycles=True)
    import time
    time.sleep(0.05)
    for i in range(3):
        hvd.allreduce(torch.ones(10), name="tl.tensor")
    hvd.allgather(torch.ones(2, 2), name="tl.gather")
    hvd.stop_timeline()
    time.sleep(0.1)
    hvd.shutdown()
    hvd.init()  # elastic reset path: init after shutdown
    ok = hvd.allreduce(torch.ones(2), op=hvd.Sum).tolist() == [size, size]
    hvd.shutdown()
    if rank == 0:
        events = json.load(open(path))
        names = {e.get("name") for e in events}
        assert "ALLREDUCE" in names and "ALLGATHER" in names and "CYCLE_START" in names
        assert any(str(n).startswith("NEGOTIATE_") for n in names)
        # balanced begin/end per tensor
        depth = {}
        for e in events:
            if e["ph"] == "B":
                depth[e["pid"]] = depth.get(e["pid"], 0) + 1
            elif e["ph"] == "E":
                depth[e["pid"]] = depth.get(e["pid"], 0) - 1
                assert depth[e["pid"]] >= 0
        assert all(v == 0 for v in depth.values())
    return ok


def test_timeline_and_reinit(tmp_path):
    assert all(run_parallel(_reinit_and_timeline, np=2, args=(str(tmp_path / "tl.json"),)))


def _process_sets(rank, size):
    import horovod_b200.torch as hvd
    even = hvd.ProcessSet([0, 2])
    odd = hvd.ProcessSet([1, 3])
    hvd.init(process_sets=[even, odd])
    mine = even if rank % 2 == 0 else odd
    other = odd if rank % 2 == 0 else even
    assert mine.included() and not other.included()
    assert mine.size() == 2 and mine.rank() == rank // 2
    out = hvd.allreduce(torch.ones(3) * rank, op=hvd.Sum, process_set=mine, name="a")
    assert out[0].item() == (2 if rank % 2 == 0 else 4)
    g = hvd.allgather(torch.tensor([float(rank)]), process_set=mine, name="g")
    assert g.tolist() == ([0.0, 2.0] if rank % 2 == 0 else [1.0, 3.0])
    b = hvd.broadcast(torch.tensor([float(rank)]), root_rank=mine.ranks[1],
                      process_set=mine, name="b")
    assert b.item() == mine.ranks[1]
    with pytest.raises(ValueError):
        hvd.allreduce(torch.ones(1), process_set=other)
    tot = hvd.allreduce(torch.ones(1), op=hvd.Sum, name="tot")
    assert tot.item() == size
    hvd.shutdown()
    return True


def test_static_process_sets():
    assert all(run_parallel(_process_sets, np=4))


def _dynamic_process_sets(rank, size):
    import horovod_b200.torch as hvd
    hvd.init(process_sets="dynamic")
    ps = hvd.add_process_set([0, 1])
    assert ps.process_set_id is not None and ps.process_set_id != 0
    if rank in (0, 1):
        out = hvd.allreduce(torch.ones(2), op=hvd.Sum, process_set=ps, name="in.set")
        assert out.tolist() == [2.0, 2.0]
    assert hvd.remove_process_set(ps)
    assert ps.process_set_id is None
    # Unnamed ops are numbered per process, so after a set-only op the
    # global op needs an explicit name to match across ranks.
    assert hvd.allreduce(torch.ones(1), op=hvd.Sum, name="global").item() == size
    hvd.shutdown()
    return True


def test_dynamic_process_sets():
    assert all(run_parallel(_dynamic_process_sets, np=3))


def _peer_leaves_early(rank, size):
    import time
    import horovod_b200.torch as hvd
    from horovod_b200.common.exceptions import HorovodInternalError
    hvd.init()
    hvd.allreduce(torch.ones(2), name="first")
    if rank == 0:
        hvd.shutdown()
        return True
    time.sleep(0.5)  # rank 0 is gone by now and has told the job to stop
    ok = hvd.rank() == 1 and hvd.size() == size and hvd.local_rank() == 1
    try:
        hvd.allreduce(torch.ones(2), name="second")
        ok = False
    except HorovodInternalError:
        pass
    hvd.shutdown()
    return ok


def test_rank_and_size_survive_a_peers_shutdown():
    assert all(run_parallel(_peer_leaves_early, np=2))


def _autotune_job(rank, size, log_path):
    os.environ["HOROVOD_AUTOTUNE"] = "1"
    os.environ["HOROVOD_AUTOTUNE_LOG"] = log_path
    os.environ["HOROVOD_AUTOTUNE_WARMUP_SAMPLES"] = "1"
    os.environ["HOROVOD_AUTOTUNE_STEPS_PER_SAMPLE"] = "2"
    os.environ["HOROVOD_AUTOTUNE_BAYES_OPT_MAX_SAMPLES"] = "3"
    os.environ["HOROVOD_CYCLE_TIME"] = "0.5"
    import horovod_b200.torch as hvd
    hvd.init()
    ok = True
    # Many steps of a few tensors each: every step feeds the tuner's byte
    # counter; results must stay correct while fusion threshold and cycle
    # time change underneath, and both ranks must keep agreeing.
    for step in range(150):
        hs = [hvd.allreduce_async(torch.full((257,), float(rank + i)), op=hvd.Sum,
                                  name="tune.%d" % i) for i in range(4)]
        for i, h in enumerate(hs):
            out = hvd.synchronize(h)
            ok = ok and bool((out == sum(r + i for r in range(size))).all())
    hvd.shutdown()
    return ok


def test_autotune_runs_end_to_end_and_logs(tmp_path):
    import os as _os
    log = str(tmp_path / "autotune.csv")
    assert all(run_parallel(_autotune_job, np=2, args=(log,), timeout=300))
    assert _os.path.exists(log), "rank 0 writes the autotune log"
    lines = open(log).read().strip().splitlines()
    assert len(lines) >= 2, lines  # header + at least one sample
    assert "fusion" in lines[0].lower() and "cycle" in lines[0].lower()
