"""Four CPU ranks: what two ranks cannot show. Ring allreduce with ragged
chunks, two-level Adasum against the pairwise oracle applied level by level,
uneven allgather / alltoall / reducescatter, overlapping process sets used
concurrently, join with three survivors, fusion of mixed dtypes."""
import os

import torch

from parallel_utils import run_parallel


def _vec(seed, n, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(n, generator=g, dtype=torch.float64).to(dtype)


def _adasum_pair(a, b):
    dot, na, nb = float(a @ b), float(a @ a), float(b @ b)
    ca = 1.0 - dot / (2 * na) if na >= 1e-300 else 1.0
    cb = 1.0 - dot / (2 * nb) if nb >= 1e-300 else 1.0
    return ca * a + cb * b


def _four(rank, size):
    import horovod_b200.torch as hvd
    hvd.init()
    res = {}
    # allreduce: sizes around the ring's chunk boundaries, several dtypes
    ok = True
    for dtype, tol in ((torch.float32, 1e-5), (torch.float64, 1e-12), (torch.int64, 0),
                       (torch.bfloat16, 0.1), (torch.float16, 2e-2)):
        for n in (1, 3, 4, 5, 1023, 4099):
            x = _vec(100 * rank + n, n, torch.float64)
            if not dtype.is_floating_point:
                x = (x * 10).round()
            out = hvd.allreduce(x.to(dtype), op=hvd.Sum, name="ar.%s.%d" % (dtype, n))
            ref = sum((_vec(100 * r + n, n, torch.float64) * (1 if dtype.is_floating_point else 10))
                      .round().to(dtype).double() if not dtype.is_floating_point
                      else _vec(100 * r + n, n, torch.float64).to(dtype).double()
                      for r in range(size))
            err = (out.double() - ref).abs().max().item()
            ok = ok and err <= tol * max(1.0, ref.abs().max().item()) * size
    res["allreduce"] = ok

    # Adasum over 4 ranks = pairs (0,1), (2,3), then the pair of results
    n = 777
    mine = _vec(7 + rank, n, torch.float64)
    out = hvd.allreduce(mine.float(), op=hvd.Adasum, name="adasum4")
    v = [_vec(7 + r, n, torch.float64).float().double() for r in range(size)]
    ref = _adasum_pair(_adasum_pair(v[0], v[1]), _adasum_pair(v[2], v[3]))
    res["adasum"] = (out.double() - ref).abs().max().item() < 1e-4 * max(1.0, ref.abs().max().item())

    # uneven allgather / alltoall / reducescatter
    g = hvd.allgather(torch.full((rank + 1, 2), float(rank)), name="ag4")
    res["allgather"] = torch.equal(g, torch.cat([torch.full((r + 1, 2), float(r))
                                                 for r in range(size)]))
    splits = torch.tensor([(rank + p) % 3 for p in range(size)], dtype=torch.int32)
    send = torch.arange(int(splits.sum()), dtype=torch.float32) + 100 * rank
    recv, rsplits = hvd.alltoall(send, splits=splits, name="a2a4")
    exp, exp_splits = [], []
    for r in range(size):
        s = [(r + p) % 3 for p in range(size)]
        off = sum(s[:rank])
        exp.append(torch.arange(sum(s), dtype=torch.float32)[off:off + s[rank]] + 100 * r)
        exp_splits.append(s[rank])
    res["alltoall"] = torch.equal(recv, torch.cat(exp)) and rsplits.tolist() == exp_splits
    rows = 10  # 10 rows over 4 ranks: 3, 3, 2, 2
    full = sum(_vec(50 + r, rows * 3, torch.float64).view(rows, 3) for r in range(size))
    part = hvd.reducescatter(_vec(50 + rank, rows * 3, torch.float64).view(rows, 3),
                             op=hvd.Sum, name="rs4")
    lo = [0, 3, 6, 8, 10]
    res["reducescatter"] = torch.allclose(part, full[lo[rank]:lo[rank + 1]], atol=1e-12)

    hvd.shutdown()
    return res


def test_four_rank_collectives():
    for rep in run_parallel(_four, np=4, timeout=300):
        bad = [k for k, v in rep.items() if not v]
        assert not bad, bad


def _sets_and_join(rank, size):
    import os
    os.environ["HOROVOD_DYNAMIC_PROCESS_SETS"] = "1"
    import horovod_b200.torch as hvd
    hvd.init()
    res = {}
    front = hvd.add_process_set([0, 1, 2])
    back = hvd.add_process_set([1, 2, 3])
    handles = []
    if front.included():
        handles.append(("front", hvd.allreduce_async(torch.full((5,), float(rank)), op=hvd.Sum,
                                                     name="ps.front", process_set=front)))
    if back.included():
        handles.append(("back", hvd.allreduce_async(torch.full((5,), float(rank)), op=hvd.Sum,
                                                    name="ps.back", process_set=back)))
    handles.append(("all", hvd.allreduce_async(torch.full((5,), float(rank)), op=hvd.Sum,
                                               name="ps.all")))
    expect = {"front": 3.0, "back": 6.0, "all": 6.0}
    res["sets"] = all(float(hvd.synchronize(h)[0]) == expect[k] for k, h in handles)
    if back.included():
        b = hvd.broadcast(torch.full((2,), float(rank)), root_rank=3, name="ps.bc",
                          process_set=back)
        res["set_broadcast"] = float(b[0]) == 3.0
    hvd.remove_process_set(front)
    hvd.remove_process_set(back)

    # join: rank r runs r+1 steps; the others' averages count the joined ranks as zeros
    outs = []
    for step in range(rank + 1):
        outs.append(float(hvd.allreduce(torch.ones(3), op=hvd.Average, name="uneven")[0]))
    last = hvd.join()
    res["join_values"] = outs == [1.0, 0.75, 0.5, 0.25][:rank + 1]
    res["last_joined"] = last == 3
    # mixed dtypes submitted together still fuse per dtype and come back right
    hs = [hvd.allreduce_async(torch.full((9,), float(rank), dtype=dt), op=hvd.Sum,
                              name="mix.%d" % i)
          for i, dt in enumerate([torch.float32, torch.float64, torch.float32, torch.int32,
                                  torch.float64, torch.float32])]
    res["mixed"] = all(float(hvd.synchronize(h)[0]) == 6.0 for h in hs)
    hvd.shutdown()
    return res


def test_process_sets_join_and_mixed_dtypes_on_four_ranks():
    for rep in run_parallel(_sets_and_join, np=4, timeout=300):
        bad = [k for k, v in rep.items() if not v]
        assert not bad, bad


def _threads(rank, size):
    import threading
    import horovod_b200.torch as hvd
    hvd.init()
    results = {}

    def worker(tid):
        ok = True
        for step in range(30):
            out = hvd.allreduce(torch.full((64,), float(rank + tid)), op=hvd.Sum,
                                name="thr.%d" % tid)
            ok = ok and float(out[0]) == sum(r + tid for r in range(size))
        results[tid] = ok

    threads = [threading.Thread(target=worker, args=(t,)) for t in range(4)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=120)
    alive = any(t.is_alive() for t in threads)
    hvd.shutdown()
    return (not alive) and all(results.get(t) for t in range(4))


def test_collectives_from_several_python_threads():
    assert all(run_parallel(_threads, np=2, timeout=300))


def _grouped_extras(rank, size, groups_on_their_own=False):
    if groups_on_their_own:
        # every group is fused by itself, never with tensors outside it
        os.environ["HOROVOD_DISABLE_GROUP_FUSION"] = "1"
    import horovod_b200.torch as hvd
    hvd.init()
    ok = True
    for _ in range(2):  # the second pass finds the responses in the cache
        gathered = hvd.grouped_allgather([torch.full((rank + 1, 2), float(rank)),
                                          torch.full((2,), float(10 + rank))], name="gag")
        ok = ok and torch.equal(gathered[0], torch.cat([torch.full((r + 1, 2), float(r))
                                                 for r in range(size)]))
        ok = ok and gathered[1].tolist() == [float(10 + r) for r in range(size) for _ in range(2)]
        shards = hvd.grouped_reducescatter([torch.arange(size * 2, dtype=torch.float32) + rank,
                                            torch.ones(size, 3) * (rank + 1)], op=hvd.Sum, name="grs")
        tot = sum(range(size))
        exp0 = (torch.arange(size * 2, dtype=torch.float32) * size + tot)[rank * 2:(rank + 1) * 2]
        ok = ok and torch.equal(shards[0], exp0) and bool((shards[1] == sum(range(1, size + 1))).all())
        # mixed dtypes in one group: the outputs keep the order of the inputs
        mixed = hvd.grouped_reducescatter([torch.full((size, 2), float(rank + 1)),
                                           torch.full((2 * size,), rank + 1, dtype=torch.int32),
                                           torch.full((size,), float(rank + 1), dtype=torch.float64)],
                                          op=hvd.Sum, name="grs.mixed")
        tot = size * (size + 1) // 2
        ok = ok and [m.dtype for m in mixed] == [torch.float32, torch.int32, torch.float64]
        ok = ok and [tuple(m.shape) for m in mixed] == [(1, 2), (2,), (1,)]
        ok = ok and all(bool((m.double() == tot).all()) for m in mixed)
        h = hvd.grouped_allgather_async([torch.full((1,), rank, dtype=torch.int64),
                                         torch.full((rank + 1,), float(rank))], name="gag.mixed")
        got = hvd.synchronize(h)
        ok = ok and got[0].tolist() == list(range(size))
        ok = ok and got[1].tolist() == [float(r) for r in range(size) for _ in range(r + 1)]
        ok = ok and hvd.grouped_allgather([], name="gag.none") == []
    hvd.barrier()
    hvd.shutdown()
    return ok


def test_grouped_allgather_reducescatter_and_barrier():
    assert all(run_parallel(_grouped_extras, np=3, timeout=300))


def test_grouped_ops_with_groups_fused_on_their_own():
    """HOROVOD_DISABLE_GROUP_FUSION=1: the same results, twice in one job so
    that the second pass goes through the cached responses."""
    assert all(run_parallel(_grouped_extras, np=3, args=(True,), timeout=300))


def _alltoall_even_and_explicit(rank, size):
    """An alltoall without splits (every rank's first dimension travels in the
    response, so no split table is exchanged) with a different dim 0 on every
    rank, repeated (cached response), then the same name with explicit splits
    and back again: the cached "even split" response must not be reused for
    explicit splits."""
    import horovod_b200.torch as hvd
    hvd.init()
    ok = True
    for it in range(3):
        rows = size * (rank + 1)  # rank r sends r + 1 rows to every peer
        x = (torch.arange(rows * 3, dtype=torch.float32).view(rows, 3) + 1000 * rank + it)
        out = hvd.alltoall(x, name="a2a.same")
        want = torch.cat([(torch.arange(size * (r + 1) * 3, dtype=torch.float32)
                           .view(size * (r + 1), 3) + 1000 * r + it)[rank * (r + 1):(rank + 1) * (r + 1)]
                          for r in range(size)])
        ok = ok and torch.equal(out, want)
        # explicit, uneven splits under the same name
        splits = torch.tensor([(rank + p) % 3 for p in range(size)], dtype=torch.int32)
        y = torch.full((int(splits.sum()), 2), float(rank))
        out2, rsplits = hvd.alltoall(y, splits=splits, name="a2a.same")
        exp_splits = [(r + rank) % 3 for r in range(size)]
        ok = ok and rsplits.tolist() == exp_splits
        ok = ok and out2[:, 0].tolist() == [float(r) for r in range(size)
                                            for _ in range(exp_splits[r])]
    hvd.shutdown()
    return ok


def test_alltoall_even_split_needs_no_split_exchange_and_mixes_with_explicit_splits():
    assert all(run_parallel(_alltoall_even_and_explicit, np=4, timeout=300))


def _randomised_sets(rank, size):
    """Rounds of randomly sized, typed and scaled allreduces (single and
    grouped, in place and not), all in flight together so that the controller
    fuses what it can; every result is checked by the fp64 host shadow."""
    os.environ["HOROVOD_SHADOW_CHECK"] = "all"
    import random
    import horovod_b200.torch as hvd
    hvd.init()
    plan = random.Random(1234)            # the same plan on every rank
    data = torch.Generator().manual_seed(99 + rank)   # different values
    dtypes = [torch.float32, torch.float64, torch.float16, torch.bfloat16, torch.int32, torch.int64]
    checked = 0
    for rnd in range(6):
        handles = []
        for i in range(plan.randint(3, 12)):
            dtype = plan.choice(dtypes)
            shape = [plan.randint(1, 40) for _ in range(plan.randint(1, 3))]
            op = plan.choice([hvd.Sum, hvd.Average] if dtype.is_floating_point else [hvd.Sum])
            pre = plan.choice([1.0, 0.5, 2.0]) if dtype.is_floating_point else 1.0

            def make():
                if dtype.is_floating_point:
                    return torch.randn(shape, generator=data).to(dtype)
                return torch.randint(-50, 50, shape, generator=data, dtype=dtype)
            name = "rand.%d.%d" % (rnd, i)
            kind = plan.choice(["single", "inplace", "group"])
            if kind == "single":
                handles.append(hvd.allreduce_async(make(), op=op, prescale_factor=pre, name=name))
            elif kind == "inplace":
                handles.append(hvd.allreduce_async_(make(), op=op, prescale_factor=pre, name=name))
            else:
                members = [make() for _ in range(plan.randint(2, 4))]
                handles.append(hvd.grouped_allreduce_async(members, op=op, prescale_factor=pre,
                                                           name=name))
        plan.shuffle(handles)             # waited for in another order than issued
        for h in handles:
            hvd.synchronize(h)            # raises ShadowMismatch on a wrong result
            checked += 1
    from horovod_b200.torch import mpi_ops
    ok = checked >= 18 and not mpi_ops._shadow_map and mpi_ops._shadow_counter[0] == checked
    hvd.shutdown()
    return ok


def test_randomised_tensor_sets_against_the_host_shadow():
    assert all(run_parallel(_randomised_sets, np=3, timeout=600))


def _two_models_on_two_process_sets(rank, size):
    """Ranks {0, 1} and {2, 3} train their own model at the same time, each
    with a DistributedOptimizer restricted to its set: parameters agree
    inside a set, differ between the sets, and match what one process
    computes from the set's combined batches."""
    import horovod_b200.torch as hvd
    sets = [hvd.ProcessSet([0, 1]), hvd.ProcessSet([2, 3])]
    hvd.init(process_sets=sets)
    mine = sets[rank // 2]
    torch.manual_seed(7 + rank // 2)                 # one initialisation per set
    model = torch.nn.Linear(5, 2)
    reference = torch.nn.Linear(5, 2)
    reference.load_state_dict(model.state_dict())
    opt = hvd.DistributedOptimizer(torch.optim.SGD(model.parameters(), lr=0.1, momentum=0.9),
                                   named_parameters=model.named_parameters(), process_set=mine)
    hvd.broadcast_parameters(model.state_dict(), root_rank=mine.ranks[0], process_set=mine)
    hvd.broadcast_optimizer_state(opt, root_rank=mine.ranks[0], process_set=mine)
    ref_opt = torch.optim.SGD(reference.parameters(), lr=0.1, momentum=0.9)
    for step in range(4):
        batches = [torch.randn(6, 5, generator=torch.Generator().manual_seed(1000 * step + r))
                   for r in mine.ranks]
        opt.zero_grad()
        model(batches[mine.rank()]).pow(2).mean().backward()
        opt.step()
        ref_opt.zero_grad()
        reference(torch.cat(batches)).pow(2).mean().backward()
        ref_opt.step()
    flat = torch.cat([p.detach().reshape(-1) for p in model.parameters()])
    expect = torch.cat([p.detach().reshape(-1) for p in reference.parameters()])
    everyone = hvd.allgather(flat.unsqueeze(0), name="ps.models")
    ok = bool(torch.allclose(flat, expect, atol=1e-6))
    ok = ok and bool(torch.equal(everyone[0], everyone[1]) and torch.equal(everyone[2], everyone[3]))
    ok = ok and not bool(torch.allclose(everyone[0], everyone[2]))
    hvd.shutdown()
    return ok


def test_two_models_train_side_by_side_on_two_process_sets():
    assert all(run_parallel(_two_models_on_two_process_sets, np=4, timeout=300))


def _uneven_batches_with_join(rank, size):
    """Every rank has another number of batches: the ones that run out call
    join() and stand in with zeros while the others go on training; the rank
    that joined last holds the newest weights and hands them out."""
    import horovod_b200.torch as hvd
    hvd.init()
    torch.manual_seed(3)
    model = torch.nn.Linear(4, 1)
    opt = hvd.DistributedOptimizer(torch.optim.SGD(model.parameters(), lr=0.05),
                                   named_parameters=model.named_parameters())
    hvd.broadcast_parameters(model.state_dict(), root_rank=0)
    steps = 2 + 2 * rank                               # rank size-1 trains longest
    for step in range(steps):
        opt.zero_grad()
        x = torch.randn(3, 4, generator=torch.Generator().manual_seed(50 * step + rank))
        model(x).pow(2).mean().backward()
        opt.step()
    last = hvd.join()
    hvd.broadcast_parameters(model.state_dict(), root_rank=last)
    flat = torch.cat([p.detach().reshape(-1) for p in model.parameters()])
    everyone = hvd.allgather(flat.unsqueeze(0), name="join.models")
    ok = last == size - 1 and all(bool(torch.equal(everyone[0], everyone[r])) for r in range(size))
    hvd.shutdown()
    return ok


def test_training_with_uneven_batches_ends_with_join():
    assert all(run_parallel(_uneven_batches_with_join, np=3, timeout=300))


def _more_names_than_cache_entries(rank, size):
    """A working set of tensor names three times the response cache: entries
    are evicted and their bit positions reused all the time, in an order that
    differs from pass to pass, while results stay right (Average of rank-
    dependent values) and repeated names still hit the cache."""
    os.environ["HOROVOD_CACHE_CAPACITY"] = "16"
    import random
    import horovod_b200.torch as hvd
    hvd.init()
    names = ["t%02d" % i for i in range(48)]
    ok = True
    for rnd in range(5):
        order = list(names)
        random.Random(rnd).shuffle(order)              # the same order on every rank
        handles = []
        for i, name in enumerate(order):
            shape = (1 + int(name[1:]) % 7,)            # a name keeps its shape
            value = torch.full(shape, float(rank + int(name[1:])))
            handles.append((name, hvd.allreduce_async(value, op=hvd.Average, name=name)))
            if i % 5 == 4:                              # waited for in small bursts
                for n, h in handles:
                    got = hvd.synchronize(h)
                    ok = ok and bool((got == (size - 1) / 2.0 + int(n[1:])).all())
                handles = []
        for n, h in handles:
            ok = ok and bool((hvd.synchronize(h) == (size - 1) / 2.0 + int(n[1:])).all())
    # a small hot set that fits the cache keeps working after all the churn
    for rnd in range(20):
        got = hvd.allreduce(torch.ones(3) * rank, op=hvd.Sum, name="hot%d" % (rnd % 4))
        ok = ok and bool((got == sum(range(size))).all())
    hvd.shutdown()
    return ok


def test_more_tensor_names_than_response_cache_entries():
    assert all(run_parallel(_more_names_than_cache_entries, np=3, timeout=300))


def _a_name_changes_shape_type_and_op(rank, size):
    """The cached response of a name stops fitting (other shape, dtype,
    scale factor, op, or another collective altogether): every rank sees the
    same invalidation and the new request is negotiated afresh."""
    import horovod_b200.torch as hvd
    hvd.init()
    ok = True
    total = sum(range(1, size + 1))
    for shape, dtype, pre in [((4,), torch.float32, 1.0), ((4,), torch.float32, 1.0),
                              ((6,), torch.float32, 1.0), ((6,), torch.float64, 1.0),
                              ((6,), torch.float64, 0.5), ((2, 3), torch.float64, 0.5),
                              ((4,), torch.float32, 1.0)]:
        got = hvd.allreduce(torch.full(shape, float(rank + 1), dtype=dtype), op=hvd.Sum,
                            prescale_factor=pre, name="same.name")
        ok = ok and got.dtype == dtype and tuple(got.shape) == shape and \
            bool((got == pre * total).all())
    got = hvd.allreduce(torch.full((4,), float(rank + 1)), op=hvd.Max, name="same.name")
    ok = ok and bool((got == size).all())
    gathered = hvd.allgather(torch.full((1, 2), float(rank)), name="same.name")
    ok = ok and gathered[:, 0].tolist() == [float(r) for r in range(size)]
    got = hvd.allreduce(torch.full((4,), float(rank + 1)), op=hvd.Sum, name="same.name")
    ok = ok and bool((got == total).all())
    hvd.shutdown()
    return ok


def test_a_cached_name_that_changes_shape_type_scale_op_and_collective():
    assert all(run_parallel(_a_name_changes_shape_type_and_op, np=3, timeout=300))


def _eight_ranks(rank, size):
    """Every collective, Adasum over three levels and ten process sets (ids
    beyond the eight that the device kernels serve) on eight ranks, each
    result also checked by the host shadow."""
    os.environ["HOROVOD_SHADOW_CHECK"] = "all"
    import horovod_b200.torch as hvd
    hvd.init()
    ok = True
    ok &= hvd.allreduce(torch.ones(1000) * rank, op=hvd.Sum, name="a").eq(sum(range(size))).all().item()
    g = hvd.allgather(torch.full((rank + 1, 3), float(rank)), name="g")
    ok &= g.shape[0] == size * (size + 1) // 2
    a = hvd.alltoall(torch.arange(size * 2.0) + 100 * rank, name="a2a")
    ok &= a.tolist() == [100.0 * r + 2 * rank + j for r in range(size) for j in range(2)]
    r = hvd.reducescatter(torch.ones(size * 2 + 3, 4) * (rank + 1), op=hvd.Sum, name="rs")
    ok &= float(r[0, 0]) == size * (size + 1) / 2 and r.shape[0] == (3 if rank < 3 else 2)
    b = torch.full((5,), float(rank)); hvd.broadcast_(b, root_rank=5, name="b"); ok &= b.tolist() == [5.0] * 5
    ad = hvd.allreduce(torch.ones(64) * (rank + 1), op=hvd.Adasum, name="ad")
    ok &= bool(torch.isfinite(ad).all())
    sets = []
    os.environ["HOROVOD_DYNAMIC_PROCESS_SETS"] = "1"
    hvd.shutdown()
    hvd.init()
    for i in range(10):                       # ids beyond 8
        sets.append(hvd.add_process_set([i % size, (i + 1) % size, (i + 3 + i // 8) % size]))
    for i, ps in enumerate(sets):
        if ps.included():
            got = hvd.allreduce(torch.ones(4), op=hvd.Sum, name="ps%d" % i, process_set=ps)
            ok &= bool((got == 3).all())
    hvd.barrier()
    hvd.shutdown()
    return bool(ok)



def test_every_collective_and_many_process_sets_on_eight_ranks():
    assert all(run_parallel(_eight_ranks, np=8, timeout=400))
