"""More behaviours of the reference's torch test-suite on 2 CPU ranks
(test/parallel/test_torch.py): argument errors of alltoall and broadcast,
join against allgather/broadcast, optimizer corner cases (requires_grad
toggled between steps, parameters without names, synchronize() + step()
warning), model parallelism inside a rank."""
import warnings

import torch
import torch.nn as nn
import torch.nn.functional as F

from parallel_utils import run_parallel


def _argument_errors(rank, size):
    import horovod_b200.torch as hvd
    hvd.init()
    res = {}

    def raises(fn, *types):
        try:
            fn()
            return False
        except types:
            return True

    x = torch.arange(12, dtype=torch.float32).view(6, 2)
    # alltoall: wrong number of splits, splits that exceed dim 0, non-integer splits
    res["a2a_len"] = raises(lambda: hvd.alltoall(x, splits=torch.tensor([1] * (size + 1)),
                                                 name="e1"), ValueError, RuntimeError)
    res["a2a_sum"] = raises(lambda: hvd.alltoall(x, splits=torch.tensor([5] * size), name="e2"),
                            ValueError, RuntimeError)
    res["a2a_type"] = raises(lambda: hvd.alltoall(x, splits=torch.tensor([1.5] * size),
                                                  name="e3"), ValueError, RuntimeError, TypeError)
    # equal split needs dim 0 divisible by size
    odd = torch.zeros(size * 2 + 1, 2)
    res["a2a_equal"] = raises(lambda: hvd.alltoall(odd, name="e4"), ValueError, RuntimeError)
    # broadcast: root outside the job
    res["bc_root"] = raises(lambda: hvd.broadcast(x, root_rank=size + 3, name="e5"),
                            ValueError, RuntimeError)
    # still healthy afterwards
    ok = hvd.allreduce(torch.ones(3), op=hvd.Sum, name="after.errors")
    res["healthy"] = bool((ok == size).all())
    hvd.shutdown()
    return res


def test_argument_errors():
    for rep in run_parallel(_argument_errors, np=2):
        assert all(rep.values()), rep


def _join_vs_other_ops(rank, size, op):
    import horovod_b200.torch as hvd
    hvd.init()
    t = torch.ones(17, 3)
    raised = None
    if rank == 0:
        hvd.join()
    else:
        try:
            if op == "allgather":
                hvd.allgather(t, name="j.ag")
            else:
                hvd.broadcast(t, root_rank=1, name="j.bc")
            raised = False
        except RuntimeError:
            raised = True
        hvd.join()
    hvd.shutdown()
    return raised


def test_join_refuses_allgather_and_broadcast():
    for op in ("allgather", "broadcast"):
        out = run_parallel(_join_vs_other_ops, np=2, args=(op,))
        assert out[1] is True, (op, out)


def _join_vs_cached_ops(rank, size):
    """The same allgather first runs normally (and is cached), then again
    while rank 0 has joined: the cached response must not be used."""
    import horovod_b200.torch as hvd
    hvd.init()
    t = torch.full((rank + 2, 3), float(rank))
    for _ in range(3):  # cached after the first round
        out = hvd.allgather(t, name="jc.ag")
        assert out.shape[0] == sum(r + 2 for r in range(size))
    raised = None
    if rank == 0:
        hvd.join()
    else:
        try:
            hvd.allgather(t, name="jc.ag")
            raised = False
        except RuntimeError:
            raised = True
        hvd.join()
    # and afterwards it works again for everybody
    out = hvd.allgather(t, name="jc.ag")
    ok = out.shape[0] == sum(r + 2 for r in range(size))
    hvd.shutdown()
    return raised, ok


def test_join_refuses_a_cached_allgather():
    out = run_parallel(_join_vs_cached_ops, np=2)
    assert out[1][0] is True, out
    assert out[0][1] and out[1][1], out


def _optimizer_corner_cases(rank, size):
    import horovod_b200.torch as hvd
    hvd.init()
    res = {}
    torch.manual_seed(3)

    # requires_grad toggled between steps (two sub-networks trained in turn)
    gen, disc = nn.Linear(4, 4), nn.Linear(4, 1)
    hvd.broadcast_parameters(gen.state_dict(), root_rank=0)
    hvd.broadcast_parameters(disc.state_dict(), root_rank=0)
    named = [("gen." + n, p) for n, p in gen.named_parameters()] + \
            [("disc." + n, p) for n, p in disc.named_parameters()]
    opt = hvd.DistributedOptimizer(
        torch.optim.SGD(list(gen.parameters()) + list(disc.parameters()), lr=0.1),
        named_parameters=named)
    x = torch.randn(5, 4)
    ok = True
    for step in range(4):
        train_gen = step % 2 == 0
        for p in gen.parameters():
            p.requires_grad_(train_gen)
        for p in disc.parameters():
            p.requires_grad_(not train_gen)
        opt.zero_grad()
        disc(gen(x)).sum().backward()
        opt.step()
    agree = hvd.allreduce(torch.cat([p.detach().flatten() for p in gen.parameters()]),
                          op=hvd.Average, name="toggle.check")
    ok = ok and torch.allclose(agree, torch.cat([p.detach().flatten() for p in gen.parameters()]),
                               atol=1e-6)
    res["toggle_requires_grad"] = ok

    # no named_parameters at all: names are generated
    model = nn.Linear(3, 2)
    hvd.broadcast_parameters(model.state_dict(), root_rank=0)
    opt = hvd.DistributedOptimizer(torch.optim.SGD(model.parameters(), lr=0.1))
    opt.zero_grad()
    model(torch.randn(2, 3)).sum().backward()
    opt.step()
    res["no_names"] = True

    # named_parameters that miss a parameter are refused
    model = nn.Linear(3, 2)
    try:
        hvd.DistributedOptimizer(torch.optim.SGD(model.parameters(), lr=0.1),
                                 named_parameters=list(model.named_parameters())[:1])
        res["missing_names"] = False
    except ValueError:
        res["missing_names"] = True

    # synchronize() followed by step() outside skip_synchronize() warns
    model = nn.Linear(1, 1)
    hvd.broadcast_parameters(model.state_dict(), root_rank=0)
    opt = hvd.DistributedOptimizer(torch.optim.SGD(model.parameters(), lr=0.1),
                                   named_parameters=model.named_parameters())
    opt.zero_grad()
    F.mse_loss(model(torch.zeros(1, 1)), torch.ones(1, 1)).backward()
    opt.synchronize()
    with warnings.catch_warnings(record=True) as ws:
        warnings.simplefilter("always")
        opt.step()
    res["sync_step_warning"] = any(
        "optimizer.step() called without optimizer.skip_synchronize()" in str(w.message)
        for w in ws)

    # model parallelism inside a rank: two sub-modules chained, one optimizer
    class TwoStage(nn.Module):
        def __init__(self):
            super().__init__()
            torch.manual_seed(11)
            self.a = nn.Linear(6, 6)
            self.b = nn.Linear(6, 2)

        def forward(self, inp):
            return self.b(torch.relu(self.a(inp)))

    model = TwoStage()
    opt = hvd.DistributedOptimizer(torch.optim.SGD(model.parameters(), lr=0.1),
                                   named_parameters=model.named_parameters())
    g = torch.Generator().manual_seed(50 + rank)
    opt.zero_grad()
    model(torch.randn(4, 6, generator=g)).sum().backward()
    opt.step()
    flat = torch.cat([p.detach().flatten() for p in model.parameters()])
    res["model_parallel"] = torch.allclose(
        hvd.allreduce(flat, op=hvd.Average, name="mp.check"), flat, atol=1e-6)
    hvd.shutdown()
    return res


def test_optimizer_corner_cases():
    for rep in run_parallel(_optimizer_corner_cases, np=2, timeout=300):
        bad = [k for k, v in rep.items() if not v]
        assert not bad, bad


def _shadow_checks(rank, size):
    import os
    os.environ["HOROVOD_SHADOW_CHECK"] = "all"   # CPU tensors too; on a GPU box "1" checks the kernels
    import horovod_b200.torch as hvd
    from horovod_b200.torch import mpi_ops
    only_first = hvd.ProcessSet([0])
    hvd.init(process_sets=[only_first])
    res = {}
    x = torch.randn(1000, generator=torch.Generator().manual_seed(rank))
    expect = sum(torch.randn(1000, generator=torch.Generator().manual_seed(r)) for r in range(size))
    res["sum"] = torch.allclose(hvd.allreduce(x, op=hvd.Sum, name="s.sum"), expect, atol=1e-5)
    y = x.clone()
    hvd.allreduce_(y, op=hvd.Average, prescale_factor=2.0, name="s.inplace")
    res["inplace_scaled"] = torch.allclose(y, 2.0 * expect / size, atol=1e-5)
    res["ints"] = hvd.allreduce(torch.arange(5) + rank, op=hvd.Sum, name="s.int").tolist() == \
        [size * i + sum(range(size)) for i in range(5)]
    res["half"] = float(hvd.allreduce(torch.ones(8).half(), op=hvd.Sum, name="s.half")[0]) == size
    group = [torch.full((3,), float(rank + 1)), torch.full((2, 2), 2.0 * (rank + 1)).half()]
    out = hvd.grouped_allreduce(group, op=hvd.Sum, name="s.group")
    tot = sum(range(1, size + 1))
    res["group"] = out[0].tolist() == [float(tot)] * 3 and float(out[1][0, 0]) == 2.0 * tot
    hvd.grouped_allreduce_(group, op=hvd.Average, name="s.group.inplace")
    res["group_inplace"] = group[0].tolist() == [tot / size] * 3
    # the ops that only move data are shadowed too and must match exactly
    g = hvd.allgather(torch.full((rank + 1, 2), float(rank)), name="s.ag")
    res["allgather"] = g.shape[0] == sum(range(1, size + 1))
    b = torch.full((4,), float(rank))
    hvd.broadcast_(b, root_rank=size - 1, name="s.bc")
    res["broadcast"] = b.tolist() == [float(size - 1)] * 4
    a, rs = hvd.alltoall(torch.arange(size * 2.0) + 10 * rank,
                         splits=torch.tensor([2] * size, dtype=torch.int32), name="s.a2a")
    res["alltoall"] = a.tolist() == [10.0 * r + 2 * rank + j for r in range(size) for j in range(2)]
    r_ = hvd.reducescatter(torch.ones(size * 3, 2) * (rank + 1), op=hvd.Sum, name="s.rs")
    res["reducescatter"] = tuple(r_.shape) == (3, 2) and float(r_[0, 0]) == tot
    res["shadows_done"] = not mpi_ops._shadow_map and mpi_ops._shadow_counter[0] == 10
    # an op that only some ranks issue (a process set) must not shift the names of later
    # shadows: they are named after their ops, not numbered per process
    if rank == 0:
        hvd.allreduce(torch.ones(2), op=hvd.Sum, name="s.alone", process_set=only_first)
    res["set_named"] = float(hvd.allreduce(torch.ones(2) * rank, op=hvd.Sum, name="s.all")[0]) == \
        sum(range(size))
    # a result that differs from the fp64 shadow is reported: 1 + 2^-9 is not a bf16 number
    mpi_ops._shadow_tolerance = lambda dtype, wire, ranks: (0.0, 0.0)
    z = torch.tensor([1.0 if rank == 0 else 2.0 ** -9]).bfloat16()
    try:
        hvd.allreduce(z, op=hvd.Sum, name="s.lossy")
        res["mismatch_reported"] = False
    except hvd.ShadowMismatch as e:
        res["mismatch_reported"] = "1 of 1 elements" in str(e)
    hvd.set_shadow_check(False)
    before = mpi_ops._shadow_counter[0]
    hvd.allreduce(z, op=hvd.Sum, name="s.off")
    res["switched_off"] = mpi_ops._shadow_counter[0] == before
    hvd.shutdown()
    return res


def test_shadow_check_recomputes_allreduces_on_the_host_and_reports_differences():
    for rep in run_parallel(_shadow_checks, np=2, timeout=300):
        bad = [k for k, v in rep.items() if not v]
        assert not bad, bad
