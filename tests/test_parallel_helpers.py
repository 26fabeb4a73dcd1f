"""horovod_b200.parallel: the two-call set-up, metric averaging in one fused
allreduce, the warm-up learning-rate schedule and the per-rank sampler, on two
CPU ranks."""
import torch

from parallel_utils import run_parallel


def _helpers(rank, size):
    import horovod_b200.torch as hvd
    from horovod_b200 import parallel
    hvd.init()
    res = {}
    torch.manual_seed(rank)  # different initial weights on purpose
    model = torch.nn.Linear(4, 2)
    opt = torch.optim.SGD(model.parameters(), lr=0.1 * size, momentum=0.9)
    model, dopt = parallel.data_parallel_setup(model, opt)
    flat = torch.cat([p.detach().flatten() for p in model.parameters()])
    res["same_start"] = torch.allclose(hvd.allreduce(flat, op=hvd.Average, name="w0"), flat)

    # metrics: one allreduce for the whole dict
    out = parallel.average_metrics({"loss": 1.0 + rank, "acc": torch.tensor(0.5 * rank), "n": 3})
    res["metrics"] = (abs(out["loss"] - (1.0 + (size - 1) / 2)) < 1e-9
                      and abs(out["acc"] - 0.25 * (size - 1)) < 1e-9 and out["n"] == 3.0
                      and parallel.average_metrics({}) == {})

    # warm-up: from the single-rank rate to the full rate in 4 steps, then decay
    sched = parallel.warmup_lr_scheduler(dopt, warmup_steps=4,
                                         after=lambda step: 0.5 if step >= 2 else 1.0)
    rates = []
    for _ in range(8):
        rates.append(dopt.param_groups[0]["lr"])
        dopt.zero_grad()
        model(torch.randn(3, 4)).sum().backward()
        dopt.step()
        sched.step()
    full = 0.1 * size
    expect = [full * (1 + (size - 1) * k / 4) / size for k in (1, 2, 3, 4)] + \
        [full, full, full * 0.5, full * 0.5]
    res["warmup"] = all(abs(a - b) < 1e-9 for a, b in zip(rates, expect))

    # sampler: the ranks' shards are disjoint and cover the dataset
    data = torch.utils.data.TensorDataset(torch.arange(10))
    sampler = parallel.shard_sampler(data, shuffle=False)
    mine = list(iter(sampler))
    everyone = hvd.allgather_object(mine)
    res["sampler"] = sorted(i for part in everyone for i in part) == list(range(10))
    hvd.shutdown()
    return res


def test_parallel_helpers():
    for rep in run_parallel(_helpers, np=2, timeout=300):
        bad = [k for k, v in rep.items() if not v]
        assert not bad, bad
