"""DistributedOptimizer, broadcast of optimizer state for the torch optimizer
classes, compression, gradient accumulation, groups, unused parameters,
gradient clipping with synchronize(), sparse gradients, Adasum optimizer,
SyncBatchNorm: 2 CPU ranks. Mirrors test/parallel/test_torch.py:1490-2100."""
import torch
import torch.nn as nn
import torch.nn.functional as F

from parallel_utils import run_parallel


def _net():
    torch.manual_seed(0)
    return nn.Sequential(nn.Linear(8, 16), nn.ReLU(), nn.Linear(16, 4))


def _data(rank):
    g = torch.Generator().manual_seed(100 + rank)
    return torch.randn(6, 8, generator=g), torch.randint(0, 4, (6,), generator=g)


OPTIMIZERS = [
    ("SGD", lambda p: torch.optim.SGD(p, lr=0.1, momentum=0.9)),
    ("Adam", lambda p: torch.optim.Adam(p, lr=0.01)),
    ("AdamW", lambda p: torch.optim.AdamW(p, lr=0.01)),
    ("Adagrad", lambda p: torch.optim.Adagrad(p, lr=0.1)),
    ("Adadelta", lambda p: torch.optim.Adadelta(p)),
    ("Adamax", lambda p: torch.optim.Adamax(p)),
    ("RMSprop", lambda p: torch.optim.RMSprop(p, lr=0.01, momentum=0.5)),
    ("Rprop", lambda p: torch.optim.Rprop(p)),
    ("ASGD", lambda p: torch.optim.ASGD(p)),
    ("NAdam", lambda p: torch.optim.NAdam(p)),
    ("RAdam", lambda p: torch.optim.RAdam(p)),
]


def _broadcast_state(rank, size):
    import horovod_b200.torch as hvd
    hvd.init()
    report = {}
    for name, make in OPTIMIZERS:
        model = _net()
        # ranks diverge: different weights, different lr, different history
        with torch.no_grad():
            for p in model.parameters():
                p.add_(rank * 0.5)
        opt = make(model.parameters())
        for group in opt.param_groups:
            group["lr"] = group["lr"] * (1 + rank)
        steps = 2 if rank == 0 else 0  # only the root has optimizer state
        x, y = _data(rank)
        for _ in range(steps):
            opt.zero_grad()
            F.cross_entropy(model(x), y).backward()
            opt.step()
        hvd.broadcast_parameters(model.state_dict(), root_rank=0)
        hvd.broadcast_optimizer_state(opt, root_rank=0)
        sd = opt.state_dict()
        flat = []
        for pid in sorted(sd["state"]):
            for k in sorted(sd["state"][pid]):
                v = sd["state"][pid][k]
                flat.append(v.detach().double().flatten() if torch.is_tensor(v)
                            else torch.tensor([float(v)], dtype=torch.float64))
        flat.append(torch.tensor([float(g["lr"]) for g in sd["param_groups"]],
                                 dtype=torch.float64))
        flat += [p.detach().double().flatten() for p in model.parameters()]
        vec = torch.cat(flat)
        ref = hvd.broadcast(vec, root_rank=0, name="check.%s" % name)
        report[name] = (len(sd["state"]), float((vec - ref).abs().max()))
    hvd.shutdown()
    return report


def test_broadcast_optimizer_state_for_every_optimizer():
    out = run_parallel(_broadcast_state, np=2, timeout=300)
    for rep in out:
        for name, (n_state, diff) in rep.items():
            assert diff == 0.0, (name, diff)
            if name != "SGD":
                assert n_state > 0, name


def _optimizer_features(rank, size):
    import horovod_b200.torch as hvd
    hvd.init()
    x, y = _data(rank)
    xs, ys = zip(*[_data(r) for r in range(size)])

    def reference(steps, lr=0.1, accumulate=1, clip=None):
        model = _net()
        opt = torch.optim.SGD(model.parameters(), lr=lr)
        for _ in range(steps):
            opt.zero_grad()
            # average over ranks of the (accumulated) per-rank gradients
            for r in range(size):
                for _a in range(accumulate):
                    (F.cross_entropy(model(xs[r]), ys[r]) / size).backward()
            if clip is not None:
                torch.nn.utils.clip_grad_norm_(model.parameters(), clip)
            opt.step()
        return [p.detach().clone() for p in model.parameters()]

    def close(model, ref, tol=1e-5):
        return all(torch.allclose(a, b, atol=tol) for a, b in zip(model.parameters(), ref))

    results = {}
    # plain
    model = _net()
    opt = hvd.DistributedOptimizer(torch.optim.SGD(model.parameters(), lr=0.1),
                                   named_parameters=model.named_parameters())
    for _ in range(3):
        opt.zero_grad()
        F.cross_entropy(model(x), y).backward()
        opt.step()
    results["plain"] = close(model, reference(3))

    # fp16 / bf16 compression (CPU path: casts in Python)
    for comp, tol in ((hvd.Compression.fp16, 2e-3), (hvd.Compression.bf16, 2e-2)):
        model = _net()
        opt = hvd.DistributedOptimizer(torch.optim.SGD(model.parameters(), lr=0.1),
                                       named_parameters=model.named_parameters(),
                                       compression=comp)
        for _ in range(3):
            opt.zero_grad()
            F.cross_entropy(model(x), y).backward()
            opt.step()
        results["comp.%s" % comp.__name__] = close(model, reference(3), tol)

    # backward_passes_per_step: gradients accumulate locally, one reduction
    model = _net()
    opt = hvd.DistributedOptimizer(torch.optim.SGD(model.parameters(), lr=0.1),
                                   named_parameters=model.named_parameters(),
                                   backward_passes_per_step=2)
    for _ in range(2):
        opt.zero_grad()
        for _a in range(2):
            F.cross_entropy(model(x), y).backward()
        opt.step()
    results["accumulate"] = close(model, reference(2, accumulate=2))

    # explicit groups (grouped allreduce) and predivide factor
    model = _net()
    opt = hvd.DistributedOptimizer(torch.optim.SGD(model.parameters(), lr=0.1),
                                   named_parameters=model.named_parameters(), groups=2,
                                   gradient_predivide_factor=2.0)
    for _ in range(3):
        opt.zero_grad()
        F.cross_entropy(model(x), y).backward()
        opt.step()
    results["groups"] = close(model, reference(3))

    # gradient clipping: synchronize(), clip, step inside skip_synchronize()
    model = _net()
    opt = hvd.DistributedOptimizer(torch.optim.SGD(model.parameters(), lr=0.1),
                                   named_parameters=model.named_parameters())
    for _ in range(2):
        opt.zero_grad()
        F.cross_entropy(model(x), y).backward()
        opt.synchronize()
        torch.nn.utils.clip_grad_norm_(model.parameters(), 0.05)
        with opt.skip_synchronize():
            opt.step()
    results["clip"] = close(model, reference(2, clip=0.05))

    # a parameter that gets no gradient on one rank is still reduced (zeros)
    class TwoHeads(nn.Module):
        def __init__(self):
            super().__init__()
            torch.manual_seed(1)
            self.a = nn.Linear(8, 4)
            self.b = nn.Linear(8, 4)

        def forward(self, inp, use_b):
            return self.a(inp) + (self.b(inp) if use_b else 0)

    model = TwoHeads()
    opt = hvd.DistributedOptimizer(torch.optim.SGD(model.parameters(), lr=0.1),
                                   named_parameters=model.named_parameters())
    before = model.b.weight.detach().clone()
    opt.zero_grad()
    F.cross_entropy(model(x, use_b=(rank == 0)), y).backward()
    opt.step()
    moved = not torch.equal(before, model.b.weight)
    agree = hvd.allreduce(model.b.weight.detach(), op=hvd.Average, name="chk.b")
    results["unused"] = moved and torch.allclose(agree, model.b.weight, atol=1e-6)

    # zero_grad between backward and step is refused
    model = _net()
    opt = hvd.DistributedOptimizer(torch.optim.SGD(model.parameters(), lr=0.1),
                                   named_parameters=model.named_parameters())
    F.cross_entropy(model(x), y).backward()
    try:
        opt.zero_grad()
        results["zero_grad_guard"] = False
    except AssertionError:
        results["zero_grad_guard"] = True
    opt.step()

    # duplicate names are refused
    try:
        hvd.DistributedOptimizer(torch.optim.SGD(model.parameters(), lr=0.1),
                                 named_parameters=[("a", p) for p in model.parameters()])
        results["dup_names"] = False
    except ValueError:
        results["dup_names"] = True

    # sparse gradients: as allgathers, or densified
    for dense in (False, True):
        torch.manual_seed(0)
        emb = nn.Embedding(10, 3, sparse=True)
        opt = hvd.DistributedOptimizer(torch.optim.SGD(emb.parameters(), lr=1.0),
                                       named_parameters=emb.named_parameters(),
                                       sparse_as_dense=dense)
        w0 = emb.weight.detach().clone()
        opt.zero_grad()
        emb(torch.tensor([rank, 5])).sum().backward()
        opt.step()
        exp = w0.clone()
        for r in range(size):
            exp[r] -= 1.0 / size
        exp[5] -= 1.0
        results["sparse.%s" % dense] = torch.allclose(emb.weight.detach(), exp, atol=1e-6)

    # Adasum optimizer: identical data on every rank -> same as one local step
    model = _net()
    opt = hvd.DistributedOptimizer(torch.optim.SGD(model.parameters(), lr=0.1),
                                   named_parameters=model.named_parameters(), op=hvd.Adasum)
    ref = _net()
    ropt = torch.optim.SGD(ref.parameters(), lr=0.1)
    for _ in range(2):
        for m, o in ((model, opt), (ref, ropt)):
            o.zero_grad()
            F.cross_entropy(m(xs[0]), ys[0]).backward()
            o.step()
    results["adasum"] = all(torch.allclose(a, b, atol=1e-5)
                            for a, b in zip(model.parameters(), ref.parameters()))
    hvd.shutdown()
    return results


def test_distributed_optimizer_features():
    for rep in run_parallel(_optimizer_features, np=2, timeout=300):
        bad = [k for k, ok in rep.items() if not ok]
        assert not bad, bad


def _sync_bn(rank, size):
    import horovod_b200.torch as hvd
    hvd.init()
    torch.manual_seed(0)
    full = torch.randn(8, 3, 5, 5)
    w = torch.randn(3)
    mine = full[rank * 4:(rank + 1) * 4].clone().requires_grad_(True)
    bn = hvd.SyncBatchNorm(3)
    with torch.no_grad():
        bn.weight.copy_(w)
    out = bn(mine)
    (out * torch.arange(out.numel(), dtype=torch.float32).view_as(out) / 100).sum().backward()

    ref_in = full.clone().requires_grad_(True)
    ref_bn = nn.BatchNorm2d(3)
    with torch.no_grad():
        ref_bn.weight.copy_(w)
    ref_out = ref_bn(ref_in)
    scale = torch.zeros_like(ref_out)
    scale[rank * 4:(rank + 1) * 4] = \
        torch.arange(out.numel(), dtype=torch.float32).view_as(out) / 100
    # every rank's loss only covers its slice; the input gradient of the full
    # batch is the sum over ranks
    other = 1 - rank
    scale[other * 4:(other + 1) * 4] = \
        torch.arange(out.numel(), dtype=torch.float32).view_as(out) / 100
    (ref_out * scale).sum().backward()
    ok = torch.allclose(out, ref_out[rank * 4:(rank + 1) * 4], atol=1e-5)
    ok = ok and torch.allclose(mine.grad, ref_in.grad[rank * 4:(rank + 1) * 4], atol=1e-4)
    ok = ok and torch.allclose(bn.running_mean, ref_bn.running_mean, atol=1e-5)
    ok = ok and torch.allclose(bn.running_var, ref_bn.running_var, atol=1e-5)
    hvd.shutdown()
    return ok


def test_sync_batch_norm_matches_full_batch():
    assert all(run_parallel(_sync_bn, np=2))


def _force_allreduce_every_optimizer(rank, size):
    """Every rank back-propagates through a different part of the model (rank 0
    never touches the last layer), for every optimizer class PyTorch ships:
    step() must reduce all gradients, the missing ones as zeros, and leave
    identical parameters on all ranks (parity: test_force_allreduce,
    test/parallel/test_torch.py:1791-1858)."""
    import inspect
    import torch.nn.functional as F
    import horovod_b200.torch as hvd
    hvd.init()
    torch.manual_seed(3)
    x, y = torch.randn(16, 20), torch.randn(16, 5)

    class Net(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.fc1 = torch.nn.Linear(20, 8)
            self.fc2 = torch.nn.Linear(8, 5)
            self.fc3 = torch.nn.Linear(5, 5)

        def forward(self, inp):
            hidden = F.relu(self.fc1(inp))
            first = self.fc2(hidden)
            return first, self.fc3(F.relu(first))

    classes = sorted((c for c in torch.optim.Optimizer.__subclasses__()
                      if c.__module__.startswith("torch.optim")
                      and c not in (torch.optim.LBFGS, torch.optim.SparseAdam)),
                     key=lambda c: c.__name__)
    failures = []
    for cls in classes:
        for wanted in (dict(lr=0.2, momentum=0.9, weight_decay=0.1, centered=True), dict(lr=0.2)):
            accepted = inspect.signature(cls.__init__).parameters
            kwargs = {k: v for k, v in wanted.items() if k in accepted}
            model = Net()
            hvd.broadcast_parameters(model.state_dict(), root_rank=0)
            try:
                base = cls(model.parameters(), **kwargs)
            except ValueError:
                continue  # an optimizer that refuses this model (matrices only, say)
            opt = hvd.DistributedOptimizer(base, named_parameters=model.named_parameters())
            first, second = model(x)
            loss = F.mse_loss(first if rank == 0 else second, y, reduction="sum")
            opt.zero_grad()
            loss.backward()
            opt.step()
            flat = torch.cat([p.detach().flatten() for p in model.parameters()])
            same = hvd.allreduce(flat, op=hvd.Average, name="fa.%s.%d" % (cls.__name__,
                                                                          len(kwargs)))
            if not torch.allclose(same, flat, atol=1e-5, equal_nan=True):
                failures.append(cls.__name__)
    hvd.shutdown()
    return failures, len(classes)


def test_step_reduces_every_gradient_for_every_optimizer_class():
    for failures, n in run_parallel(_force_allreduce_every_optimizer, np=2, timeout=600):
        assert n >= 8 and failures == [], failures
