"""CPU plumbing check: a 784-512-10 MLP trained for 10 SGD steps on 2 ranks
through hvd.DistributedOptimizer must match a single process trained on the
concatenated 64-sample batch to 1e-5."""
import torch

from parallel_utils import run_parallel


def _batch(rank):
    g = torch.Generator().manual_seed(1 + rank)
    return torch.randn(32, 784, generator=g), torch.randint(0, 10, (32,), generator=g)


def _model():
    from horovod_b200.models import MLP
    torch.manual_seed(0)
    return MLP()


def _train_rank(rank, size):
    import horovod_b200.torch as hvd
    hvd.init()
    model = _model()
    if rank != 0:  # parameters must come from rank 0, not from the local seed
        for p in model.parameters():
            p.data.add_(1.0)
    opt = torch.optim.SGD(model.parameters(), lr=0.01, momentum=0.9)
    opt = hvd.DistributedOptimizer(opt, named_parameters=model.named_parameters())
    hvd.broadcast_parameters(model.state_dict(), root_rank=0)
    hvd.broadcast_optimizer_state(opt, root_rank=0)
    x, y = _batch(rank)
    for _ in range(10):
        opt.zero_grad()
        torch.nn.functional.cross_entropy(model(x), y).backward()
        opt.step()
    out = [p.detach().clone() for p in model.parameters()]
    hvd.shutdown()
    return out


def test_two_rank_mlp_matches_single_process():
    results = run_parallel(_train_rank, np=2)
    model = _model()
    opt = torch.optim.SGD(model.parameters(), lr=0.01, momentum=0.9)
    xs, ys = zip(*[_batch(r) for r in range(2)])
    x, y = torch.cat(xs), torch.cat(ys)
    for _ in range(10):
        opt.zero_grad()
        torch.nn.functional.cross_entropy(model(x), y).backward()
        opt.step()
    for rank_params in results:
        for got, want in zip(rank_params, model.parameters()):
            assert abs(got - want.detach().numpy()).max() <= 1e-5
