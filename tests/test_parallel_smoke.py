import torch

from parallel_utils import run_parallel


def _basic(rank, size):
    import horovod_b200.torch as hvd
    hvd.init()
    assert hvd.rank() == rank and hvd.size() == size
    t = torch.arange(10, dtype=torch.float32) * (rank + 1)
    s = hvd.allreduce(t, op=hvd.Sum)
    a = hvd.allreduce(t)
    g = hvd.allgather(torch.full((rank + 1, 2), float(rank)))
    b = hvd.broadcast(t, root_rank=1)
    hvd.shutdown()
    return s.tolist(), a.tolist(), g.tolist(), b.tolist()


def test_two_ranks_basic():
    out = run_parallel(_basic, np=2)
    base = torch.arange(10, dtype=torch.float32)
    for s, a, g, b in out:
        assert s == (base * 3).tolist()
        assert a == (base * 1.5).tolist()
        assert g == [[0.0, 0.0], [1.0, 1.0], [1.0, 1.0]]
        assert b == (base * 2).tolist()
