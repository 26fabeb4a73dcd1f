"""Two-level (hierarchical) allreduce and allgather on CPU ranks laid out as
two hosts of two ranks each (distinct cross ranks on one box, the way the
reference's own tests fake a second host), against the flat results; and the
policy of the persistent fusion buffer."""
import os

import torch

from parallel_utils import run_parallel


def _vec(seed, n, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(n, generator=g, dtype=torch.float64).to(dtype)


def _two_hosts(rank, size, hierarchical):
    local = 2
    os.environ.update({
        "HOROVOD_LOCAL_RANK": str(rank % local), "HOROVOD_LOCAL_SIZE": str(local),
        "HOROVOD_CROSS_RANK": str(rank // local), "HOROVOD_CROSS_SIZE": str(size // local),
        "HOROVOD_HOSTNAME": "host-%d" % (rank // local),
        "HOROVOD_HIERARCHICAL_ALLREDUCE": "1" if hierarchical else "0",
        "HOROVOD_HIERARCHICAL_ALLGATHER": "1" if hierarchical else "0",
    })
    import horovod_b200.torch as hvd
    hvd.init()
    assert (hvd.local_size(), hvd.cross_size(), hvd.local_rank(), hvd.cross_rank()) == \
        (local, size // local, rank % local, rank // local)
    assert hvd.runtime_params()["hierarchical_allreduce"] == hierarchical
    assert hvd.runtime_params()["hierarchy_usable"]
    ok = True
    for dtype, tol in ((torch.float32, 1e-5), (torch.float64, 1e-12), (torch.int32, 0),
                       (torch.float16, 2e-2)):
        for n in (1, 2, 3, 5, 1000, 4099):
            x = _vec(10 * rank + n, n, torch.float64)
            x = (x * 10).round().to(dtype) if not dtype.is_floating_point else x.to(dtype)
            for op, name in ((hvd.Sum, "sum"), (hvd.Average, "avg")):
                if op == hvd.Average and not dtype.is_floating_point:
                    continue
                out = hvd.allreduce(x, op=op, name="h.%s.%s.%d" % (name, dtype, n))
                parts = []
                for r in range(size):
                    v = _vec(10 * r + n, n, torch.float64)
                    parts.append(((v * 10).round().to(dtype) if not dtype.is_floating_point
                                  else v.to(dtype)).double())
                ref = sum(parts) / (size if op == hvd.Average else 1)
                err = (out.double() - ref).abs().max().item()
                ok = ok and err <= tol * max(1.0, ref.abs().max().item()) * size
    # min/max travel through the same two levels
    m = hvd.allreduce(torch.tensor([float(rank), -float(rank)]), op=hvd.Max, name="h.max")
    ok = ok and m.tolist() == [float(size - 1), 0.0]
    # a fused group of odd-sized tensors
    xs = [_vec(rank * 7 + i, s) for i, s in enumerate((3, 129, 77, 2048, 5))]
    outs = hvd.grouped_allreduce(xs, op=hvd.Sum, name="h.grp")
    for i, (s, o) in enumerate(zip((3, 129, 77, 2048, 5), outs)):
        ref = sum(_vec(r * 7 + i, s).double() for r in range(size))
        ok = ok and (o.double() - ref).abs().max().item() < 1e-4
    # allgather with a different dim 0 on every rank
    g = hvd.allgather(torch.full((rank + 1, 3), float(rank)), name="h.ag")
    exp = torch.cat([torch.full((r + 1, 3), float(r)) for r in range(size)])
    ok = ok and torch.equal(g, exp)
    hvd.shutdown()
    return ok


def test_hierarchical_allreduce_and_allgather_match_flat_results():
    assert all(run_parallel(_two_hosts, np=4, args=(True,), timeout=240))


def test_same_layout_without_the_hierarchical_flags():
    assert all(run_parallel(_two_hosts, np=4, args=(False,), timeout=240))


def test_fusion_buffer_is_kept_until_the_threshold_changes():
    from horovod_b200 import _C
    MB = 1 << 20
    sizes, reallocs = _C.testing.fusion_buffer_probe([
        (1 * MB, 64 * MB),    # first use: sized for the threshold
        (10 * MB, 64 * MB),   # fits: kept
        (64 * MB, 64 * MB),   # fits exactly: kept
        (80 * MB, 64 * MB),   # larger than the threshold: grows to the request
        (1 * MB, 64 * MB),    # still fine for this threshold: kept
        (1 * MB, 8 * MB),     # the autotuner shrank the threshold: a smaller buffer
        (2 * MB, 8 * MB),     # kept
        (1 * MB, 128 * MB),   # threshold raised: grows again
    ])
    assert sizes == [64 * MB, 64 * MB, 64 * MB, 80 * MB, 80 * MB, 8 * MB, 8 * MB, 128 * MB]
    assert reallocs == 4
