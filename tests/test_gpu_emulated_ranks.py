"""The cross-rank kernel protocols on ONE GPU: the kernels of 2 to 8 "ranks"
run as one cooperative launch (grid = CTAs per rank x ranks), every rank on
its own slice of one device buffer, so that flag waits, chunk counters, launch
credits, region layouts and the host-side exchange planner are exercised
without a second GPU. What runs is the production kernel body (peer loads and
stores; multimem cannot be emulated). Every result is compared with a plain
PyTorch computation on the same inputs; every wait is bounded (2 s) and the
kernels' status record must stay clean.

Parity: the multi-rank cases of test/parallel/test_torch.py (allreduce,
allgather, broadcast, alltoall, reducescatter variants), which the reference
runs on several processes.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu

CLEAN = (0, 0, 0, 0)


def _ext():
    from horovod_b200 import _C
    if not hasattr(_C, "emulated_allreduce"):
        raise RuntimeError("the extension was built without the emulation entry points")
    return _C


def _dev():
    return torch.device("cuda", 0)


def _rand(seed, n, dtype):
    g = torch.Generator().manual_seed(seed)
    if dtype == torch.int32:
        return torch.randint(-1000, 1000, (n,), generator=g, dtype=torch.int32)
    return torch.randn(n, generator=g, dtype=torch.float32).to(dtype)


@pytest.mark.parametrize("world", [2, 3, 4, 8])
@pytest.mark.parametrize("algo,sub_chunk_kb", [("oneshot", 0), ("twoshot", 0), ("twoshot", 4)])
def test_fused_allreduce_protocols(world, algo, sub_chunk_kb):
    """One-shot (one barrier, everybody reads everybody), two-shot in one step
    and two-shot pipelined over 4 KB sub-chunks (packed / reduced counters),
    on a list of tensors of awkward sizes, with pre- and postscale."""
    C = _ext()
    sizes = [1001, 7, (1 << 16) + 3, 1, 40000]
    pre, post = 0.5, 0.25
    host = [[_rand(100 * r + i, n, torch.float32) for i, n in enumerate(sizes)]
            for r in range(world)]
    ranks = [[t.to(_dev()) for t in lst] for lst in host]
    status = C.emulated_allreduce(ranks, algo=algo, ctas=4, sub_chunk_kb=sub_chunk_kb,
                                  prescale=pre, postscale=post)
    assert tuple(status) == CLEAN
    for i in range(len(sizes)):
        want = sum((host[r][i] * pre).double() for r in range(world)) * post
        for r in range(world):
            got = ranks[r][i].cpu().double()
            assert torch.allclose(got, want, rtol=1e-5, atol=1e-5), (world, algo, i, r)


@pytest.mark.parametrize("world", [2, 5])
def test_fused_allreduce_dtypes_and_repeated_launches(world):
    """int32 (exact), bf16 tensors and fp32 tensors with a bf16 wire; three
    launches in a row on the same staging area (epochs keep counting up)."""
    C = _ext()
    ints = [[_rand(7 * r + i, n, torch.int32).to(_dev()) for i, n in enumerate([333, 4097])]
            for r in range(world)]
    before = [[t.clone() for t in lst] for lst in ints]
    assert tuple(C.emulated_allreduce(ints, algo="twoshot", ctas=2, sub_chunk_kb=4,
                                      launches=3)) == CLEAN
    for i in range(2):
        total = sum(before[r][i] for r in range(world))
        for r in range(world):
            # every launch sums the ranks' current values again: total * world^2
            assert torch.equal(ints[r][i], total * world * world)

    bf = [[_rand(11 * r + 1, 50001, torch.bfloat16).to(_dev())] for r in range(world)]
    ref = sum(t[0].double() for t in bf)
    assert tuple(C.emulated_allreduce(bf, algo="oneshot", ctas=4)) == CLEAN
    for r in range(world):
        assert torch.allclose(bf[r][0].double(), ref, rtol=4e-2, atol=4e-2 * world)

    fp = [[_rand(13 * r + 2, 30011, torch.float32).to(_dev())] for r in range(world)]
    ref = sum(t[0].to(torch.bfloat16).double() for t in fp)
    assert tuple(C.emulated_allreduce(fp, algo="twoshot", ctas=4, bf16_wire=True)) == CLEAN
    for r in range(world):
        assert torch.allclose(fp[r][0].double(), ref, rtol=4e-2, atol=4e-2 * world)


@pytest.mark.parametrize("world", [2, 3, 4, 8])
def test_pushed_reducescatter(world):
    """Shards pushed into the owners' region slots chunk by chunk (4 KB chunks,
    so every launch announces many), ragged rows, a region so small that the
    shards take several windows, pre/postscale, 16-bit and integer types."""
    C = _ext()
    cases = [(torch.float32, 5 * world + 3, 1001, 0.5, 2.0, 64),   # several windows
             (torch.float32, world, 1, 1.0, 1.0, 64),              # one element per rank
             (torch.float32, world - 1, 5, 1.0, 1.0, 64),          # a rank with an empty shard
             (torch.bfloat16, 2 * world + 1, 10003, 1.0, 1.0, 256),
             (torch.int32, 4 * world + 1, 3333, 1.0, 1.0, 128)]
    for ci, (dtype, rows, width, pre, post, region_kb) in enumerate(cases):
        host = [_rand(17 * r + ci, rows * width, dtype).view(rows, width) for r in range(world)]
        outs, status = C.emulated_reducescatter([t.to(_dev()) for t in host], ctas=4, chunk_kb=4,
                                                prescale=pre, postscale=post,
                                                region_kb=region_kb)
        assert tuple(status) == CLEAN, (world, ci)
        ref = sum((t.double() * pre).to(dtype).double() for t in host) * post
        base, extra = rows // world, rows % world
        for r in range(world):
            lo = r * base + min(r, extra)
            hi = lo + base + (1 if r < extra else 0)
            assert tuple(outs[r].shape) == (hi - lo, width)
            if dtype == torch.int32:
                assert torch.equal(outs[r].cpu().double(), ref[lo:hi])
            else:
                tol = 1e-5 if dtype == torch.float32 else 4e-2
                assert torch.allclose(outs[r].cpu().double(), ref[lo:hi], rtol=tol,
                                      atol=tol * world), (world, ci, r)


@pytest.mark.parametrize("world", [2, 3, 4, 8])
@pytest.mark.parametrize("push", [False, True])
def test_exchange_allgather_broadcast_alltoall(world, push):
    """The exchange kernel behind allgather, broadcast and alltoall with the
    production planner: pulled (staged in the sender's region) and pushed
    (stored into the receivers' regions), several chunks per CTA and block
    (64 KB chunks, two CTAs), a region small enough for several rounds (launch
    credits between them), uneven rows, empty blocks and odd byte counts."""
    C = _ext()
    # allgather with a different number of rows on every rank (1.2 MB x (r + 1))
    host = [_rand(23 * r, (r + 1) * 8000 * 37, torch.float32).view(-1, 37) for r in range(world)]
    outs, status, rounds = C.emulated_exchange("allgather", [t.to(_dev()) for t in host],
                                               push=push, ctas=2, chunk_kb=64, region_kb=2048)
    assert tuple(status) == CLEAN
    assert rounds > 1  # the region does not hold everything at once
    want = torch.cat(host)
    for r in range(world):
        assert torch.equal(outs[r].cpu(), want), (world, push, r)

    # broadcast from the last rank, odd length, bytes
    src = torch.arange(1 << 18, dtype=torch.int32).mul_(3)[: (1 << 18) - 5]
    ins = [src.to(_dev()) if r == world - 1 else torch.zeros_like(src).to(_dev())
           for r in range(world)]
    outs, status, _ = C.emulated_exchange("broadcast", ins, root=world - 1, push=push, ctas=4,
                                          chunk_kb=64, region_kb=512)
    assert tuple(status) == CLEAN
    for r in range(world):
        assert torch.equal(outs[r].cpu(), src), (world, push, r)

    # alltoall with uneven splits, zeros included
    splits = [[(r + 2 * p) % 4 for p in range(world)] for r in range(world)]
    width = 515
    host = [_rand(31 * r + 5, sum(splits[r]) * width, torch.float32).view(-1, width)
            for r in range(world)]
    outs, status, _ = C.emulated_exchange("alltoall", [t.to(_dev()) for t in host],
                                          splits=splits, push=push, ctas=4, chunk_kb=64,
                                          region_kb=64)
    assert tuple(status) == CLEAN
    for me in range(world):
        pieces = []
        for r in range(world):
            off = sum(splits[r][:me])
            pieces.append(host[r][off:off + splits[r][me]])
        assert torch.equal(outs[me].cpu(), torch.cat(pieces)), (world, push, me)
