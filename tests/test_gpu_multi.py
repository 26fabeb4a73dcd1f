"""Multi-GPU checks of the NVLink kernels against plain PyTorch fp32/fp64
references computed from every rank's seeded inputs. Runs as child processes,
one per GPU; skipped when fewer GPUs are present."""
import os

import pytest
import torch

from parallel_utils import run_parallel

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def _ngpu():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def _world():
    n = _ngpu()
    return 8 if n >= 8 else 4 if n >= 4 else 2


def _inputs(seed_rank, n, dtype):
    g = torch.Generator().manual_seed(1000 + seed_rank)
    if dtype.is_floating_point:
        return torch.randn(n, generator=g, dtype=torch.float32).to(dtype)
    return torch.randint(-50, 50, (n,), generator=g).to(dtype)


def _collectives(rank, size, algo):
    os.environ["HOROVOD_ALLREDUCE_ALGO"] = algo
    os.environ["HOROVOD_SPIN_TIMEOUT_MS"] = "5000"
    import horovod_b200.torch as hvd
    from horovod_b200 import _C
    hvd.init()
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    report = {}
    sizes = [1, 17, 4096, 100003, (1 << 20) + 5]
    for dtype in (torch.float32, torch.bfloat16, torch.float16, torch.int32, torch.float64):
        for n in sizes:
            if algo == "nvls" and dtype in (torch.int32, torch.float64):
                continue
            x = _inputs(rank, n, dtype).to(dev)
            out = hvd.allreduce(x, op=hvd.Sum, name="ar.%s.%d" % (dtype, n))
            ref = sum(_inputs(r, n, dtype).double() for r in range(size))
            tol = {torch.float32: 1e-5, torch.float64: 1e-12, torch.int32: 0,
                   torch.bfloat16: 4e-2, torch.float16: 8e-3}[dtype]
            err = (out.double().cpu() - ref).abs().max().item()
            scale = max(1.0, ref.abs().max().item())
            assert err <= tol * scale * size, (str(dtype), n, err)
    # Average with pre/post scale over a fused group of odd-sized tensors.
    shapes = [3, 129, 2048, 77777, 5]
    xs = [_inputs(rank * 31 + i, s, torch.float32).to(dev) for i, s in enumerate(shapes)]
    outs = hvd.grouped_allreduce(xs, op=hvd.Average, name="grp")
    for i, (s, o) in enumerate(zip(shapes, outs)):
        ref = sum(_inputs(r * 31 + i, s, torch.float32).double() for r in range(size)) / size
        assert (o.double().cpu() - ref).abs().max().item() < 1e-5
    # fp32 gradients with a 16-bit wire format (cast fused into the kernel)
    for wire, tol in ((torch.bfloat16, 4e-2), (torch.float16, 8e-3)):
        xs = [_inputs(rank * 13 + i, s, torch.float32).to(dev) for i, s in enumerate(shapes)]
        hvd.synchronize(hvd.grouped_allreduce_async_(xs, op=hvd.Average, wire_dtype=wire,
                                                     name="wire.%s" % wire))
        for i, (s, o) in enumerate(zip(shapes, xs)):
            assert o.dtype == torch.float32
            ref = sum(_inputs(r * 13 + i, s, torch.float32).to(wire).double()
                      for r in range(size)) / size
            assert (o.double().cpu() - ref).abs().max().item() < tol * size, (str(wire), s)
    # allgather with a different dim 0 on every rank
    rows = rank + 1
    ag = hvd.allgather(torch.full((rows, 3), float(rank), device=dev), name="ag")
    exp = torch.cat([torch.full((r + 1, 3), float(r)) for r in range(size)])
    assert torch.equal(ag.cpu(), exp)
    # broadcast from the last rank, odd length
    b = torch.arange(1001, device=dev, dtype=torch.float32) * (rank + 1)
    hvd.broadcast_(b, root_rank=size - 1, name="bc")
    assert torch.equal(b.cpu(), torch.arange(1001, dtype=torch.float32) * size)
    # alltoall with uneven splits: rank r sends (p + 1) rows to rank p
    splits = [p + 1 for p in range(size)]
    src = torch.cat([torch.full((p + 1, 2), float(rank * 100 + p)) for p in range(size)]).to(dev)
    out, recv = hvd.alltoall(src, splits=splits, name="a2a")
    assert recv.tolist() == [rank + 1] * size
    exp = torch.cat([torch.full((rank + 1, 2), float(r * 100 + rank)) for r in range(size)])
    assert torch.equal(out.cpu(), exp)
    # alltoall without splits (even split, no split table exchanged): rank r
    # holds size * (r + 1) rows and sends r + 1 of them to every peer; twice,
    # the second time from the cached response
    for it in range(2):
        mine = (torch.arange(size * (rank + 1) * 3, dtype=torch.float32) + 1000 * rank + it) \
            .view(size * (rank + 1), 3)
        out = hvd.alltoall(mine.to(dev), name="a2a.even")
        exp = torch.cat([((torch.arange(size * (r + 1) * 3, dtype=torch.float32) + 1000 * r + it)
                          .view(size * (r + 1), 3))[rank * (r + 1):(rank + 1) * (r + 1)]
                         for r in range(size)])
        assert torch.equal(out.cpu(), exp)
    # reducescatter with ragged shards
    rs_rows = 2 * size + 1
    x = _inputs(rank + 500, rs_rows * 5, torch.float32).view(rs_rows, 5).to(dev)
    out = hvd.reducescatter(x, op=hvd.Sum, name="rs")
    full = sum(_inputs(r + 500, rs_rows * 5, torch.float32).view(rs_rows, 5).double()
               for r in range(size))
    base, extra = divmod(rs_rows, size)
    start = rank * base + min(rank, extra)
    mine = full[start:start + base + (1 if rank < extra else 0)]
    assert (out.double().cpu() - mine).abs().max().item() < 1e-5
    report["backend"] = hvd.gpu_backend()
    report["launches"] = _C.kernel_launch_count()
    torch.cuda.synchronize()
    hvd.shutdown()
    return report


@pytest.mark.parametrize("algo", ["auto", "oneshot", "twoshot", "nvls"])
def test_collectives_against_reference(algo):
    out = run_parallel(_collectives, np=_world(), args=(algo,), timeout=300)
    for rep in out:
        assert rep["backend"].startswith("symm"), rep["backend"]
        assert rep["launches"] > 0


def _adasum(rank, size):
    os.environ["HOROVOD_SPIN_TIMEOUT_MS"] = "5000"
    import horovod_b200.torch as hvd
    hvd.init()
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)

    def oracle(vs):
        vs = [v.double() for v in vs]
        while len(vs) > 1:
            nxt = []
            for i in range(0, len(vs), 2):
                a, b = vs[i], vs[i + 1]
                dot, na, nb = (a * b).sum(), (a * a).sum(), (b * b).sum()
                ca = 1 - dot / (2 * na) if na > 0 else 1.0
                cb = 1 - dot / (2 * nb) if nb > 0 else 1.0
                nxt.append(ca * a + cb * b)
            vs = nxt
        return vs[0]

    shapes = [5, 1000, 33333]
    xs = [_inputs(rank * 7 + i, s, torch.float32).to(dev) for i, s in enumerate(shapes)]
    outs = hvd.grouped_allreduce(xs, op=hvd.Adasum, name="adasum")
    for i, (s, o) in enumerate(zip(shapes, outs)):
        ref = oracle([_inputs(r * 7 + i, s, torch.float32) for r in range(size)])
        assert (o.double().cpu() - ref).abs().max().item() < 1e-4, (s,)
    # identical inputs combine to the same vector (average-like behaviour)
    same = torch.arange(64, dtype=torch.float32, device=dev) + 1
    o = hvd.allreduce(same, op=hvd.Adasum, name="adasum.same")
    assert (o - same).abs().max().item() < 1e-4
    torch.cuda.synchronize()
    hvd.shutdown()
    return True


def test_adasum_matches_pairwise_oracle():
    assert all(run_parallel(_adasum, np=_world(), timeout=300))


def _nccl_backend(rank, size):
    os.environ["HOROVOD_GPU_BACKEND"] = "nccl"
    import horovod_b200.torch as hvd
    hvd.init()
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    xs = [torch.full((n,), float(rank + 1), device=dev) for n in (7, 4096, 100001)]
    outs = hvd.grouped_allreduce(xs, op=hvd.Sum, name="g")
    tot = float(sum(range(1, size + 1)))
    ok = all(bool((o == tot).all()) for o in outs)
    m = hvd.allreduce(torch.full((9,), float(rank), device=dev), op=hvd.Max, name="max")
    ok = ok and bool((m == size - 1).all())
    backend = hvd.gpu_backend()
    torch.cuda.synchronize()
    hvd.shutdown()
    return ok, backend


def test_nccl_baseline_path():
    for ok, backend in run_parallel(_nccl_backend, np=2, timeout=300):
        assert ok and backend.startswith("nccl")


def _long_lists_and_heap(rank, size, inline):
    os.environ["HOROVOD_INLINE_DESCRIPTORS"] = inline
    os.environ["HOROVOD_SPIN_TIMEOUT_MS"] = "5000"
    import horovod_b200.torch as hvd
    hvd.init()
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    # A fused list longer than what fits the kernel parameters (descriptor ring).
    shapes = [1, 3, 17, 255, 256, 257, 4099, 65537, 9, 300001] * 10
    xs = [_inputs(rank * 211 + i, s, torch.float32).to(dev) for i, s in enumerate(shapes)]
    outs = hvd.grouped_allreduce(xs, op=hvd.Sum, name="long")
    for i, (s, o) in enumerate(zip(shapes, outs)):
        ref = sum(_inputs(r * 211 + i, s, torch.float32).double() for r in range(size))
        assert (o.double().cpu() - ref).abs().max().item() < 1e-5 * size, ("long", i, s)
    # In place on the symmetric heap: one tensor, an odd length, 16-bit types.
    for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 4e-2), (torch.float16, 8e-3),
                       (torch.float64, 1e-12)):
        for n in (5, 4096, 100003, (1 << 20) + 3):
            z = hvd.symmetric_empty(n, dtype=dtype)
            assert z.is_cuda and z.numel() == n and z.data_ptr() % 256 == 0
            z.copy_(_inputs(rank, n, dtype).to(dev))
            out = hvd.allreduce_(z, op=hvd.Average, name="heap.%s.%d" % (dtype, n))
            assert out.data_ptr() == z.data_ptr()
            ref = sum(_inputs(r, n, dtype).double() for r in range(size)) / size
            err = (z.double().cpu() - ref).abs().max().item()
            assert err <= tol * max(1.0, ref.abs().max().item()) * size, (str(dtype), n, err)
    # Many views of one flat buffer (what the optimizer reduces), unordered,
    # with gaps and ragged lengths; neighbours merge into ranges.
    flat = hvd.symmetric_empty(1 << 20)
    flat.copy_(_inputs(rank + 50, 1 << 20, torch.float32).to(dev))
    before = flat.clone()
    cuts = [(0, 1000), (1000, 4096), (8192, 8192 + 77), (16384, 300000), (300000, 300004),
            (400000, 1 << 20)]
    cuts += [(320000 + 64 * i, 320000 + 64 * i + 64) for i in range(60)]
    views = [flat[a:b] for a, b in reversed(cuts)]
    hvd.grouped_allreduce_(views, op=hvd.Sum, name="views")
    full = sum(_inputs(r + 50, 1 << 20, torch.float32).double() for r in range(size))
    covered = torch.zeros(1 << 20, dtype=torch.bool)
    for a, b in cuts:
        covered[a:b] = True
    got = flat.double().cpu()
    assert (got[covered] - full[covered]).abs().max().item() < 1e-5 * size
    assert torch.equal(flat.cpu()[~covered], before.cpu()[~covered]), "gaps were touched"
    # A tensor outside the heap in the same group: everybody stages.
    mixed = [flat[:128], torch.ones(64, device=dev)]
    flat[:128] = float(rank)
    hvd.grouped_allreduce_(mixed, op=hvd.Sum, name="mixed")
    assert bool((mixed[0] == sum(range(size))).all()) and bool((mixed[1] == size).all())
    # Reduce-scatter straight out of a symmetric input (16-byte aligned shards)
    # and through staging (ragged shards).
    for rows, cols in ((size * 1024, 8), (size * 5 + 1, 3)):
        src = hvd.symmetric_empty(rows, cols)
        src.copy_(_inputs(rank + 9, rows * cols, torch.float32).view(rows, cols).to(dev))
        keep = src.clone()
        got = hvd.reducescatter(src, op=hvd.Average, name="heap.rs.%d" % rows)
        full = sum(_inputs(r + 9, rows * cols, torch.float32).double()
                   for r in range(size)).view(rows, cols) / size
        base, extra = divmod(rows, size)
        lo = rank * base + min(rank, extra)
        hi = lo + base + (1 if rank < extra else 0)
        assert (got.double().cpu() - full[lo:hi]).abs().max().item() < 1e-5
        assert torch.equal(src, keep), "reducescatter changed its input"
    info = hvd.gpu_backend()
    torch.cuda.synchronize()
    hvd.shutdown()
    return info


@pytest.mark.parametrize("inline", ["1", "0"])
def test_long_tensor_lists_and_symmetric_heap(inline):
    if _ngpu() < 2:
        pytest.skip("needs 2 GPUs")
    for info in run_parallel(_long_lists_and_heap, np=_world(), args=(inline,), timeout=300):
        assert info.startswith("symm")


def _symmetric_gradients(rank, size):
    os.environ["HOROVOD_SPIN_TIMEOUT_MS"] = "5000"
    import torch.nn as nn
    import torch.nn.functional as F
    import horovod_b200.torch as hvd
    from horovod_b200 import _C
    hvd.init()
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)

    def net():
        torch.manual_seed(0)
        return nn.Sequential(nn.Conv2d(3, 8, 3, padding=1), nn.BatchNorm2d(8), nn.ReLU(),
                             nn.Flatten(), nn.Linear(8 * 8 * 8, 10))

    def data(r):
        g = torch.Generator().manual_seed(7 + r)
        return torch.randn(4, 3, 8, 8, generator=g), torch.randint(0, 10, (4,), generator=g)

    model = net().to(dev).to(memory_format=torch.channels_last)
    opt = hvd.DistributedOptimizer(torch.optim.SGD(model.parameters(), lr=0.1, momentum=0.9),
                                   named_parameters=model.named_parameters(),
                                   symmetric_gradients=True)
    ptrs = {n: p.grad.data_ptr() for n, p in model.named_parameters()}
    assert _C.symm_heap_info()["used"] > 0
    x, y = data(rank)
    for _ in range(3):
        opt.zero_grad()
        F.cross_entropy(model(x.to(dev)), y.to(dev)).backward()
        opt.step()
    # gradients stayed views of the flat buffer through zero_grad/backward/step
    assert all(p.grad.data_ptr() == ptrs[n] for n, p in model.named_parameters())

    ref = net()
    ropt = torch.optim.SGD(ref.parameters(), lr=0.1, momentum=0.9)
    for _ in range(3):
        ropt.zero_grad()
        for r in range(size):
            xr, yr = data(r)
            # per-rank batch statistics: forward each rank's batch separately
            (F.cross_entropy(ref(xr), yr) / size).backward()
        ropt.step()
    ok = all(torch.allclose(a.detach().cpu(), b.detach(), atol=2e-4)
             for a, b in zip(model.parameters(), ref.parameters()))
    torch.cuda.synchronize()
    hvd.shutdown()
    return ok


def test_optimizer_with_symmetric_gradients():
    if _ngpu() < 2:
        pytest.skip("needs 2 GPUs")
    assert all(run_parallel(_symmetric_gradients, np=2, timeout=300))


def _asymmetric_use(rank, size):
    os.environ["HOROVOD_SPIN_TIMEOUT_MS"] = "1000"
    import horovod_b200.torch as hvd
    hvd.init()
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    z = hvd.symmetric_empty(4096)
    z.fill_(1.0)
    hvd.allreduce_(z, op=hvd.Sum, name="warm")  # both ranks symmetric: fine
    ok = bool((z == size).all())
    # Rank 0 hands in the symmetric tensor, rank 1 an ordinary one: the
    # kernels notice (token mismatch / bounded wait) and both ranks get an
    # error instead of a wrong sum.
    x = z if rank == 0 else torch.ones(4096, device=dev)
    try:
        hvd.allreduce_(x, op=hvd.Sum, name="mixed.up")
        torch.cuda.synchronize()
        # the error may surface at the next op
        hvd.allreduce_(torch.ones(8, device=dev), op=hvd.Sum, name="after")
        torch.cuda.synchronize()
        failed = False
    except Exception as e:  # HorovodInternalError or RuntimeError
        failed = True
        msg = str(e)
        if rank == 0:
            ok = ok and "symmetric" in msg
    try:
        hvd.shutdown()
    except Exception:
        pass
    return ok, failed


def test_asymmetric_use_of_symmetric_memory_is_reported():
    if _ngpu() < 2:
        pytest.skip("needs 2 GPUs")
    out = run_parallel(_asymmetric_use, np=2, timeout=300)
    # The rank that addressed peers by symmetric offset must report it; the
    # other rank either times out on its next collective or sees the shutdown.
    assert out[0] == (True, True), out
    assert out[1][0], out


def _exchange_large(rank, size, copy_engine_min):
    """Large and mixed exchange rounds with small chunks, so every launch
    publishes many chunk counters, and enough launches in a row that both
    exchange regions are reused several times (credit waits).
    copy_engine_min: from how many bytes the rounds move their blocks with
    copy-engine peer copies ("0": never, so the kernel pulls or pushes)."""
    os.environ["HOROVOD_EXCHANGE_CHUNK_KB"] = "64"
    os.environ["HOROVOD_EXCHANGE_COPY_ENGINE_MIN_BYTES"] = copy_engine_min
    os.environ["HOROVOD_SPIN_TIMEOUT_MS"] = "5000"
    import horovod_b200.torch as hvd
    hvd.init()
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    n = (3 << 20) + 5  # 12 MB per rank and a ragged tail
    ok = True
    for it in range(3):
        # allgather with a different dim 0 on every rank
        x = _inputs(rank + it, n + rank * 1001, torch.float32).to(dev)
        got = hvd.allgather(x, name="xl.ag")
        exp = torch.cat([_inputs(r + it, n + r * 1001, torch.float32) for r in range(size)])
        ok = ok and torch.equal(got.cpu(), exp)
        # broadcast from the last rank
        b = _inputs(rank + it, 5 * n, torch.float32).to(dev)
        hvd.broadcast_(b, root_rank=size - 1, name="xl.bc")
        ok = ok and torch.equal(b.cpu(), _inputs(size - 1 + it, 5 * n, torch.float32))
    # uneven alltoall
    splits = torch.tensor([(rank + p) % 3 + 1 for p in range(size)], dtype=torch.int32)
    rows = int(splits.sum())
    send = _inputs(rank + 40, rows * (1 << 20), torch.float32).view(rows, 1 << 20).to(dev)
    recv, rsplits = hvd.alltoall(send, splits=splits, name="xl.a2a")
    pieces = []
    for r in range(size):
        s = [(r + p) % 3 + 1 for p in range(size)]
        full = _inputs(r + 40, sum(s) * (1 << 20), torch.float32).view(sum(s), 1 << 20)
        off = sum(s[:rank])
        pieces.append(full[off:off + s[rank]])
    ok = ok and torch.equal(recv.cpu(), torch.cat(pieces))
    # small tensors (20-60 KB) fused with 12 MB ones in one response, on
    # storage that is only 4-byte aligned
    counts = [5003, 3 << 20, 15001, (3 << 20) + 3, 9999]
    base = [_inputs(rank * 7 + i, c + 1, torch.float32).to(dev) for i, c in enumerate(counts)]
    handles = [hvd.allgather_async(t[1:], name="xl.mix.%d" % i) for i, t in enumerate(base)]
    for i, (h, c) in enumerate(zip(handles, counts)):
        got = hvd.synchronize(h)
        exp = torch.cat([_inputs(r * 7 + i, c + 1, torch.float32)[1:] for r in range(size)])
        ok = ok and torch.equal(got.cpu(), exp)
    # several broadcasts in flight, one with a 40 KB tensor behind big ones
    ts = [_inputs(rank + 90 + i, c, torch.float32).to(dev)
          for i, c in enumerate([2 << 20, 10000, (4 << 20) + 1, 10240])]
    hs = [hvd.broadcast_async_(t, root_rank=i % size, name="xl.bcs.%d" % i)
          for i, t in enumerate(ts)]
    for i, (h, t) in enumerate(zip(hs, ts)):
        hvd.synchronize(h)
        ok = ok and torch.equal(t.cpu(), _inputs(i % size + 90 + i, t.numel(), torch.float32))
    # a byte tensor of odd length and odd offset
    raw = torch.arange(100001, dtype=torch.uint8).add_(rank).to(dev)[3:]
    got = hvd.allgather(raw, name="xl.bytes")
    exp = torch.cat([torch.arange(100001, dtype=torch.uint8).add_(r)[3:] for r in range(size)])
    ok = ok and torch.equal(got.cpu(), exp)
    # a small op in between
    small = hvd.allgather(torch.full((3,), float(rank), device=dev), name="xl.small")
    ok = ok and small.cpu().tolist() == [float(r) for r in range(size) for _ in range(3)]
    torch.cuda.synchronize()
    hvd.shutdown()
    return ok


@pytest.mark.parametrize("copy_engine_min", ["0", str(1 << 20)])
def test_large_and_mixed_exchange_rounds(copy_engine_min):
    if _ngpu() < 2:
        pytest.skip("needs 2 GPUs")
    assert all(run_parallel(_exchange_large, np=_world(), args=(copy_engine_min,), timeout=300))


def _reducescatter_push(rank, size):
    """Reduce-scatter of tensors in ordinary memory: shards are pushed into the
    owners' exchange regions. A small staging area forces several windows per
    tensor; small chunks make every launch announce many chunks."""
    os.environ["HOROVOD_SYMM_BUFFER_MB"] = "64"
    os.environ["HOROVOD_EXCHANGE_CHUNK_KB"] = "64"
    os.environ["HOROVOD_SPIN_TIMEOUT_MS"] = "5000"
    import horovod_b200.torch as hvd
    hvd.init()
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    ok = True
    cases = [(torch.float32, 5 * size + 3, 700001, 1.0, 1.0),    # several windows, ragged rows
             (torch.float32, size, 1, 1.0, 1.0),                # one element per rank
             (torch.float32, size - 1, 5, 1.0, 1.0),            # a rank with an empty shard
             (torch.bfloat16, 2 * size + 1, 100003, 0.5, 2.0),  # 16-bit, pre/postscale
             (torch.float16, 3 * size, 4099, 1.0, 0.25),
             (torch.int32, 4 * size + 1, 33333, 1.0, 1.0),
             (torch.float64, size + 1, 77777, 1.0, 1.0)]
    for it in range(2):
        for ci, (dtype, rows, width, pre, post) in enumerate(cases):
            n = rows * width
            full = _inputs(rank * 17 + ci + it, n + 1, dtype)
            # a view that starts one element into the allocation: not 16-byte aligned
            x = full.to(dev)[1:].view(rows, width)
            out = hvd.reducescatter(x, op=hvd.Sum, prescale_factor=pre, postscale_factor=post,
                                    name="rsp.%d" % ci)
            ref = sum((_inputs(r * 17 + ci + it, n + 1, dtype)[1:].view(rows, width).double() * pre)
                      .to(dtype).double() for r in range(size)) * post
            base, extra = rows // size, rows % size
            lo = rank * base + min(rank, extra)
            hi = lo + base + (1 if rank < extra else 0)
            tol = {torch.float32: 1e-5, torch.float64: 1e-12, torch.int32: 0,
                   torch.bfloat16: 4e-2, torch.float16: 8e-3}[dtype]
            if tuple(out.shape) != (hi - lo, width):
                ok = False
                continue
            if hi > lo:
                err = (out.double().cpu() - ref[lo:hi]).abs().max().item()
                scale = max(1.0, ref.abs().max().item())
                ok = ok and err <= tol * scale * size
    # interleaved with the other users of the exchange regions
    g = hvd.allgather(torch.full((2,), float(rank), device=dev), name="rsp.ag")
    ok = ok and g.cpu().tolist() == [float(r) for r in range(size) for _ in range(2)]
    torch.cuda.synchronize()
    hvd.shutdown()
    return ok


def test_reducescatter_from_ordinary_memory():
    if _ngpu() < 2:
        pytest.skip("needs 2 GPUs")
    assert all(run_parallel(_reducescatter_push, np=_world(), timeout=300))


def _grouped_push(rank, size):
    """grouped_reducescatter / grouped_allgather of device tensors: the group
    is negotiated as one unit; the tensors of one dtype leave in one kernel
    launch; results against an fp64 PyTorch sum of the same inputs."""
    os.environ["HOROVOD_SPIN_TIMEOUT_MS"] = "5000"
    os.environ["HOROVOD_EXCHANGE_CHUNK_KB"] = "64"
    import horovod_b200.torch as hvd
    from horovod_b200 import _C
    hvd.init()
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    bad = []  # labels of the checks that failed
    shapes = [(5 * size + 3, 1001), (size, 1), (size - 1, 5), (3 * size, 4099), (2, 3),
              (7 * size + 1, 33333)]
    for it in range(3):
        for dtype, pre, post in [(torch.float32, 1.0, 1.0), (torch.bfloat16, 0.5, 2.0)]:
            def make(r):
                return [_inputs(r * 31 + i + it, rows * w + 1, dtype)[1:].view(rows, w)
                        for i, (rows, w) in enumerate(shapes)]
            # views that start one element into their allocation: not 16-byte aligned
            xs = [_inputs(rank * 31 + i + it, rows * w + 1, dtype).to(dev)[1:].view(rows, w)
                  for i, (rows, w) in enumerate(shapes)]
            hvd.allreduce(torch.zeros(1, device=dev), name="gp.sync")  # drain earlier work
            torch.cuda.synchronize()
            before = _C.kernel_launch_count()
            outs = hvd.grouped_reducescatter(xs, op=hvd.Sum, prescale_factor=pre,
                                             postscale_factor=post, name="gp.rs.%d.%s" % (it, str(dtype)[6:]))
            torch.cuda.synchronize()
            launches = _C.kernel_launch_count() - before
            if launches != 1:
                bad.append("launches=%d it=%d %s" % (launches, it, dtype))
            everyone = [make(r) for r in range(size)]
            tol = 1e-5 if dtype == torch.float32 else 4e-2
            for i, (rows, w) in enumerate(shapes):
                ref = sum((everyone[r][i].double() * pre).to(dtype).double()
                          for r in range(size)) * post
                base, extra = rows // size, rows % size
                lo = rank * base + min(rank, extra)
                hi = lo + base + (1 if rank < extra else 0)
                if tuple(outs[i].shape) != (hi - lo, w) or outs[i].dtype != dtype:
                    bad.append("shape %s it=%d tensor=%d" % (tuple(outs[i].shape), it, i))
                    continue
                if hi > lo:
                    err = (outs[i].double().cpu() - ref[lo:hi]).abs().max().item()
                    if err > tol * max(1.0, ref.abs().max().item()) * size:
                        bad.append("value err=%g it=%d tensor=%d %s" % (err, it, i, dtype))
    # mixed dtypes in one group: outputs come back in the order of the inputs
    mixed = [torch.full((size, 2), float(rank + 1), device=dev),
             torch.full((2 * size,), rank + 1, dtype=torch.int32, device=dev),
             torch.full((size, 3), float(rank + 1), dtype=torch.float16, device=dev)]
    outs = hvd.grouped_reducescatter(mixed, op=hvd.Sum, name="gp.mixed")
    tot = size * (size + 1) // 2
    if [o.dtype for o in outs] != [torch.float32, torch.int32, torch.float16]:
        bad.append("mixed dtypes %s" % [o.dtype for o in outs])
    if [tuple(o.shape) for o in outs] != [(1, 2), (2,), (1, 3)]:
        bad.append("mixed shapes %s" % [tuple(o.shape) for o in outs])
    if not all(bool((o.cpu().double() == tot).all()) for o in outs):
        bad.append("mixed values")
    gathered = hvd.grouped_allgather([torch.full((rank + 1, 3), float(rank), device=dev),
                                      torch.arange(4, device=dev) + rank,
                                      torch.full((2,), float(rank), device=dev)], name="gp.ag")
    if not torch.equal(gathered[0].cpu(), torch.cat([torch.full((r + 1, 3), float(r))
                                                     for r in range(size)])):
        bad.append("allgather 0")
    if not torch.equal(gathered[1].cpu(), torch.cat([torch.arange(4) + r for r in range(size)])):
        bad.append("allgather 1")
    if gathered[2].cpu().tolist() != [float(r) for r in range(size) for _ in range(2)]:
        bad.append("allgather 2")
    torch.cuda.synchronize()
    hvd.shutdown()
    return bad


def test_grouped_reducescatter_is_one_launch():
    if _ngpu() < 2:
        pytest.skip("needs 2 GPUs")
    failures = run_parallel(_grouped_push, np=_world(), timeout=300)
    assert all(f == [] for f in failures), failures


def _two_hosts_on_gpus(rank, size):
    """Four GPUs laid out as two hosts of two ranks (distinct cross ranks on
    one box): local_size != size, so the NCCL path is selected, and with
    HOROVOD_HIERARCHICAL_ALLREDUCE=1 every fused allreduce runs as
    ncclReduceScatter inside the host, ncclAllReduce across the hosts and
    ncclAllGather inside the host. Results against an fp64 sum."""
    local = 2
    os.environ.update({
        "HOROVOD_LOCAL_RANK": str(rank % local), "HOROVOD_LOCAL_SIZE": str(local),
        "HOROVOD_CROSS_RANK": str(rank // local), "HOROVOD_CROSS_SIZE": str(size // local),
        "HOROVOD_HOSTNAME": "host-%d" % (rank // local),
        "HOROVOD_HIERARCHICAL_ALLREDUCE": "1",
        "NCCL_NVLS_ENABLE": "0",
    })
    import horovod_b200.torch as hvd
    hvd.init()
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    ok = hvd.runtime_params()["hierarchy_usable"] and hvd.local_size() == local
    for it in range(2):
        for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 4e-2), (torch.int32, 0)):
            for n in (1, 3, 1001, (1 << 20) + 5):
                host = [_inputs(13 * r + n % 97 + it, n, dtype) for r in range(size)]
                out = hvd.allreduce(host[rank].to(dev), op=hvd.Sum,
                                    name="hier.%s.%d" % (str(dtype)[6:], n))
                ref = sum(h.double() for h in host)
                err = (out.double().cpu() - ref).abs().max().item()
                ok = ok and err <= tol * max(1.0, ref.abs().max().item()) * size
        # a fused group, averaged
        xs = [_inputs(rank * 5 + i + it, s, torch.float32).to(dev)
              for i, s in enumerate((3, 129, 77, 40000, 5))]
        outs = hvd.grouped_allreduce(xs, op=hvd.Average, name="hier.grp")
        for i, (s, o) in enumerate(zip((3, 129, 77, 40000, 5), outs)):
            ref = sum(_inputs(r * 5 + i + it, s, torch.float32).double() for r in range(size)) / size
            ok = ok and (o.double().cpu() - ref).abs().max().item() < 1e-5
    ok = ok and "nccl" in hvd.gpu_backend()
    torch.cuda.synchronize()
    hvd.shutdown()
    return ok


def test_hierarchical_allreduce_on_the_nccl_path():
    if _ngpu() < 4:
        pytest.skip("needs 4 GPUs")
    if os.environ.get("HOROVOD_TEST_HIERARCHICAL_NCCL") != "1":
        # The host-side twin (tests/test_hierarchical.py) runs everywhere; this
        # variant has not completed a run on GPUs yet (its first attempt was cut
        # short by the time limit of the call, before any result), so it is
        # opt-in until it has.
        pytest.skip("opt-in: set HOROVOD_TEST_HIERARCHICAL_NCCL=1")
    assert all(run_parallel(_two_hosts_on_gpus, np=4, timeout=300))


def _two_devices_per_rank(rank, size):
    """Every rank spreads a two-layer model over two of the box's GPUs (layer
    one on the first, layer two on the second) and trains it through
    DistributedOptimizer; gradients arrive from both devices. Compared with
    the same model trained in one piece on the concatenated batch."""
    os.environ["HOROVOD_SPIN_TIMEOUT_MS"] = "5000"
    import horovod_b200.torch as hvd
    hvd.init()
    d0, d1 = torch.device("cuda", 2 * rank), torch.device("cuda", 2 * rank + 1)
    torch.manual_seed(0)
    l1, l2 = torch.nn.Linear(16, 32), torch.nn.Linear(32, 4)
    ref1, ref2 = torch.nn.Linear(16, 32), torch.nn.Linear(32, 4)
    ref1.load_state_dict(l1.state_dict())
    ref2.load_state_dict(l2.state_dict())
    l1.to(d0)
    l2.to(d1)
    params = [("l1." + n, p) for n, p in l1.named_parameters()] + \
             [("l2." + n, p) for n, p in l2.named_parameters()]
    opt = hvd.DistributedOptimizer(torch.optim.SGD([p for _, p in params], lr=0.1),
                                   named_parameters=params)
    hvd.broadcast_parameters(dict(params), root_rank=0)
    ref_opt = torch.optim.SGD(list(ref1.parameters()) + list(ref2.parameters()), lr=0.1)
    ok, why = True, []
    for step in range(3):
        g = torch.Generator().manual_seed(100 + step)
        full = torch.randn(4 * size, 16, generator=g)
        mine = full[4 * rank:4 * rank + 4]
        opt.zero_grad()
        out = l2(torch.relu(l1(mine.to(d0))).to(d1))
        out.square().mean().backward()
        opt.step()
        ref_opt.zero_grad()
        ref2(torch.relu(ref1(full))).square().mean().backward()
        ref_opt.step()
    # (the reference runs on the CPU: allow for the different summation order)
    for (n, p), q in zip(params, list(ref1.parameters()) + list(ref2.parameters())):
        if not torch.allclose(p.detach().cpu(), q.detach(), rtol=1e-4, atol=1e-5):
            why.append("param %s differs by %g" % (n, (p.detach().cpu() - q.detach()).abs().max()))
    # plain collectives on both devices, interleaved
    for i, dev in enumerate((d0, d1, d0, d1)):
        x = torch.full((1000,), float(rank + 1), device=dev)
        s = hvd.allreduce(x, op=hvd.Sum, prescale_factor=0.5, name="md.ar.%d" % i)
        if s.device != dev or not torch.allclose(
                s.cpu(), torch.full((1000,), 0.5 * sum(range(1, size + 1)))):
            why.append("allreduce %d on %s: %s %s" % (i, dev, s.device, s[:3].tolist()))
        g = hvd.allgather(torch.full((2,), float(rank), device=dev), name="md.ag.%d" % i)
        if g.cpu().tolist() != [float(r) for r in range(size) for _ in range(2)]:
            why.append("allgather %d on %s: %s" % (i, dev, g.cpu().tolist()))
    torch.cuda.synchronize(d0)
    torch.cuda.synchronize(d1)
    hvd.shutdown()
    return why


def test_two_devices_in_one_rank():
    if _ngpu() < 2:
        pytest.skip("needs 2 GPUs")
    ranks = 2 if _ngpu() >= 4 else 1
    out = run_parallel(_two_devices_per_rank, np=ranks, timeout=300)
    assert all(not why for why in out), out


def _allreduce_pipelined(rank, size, algo):
    """The two-shot / NVLS fused allreduce as a pipeline of many small steps
    (tiny sub-chunks, pipelining from 64 KB on), over fused groups and large
    single tensors, several launches in a row."""
    os.environ["HOROVOD_ALLREDUCE_ALGO"] = algo
    os.environ["HOROVOD_ALLREDUCE_PIPELINE_MIN_BYTES"] = str(64 << 10)
    os.environ["HOROVOD_ALLREDUCE_SUBCHUNK_KB"] = "4"
    os.environ["HOROVOD_SPIN_TIMEOUT_MS"] = "5000"
    import horovod_b200.torch as hvd
    hvd.init()
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    ok = True
    for it in range(3):
        for dtype, n, tol in ((torch.float32, (3 << 20) + 5, 1e-5), (torch.bfloat16, 1 << 20, 4e-2),
                              (torch.float32, 70001, 1e-5), (torch.float16, 300007, 8e-3)):
            x = _inputs(rank + 10 * it, n, dtype).to(dev)
            out = hvd.allreduce(x, op=hvd.Sum, name="pl.%s.%d" % (dtype, n))
            ref = sum(_inputs(r + 10 * it, n, dtype).double() for r in range(size))
            err = (out.double().cpu() - ref).abs().max().item()
            ok = ok and err <= tol * size * max(1.0, ref.abs().max().item())
        shapes = [3, 129, 200001, 77777, 5, 1 << 19]
        xs = [_inputs(rank * 31 + i + it, s, torch.float32).to(dev) for i, s in enumerate(shapes)]
        outs = hvd.grouped_allreduce(xs, op=hvd.Average, name="pl.grp")
        for i, (s, o) in enumerate(zip(shapes, outs)):
            ref = sum(_inputs(r * 31 + i + it, s, torch.float32).double()
                      for r in range(size)) / size
            ok = ok and (o.double().cpu() - ref).abs().max().item() < 1e-5
        # fp32 tensors on a 16-bit wire
        xs = [_inputs(rank * 13 + i + it, s, torch.float32).to(dev) for i, s in enumerate(shapes)]
        hvd.synchronize(hvd.grouped_allreduce_async_(xs, op=hvd.Average,
                                                     wire_dtype=torch.bfloat16, name="pl.wire"))
        for i, (s, o) in enumerate(zip(shapes, xs)):
            ref = sum(_inputs(r * 13 + i + it, s, torch.float32).bfloat16().double()
                      for r in range(size)) / size
            ok = ok and (o.double().cpu() - ref).abs().max().item() < 4e-2 * size
    torch.cuda.synchronize()
    hvd.shutdown()
    return ok


@pytest.mark.parametrize("algo", ["twoshot", "nvls"])
def test_pipelined_fused_allreduce(algo):
    if _ngpu() < 2:
        pytest.skip("needs 2 GPUs")
    assert all(run_parallel(_allreduce_pipelined, np=_world(), args=(algo,), timeout=300))


def _shrink_between_steps(rank, size):
    """Ranks leave between steps: the job shuts down cleanly at a step
    boundary (no kernel or collective in flight), the upper half of the ranks
    exits, and the survivors initialise again with a smaller world. The
    symmetric arena, its peer mappings and flag words are rebuilt for the new
    membership and the kernels must give correct results at both sizes.
    Multicast is off (plain peer loads and stores) so that no departing
    process is bound to a multicast object."""
    os.environ["HOROVOD_SYMM_NVLS"] = "0"
    os.environ["HOROVOD_SPIN_TIMEOUT_MS"] = "5000"
    import horovod_b200.torch as hvd
    from horovod_b200.runner.http.http_server import RendezvousServer
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)

    def work(tag, n_ranks):
        ok = hvd.size() == n_ranks
        for n in (1000, (1 << 20) + 3):
            x = _inputs(rank, n, torch.float32).to(dev)
            out = hvd.allreduce(x, op=hvd.Sum, name="%s.ar.%d" % (tag, n))
            ref = sum(_inputs(r, n, torch.float32).double() for r in range(n_ranks))
            ok = ok and (out.double().cpu() - ref).abs().max().item() < 1e-4
        heap = hvd.symmetric_empty(70000)
        heap.copy_(_inputs(rank + 50, 70000, torch.float32))
        hvd.allreduce_(heap, op=hvd.Average, name="%s.inplace" % tag)
        ref = sum(_inputs(r + 50, 70000, torch.float32).double() for r in range(n_ranks)) / n_ranks
        ok = ok and (heap.double().cpu() - ref).abs().max().item() < 1e-5
        g = hvd.allgather(torch.full((rank + 1, 2), float(rank), device=dev), name="%s.ag" % tag)
        ok = ok and torch.equal(g.cpu(), torch.cat([torch.full((r + 1, 2), float(r))
                                                     for r in range(n_ranks)]))
        rs = hvd.reducescatter(torch.ones(4 * n_ranks, 3, device=dev) * (rank + 1),
                               op=hvd.Sum, name="%s.rs" % tag)
        ok = ok and torch.allclose(rs.cpu(), torch.full((4, 3), float(sum(range(1, n_ranks + 1)))))
        torch.cuda.synchronize()
        # the arena in use was built for exactly this membership
        return ok and hvd.gpu_backend().startswith("symm ranks=%d " % n_ranks)

    hvd.init()
    ok = work("first", size)
    # The survivors meet again through a second rendezvous server that rank 0
    # starts now; its port travels over the first session.
    survivors = max(1, size // 2)
    server = None
    port = 0
    if rank == 0:
        server = RendezvousServer()
        port = server.start()
        server.init([None] * survivors)
    port = hvd.broadcast_object(port, root_rank=0, name="shrink.port")
    hvd.shutdown()  # a step boundary: nothing in flight on any rank
    if rank >= survivors:
        return ok
    os.environ.update({"HOROVOD_SIZE": str(survivors), "HOROVOD_LOCAL_SIZE": str(survivors),
                       "HOROVOD_GLOO_RENDEZVOUS_PORT": str(port)})
    hvd.init()
    ok = ok and work("second", survivors)
    hvd.shutdown()
    if server is not None:
        server.stop()
    return ok


def test_ranks_leave_between_steps_and_the_arena_is_rebuilt():
    if _ngpu() < 2:
        pytest.skip("needs 2 GPUs")
    n = 4 if _ngpu() >= 4 else 2
    assert all(run_parallel(_shrink_between_steps, np=n, timeout=300))


def _two_streams(rank, size, backend):
    """HOROVOD_NUM_NCCL_STREAMS=2: responses alternate between two
    communication streams (each with its own arena, flag words and, on the
    NCCL path, communicator); many collectives in flight at once must still
    give the right answers, and symmetric-heap tensors keep working."""
    os.environ["HOROVOD_NUM_NCCL_STREAMS"] = "2"
    os.environ["HOROVOD_GPU_BACKEND"] = backend
    os.environ["HOROVOD_SPIN_TIMEOUT_MS"] = "5000"
    os.environ["HOROVOD_FUSION_THRESHOLD"] = str(1 << 20)  # many separate responses
    import horovod_b200.torch as hvd
    hvd.init()
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    ok = True
    for it in range(3):
        sizes = [1000, (1 << 20) + 3, 50000, 3 << 20, 17, 700001]
        xs = [_inputs(rank + i + 10 * it, n, torch.float32).to(dev) for i, n in enumerate(sizes)]
        hs = [hvd.allreduce_async(x, op=hvd.Sum, name="ts.ar.%d" % i) for i, x in enumerate(xs)]
        g = hvd.allgather_async(torch.full((rank + 1, 3), float(rank), device=dev), name="ts.ag")
        b = torch.arange(5000, device=dev, dtype=torch.float32) * (rank + 1)
        bh = hvd.broadcast_async_(b, root_rank=size - 1, name="ts.bc")
        for i, (h, n) in enumerate(zip(hs, sizes)):
            out = hvd.synchronize(h)
            ref = sum(_inputs(r + i + 10 * it, n, torch.float32).double() for r in range(size))
            ok = ok and (out.double().cpu() - ref).abs().max().item() < 1e-4
        got = hvd.synchronize(g)
        ok = ok and torch.equal(got.cpu(), torch.cat([torch.full((r + 1, 3), float(r))
                                                       for r in range(size)]))
        hvd.synchronize(bh)
        ok = ok and torch.equal(b.cpu(), torch.arange(5000, dtype=torch.float32) * size)
    if backend == "symm":
        heap = hvd.symmetric_empty(100000)
        for it in range(4):  # whichever lane is next, heap tensors go to the first
            heap.copy_(_inputs(rank + it, 100000, torch.float32))
            hvd.allreduce_(heap, op=hvd.Average, name="ts.heap")
            ref = sum(_inputs(r + it, 100000, torch.float32).double() for r in range(size)) / size
            ok = ok and (heap.double().cpu() - ref).abs().max().item() < 1e-5
    torch.cuda.synchronize()
    hvd.shutdown()
    return ok


@pytest.mark.parametrize("backend", ["symm", "nccl"])
def test_two_communication_streams(backend):
    if _ngpu() < 2:
        pytest.skip("needs 2 GPUs")
    assert all(run_parallel(_two_streams, np=_world(), args=(backend,), timeout=300))
