"""Single-GPU checks of the device path through the public API: with one
rank every collective still runs the library's own kernels (the LOCAL
variants), so packing, scaling, casting and scattering are exercised."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def hvd():
    import horovod_b200.torch as hvd
    hvd.init()
    torch.cuda.set_device(0)
    yield hvd
    hvd.shutdown()


def _dev():
    return torch.device("cuda", 0)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16,
                                   torch.float64, torch.int32, torch.int64])
@pytest.mark.parametrize("n", [1, 15, 16, 17, 1000, 1 << 20])
def test_allreduce_identity_and_scale(hvd, dtype, n):
    from horovod_b200 import _C
    x = (torch.arange(n, device=_dev()) % 97).to(dtype)
    before = _C.kernel_launch_count()
    y = hvd.allreduce(x, op=hvd.Sum, name="s.%s.%d" % (dtype, n))
    assert _C.kernel_launch_count() > before, "native kernel did not run"
    assert torch.equal(y, x)
    if dtype.is_floating_point:
        z = hvd.allreduce(x, op=hvd.Sum, prescale_factor=0.5, postscale_factor=4.0,
                          name="p.%s.%d" % (dtype, n))
        ref = (x.float() * 0.5).to(dtype).float() * 4.0 if dtype != torch.float64 else x * 2.0
        torch.testing.assert_close(z.float(), ref.float().to(z.device), rtol=1e-2, atol=1e-2)


def test_grouped_allreduce_many_odd_tensors(hvd):
    torch.manual_seed(0)
    sizes = [1, 3, 17, 255, 256, 257, 4099, 65537] * 20 + [1 << 20]
    xs = [torch.randn(s, device=_dev()) for s in sizes]
    # odd alignments: views that start 4 bytes into an allocation
    xs += [torch.randn(1001, device=_dev())[1:] for _ in range(5)]
    ys = hvd.grouped_allreduce([x.contiguous() for x in xs], op=hvd.Average, name="grp")
    for x, y in zip(xs, ys):
        torch.testing.assert_close(y, x, rtol=0, atol=0)


def test_inplace_and_async(hvd):
    x = torch.randn(12345, device=_dev())
    ref = x.clone()
    h = hvd.allreduce_async_(x, op=hvd.Sum, postscale_factor=3.0, name="inplace")
    out = hvd.synchronize(h)
    assert out.data_ptr() == x.data_ptr()
    torch.testing.assert_close(x, ref * 3.0)


def test_wire_cast_happens_inside_the_kernel(hvd):
    x = torch.randn(100003, device=_dev())
    for wire in (torch.bfloat16, torch.float16):
        y = x.clone()
        hvd.synchronize(hvd.allreduce_async_(y, op=hvd.Sum, postscale_factor=2.0,
                                             wire_dtype=wire, name="wire.%s" % wire))
        assert y.dtype == torch.float32
        torch.testing.assert_close(y, x.to(wire).float() * 2.0, rtol=0, atol=0)


def test_other_collectives_single_rank(hvd):
    x = torch.randn(7, 5, device=_dev())
    torch.testing.assert_close(hvd.allgather(x, name="ag"), x)
    torch.testing.assert_close(hvd.broadcast(x, 0, name="bc"), x)
    torch.testing.assert_close(hvd.alltoall(x, name="a2a"), x)
    out, splits = hvd.alltoall(x, splits=[7], name="a2a.s")
    torch.testing.assert_close(out, x)
    assert splits.tolist() == [7]
    torch.testing.assert_close(hvd.reducescatter(x, op=hvd.Sum, name="rs"), x)


def test_compression_and_optimizer_step(hvd, monkeypatch):
    monkeypatch.setenv("HOROVOD_FORCE_HOOKS", "1")
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(64, 32), torch.nn.ReLU(),
                                torch.nn.Linear(32, 4)).to(_dev())
    ref = torch.nn.Sequential(torch.nn.Linear(64, 32), torch.nn.ReLU(),
                              torch.nn.Linear(32, 4)).to(_dev())
    ref.load_state_dict(model.state_dict())
    opt = hvd.DistributedOptimizer(torch.optim.SGD(model.parameters(), lr=0.1),
                                   named_parameters=model.named_parameters())
    ropt = torch.optim.SGD(ref.parameters(), lr=0.1)
    x = torch.randn(16, 64, device=_dev())
    y = torch.randint(0, 4, (16,), device=_dev())
    for _ in range(3):
        for m, o in ((model, opt), (ref, ropt)):
            o.zero_grad()
            torch.nn.functional.cross_entropy(m(x), y).backward()
            o.step()
    for a, b in zip(model.parameters(), ref.parameters()):
        torch.testing.assert_close(a, b, rtol=1e-6, atol=1e-6)




def test_wait_for_a_peer_that_never_arrives_is_bounded():
    """A barrier whose second member never signals gives up after its time
    limit, reports whom it waited for, and leaves the GPU usable (this is what
    a dead peer looks like to a kernel; the failure is made on the host: the
    peer simply does not exist)."""
    from horovod_b200 import _C
    torch.cuda.set_device(0)
    code, peer, phase, block, ms, launch_err, sync_err = _C.bounded_wait_probe(0, 200)
    assert launch_err == 0 and sync_err == 0
    assert (code, peer, block) == (1, 1, 0), (code, peer, phase, block)
    assert 150.0 <= ms < 2000.0, ms
    # the context is intact
    x = torch.arange(1000, device="cuda:0", dtype=torch.float32)
    assert float(x.sum()) == 499500.0


def test_timeline_shows_device_times_of_the_kernel(hvd, tmp_path):
    """With the timeline on, the FUSED_NVLINK_KERNEL activity of an op is
    replayed from CUDA events: its length is the time the GPU spent in the
    kernel (large for 512 MB, tiny for 4 KB), not the time the host took to
    queue it, and it lies inside the op's span."""
    import json
    import time
    path = str(tmp_path / "timeline.json")
    big = torch.randn(128 << 20, device=_dev())    # 512 MB: hundreds of microseconds
    small = torch.randn(1024, device=_dev())
    torch.cuda.synchronize()
    hvd.start_timeline(path, mark_cycles=False)
    time.sleep(0.05)
    for i in range(3):
        hvd.allreduce(big, op=hvd.Sum, postscale_factor=0.5, name="tl.big")
        hvd.allreduce(small, op=hvd.Sum, postscale_factor=0.5, name="tl.small")
    torch.cuda.synchronize()
    hvd.stop_timeline()
    time.sleep(0.2)
    events = json.load(open(path))
    pids = {e["args"]["name"]: e["pid"] for e in events
            if e.get("name") == "process_name"}
    spans = {}
    for name in ("tl.big", "tl.small"):
        stack, found = [], []
        for e in (e for e in events if e.get("pid") == pids[name] and e["ph"] in "BE"):
            if e["ph"] == "B":
                stack.append(e)
            else:
                b = stack.pop()
                found.append((b["name"], b["ts"], e["ts"], len(stack)))
        assert not stack
        spans[name] = found
    for name in ("tl.big", "tl.small"):
        kernels = [(t0, t1) for n, t0, t1, depth in spans[name]
                   if n == "FUSED_NVLINK_KERNEL" and depth == 1]
        ops = [(t0, t1) for n, t0, t1, depth in spans[name] if n == "ALLREDUCE"]
        assert len(kernels) == 3 and len(ops) == 3, spans[name]
        for (k0, k1), (o0, o1) in zip(sorted(kernels), sorted(ops)):
            assert k0 <= k1 and o0 <= k0 + 50 and k1 <= o1 + 50, (name, kernels, ops)
    big_us = sorted(t1 - t0 for t0, t1 in
                    [(a, b) for n, a, b, d in spans["tl.big"] if n == "FUSED_NVLINK_KERNEL"])
    small_us = sorted(t1 - t0 for t0, t1 in
                      [(a, b) for n, a, b, d in spans["tl.small"] if n == "FUSED_NVLINK_KERNEL"])
    # 1 GB of traffic cannot take less than 100 us on any GPU; 4 KB is over
    # in a few microseconds however long the host needed to launch it.
    assert big_us[1] > 100, big_us
    assert small_us[1] < 60, small_us
