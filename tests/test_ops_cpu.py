"""CPU-side checks of the model ops and the data-parallel helpers: the
batch-norm module's fallback path equals the PyTorch composition it replaces,
the benchmark model has the reference's size, and data_parallel_setup trains
like a single process on the concatenated batch."""
import torch
import torch.nn as nn
import torch.nn.functional as F

from parallel_utils import run_parallel


def test_batch_norm_act_fallback_equals_pytorch_composition():
    from horovod_b200.ops import BatchNormAct2d
    torch.manual_seed(0)
    for relu in (True, False):
        for with_res in (True, False):
            a, b = BatchNormAct2d(6, relu=relu), nn.BatchNorm2d(6)
            with torch.no_grad():
                a.weight.uniform_(0.5, 1.5)
                a.bias.normal_()
            b.load_state_dict(a.state_dict())  # same keys, same shapes
            x1 = torch.randn(4, 6, 5, 5, requires_grad=True)
            x2 = x1.detach().clone().requires_grad_(True)
            r1 = torch.randn(4, 6, 5, 5, requires_grad=True) if with_res else None
            r2 = r1.detach().clone().requires_grad_(True) if with_res else None
            y1 = a(x1, residual=r1)
            y2 = b(x2)
            if with_res:
                y2 = y2 + r2
            if relu:
                y2 = F.relu(y2)
            torch.testing.assert_close(y1, y2)
            go = torch.randn_like(y1)
            y1.backward(go)
            y2.backward(go)
            torch.testing.assert_close(x1.grad, x2.grad)
            torch.testing.assert_close(a.weight.grad, b.weight.grad)
            torch.testing.assert_close(a.bias.grad, b.bias.grad)
            if with_res:
                torch.testing.assert_close(r1.grad, r2.grad)
            torch.testing.assert_close(a.running_mean, b.running_mean)
            torch.testing.assert_close(a.running_var, b.running_var)
            assert int(a.num_batches_tracked) == int(b.num_batches_tracked) == 1
            a.eval(), b.eval()
            torch.testing.assert_close(a(x1.detach()),
                                       F.relu(b(x2.detach())) if relu else b(x2.detach()))


def test_resnet50_has_the_reference_models_size():
    from horovod_b200.models.resnet import resnet50
    model = resnet50()
    params = list(model.parameters())
    assert len(params) == 161
    assert sum(p.numel() for p in params) == 25557032  # torchvision resnet50
    keys = model.state_dict().keys()
    assert "layer1.0.bn3.running_var" in keys and "layer1.0.downsample.1.weight" in keys


def _data_parallel(rank, size):
    import horovod_b200.torch as hvd
    from horovod_b200.parallel import data_parallel_setup
    hvd.init()
    torch.manual_seed(rank)  # ranks start from different weights
    model = nn.Sequential(nn.Linear(6, 12), nn.Tanh(), nn.Linear(12, 3))
    opt = torch.optim.SGD(model.parameters(), lr=0.05, momentum=0.9)
    model, opt = data_parallel_setup(model, opt)
    g = torch.Generator().manual_seed(100)
    xs, ys = torch.randn(size * 4, 6, generator=g), torch.randint(0, 3, (size * 4,), generator=g)
    x, y = xs[rank * 4:(rank + 1) * 4], ys[rank * 4:(rank + 1) * 4]
    for _ in range(5):
        opt.zero_grad()
        F.cross_entropy(model(x), y).backward()
        opt.step()
    # single-process run on the whole batch from rank 0's initial weights
    torch.manual_seed(0)
    ref = nn.Sequential(nn.Linear(6, 12), nn.Tanh(), nn.Linear(12, 3))
    ropt = torch.optim.SGD(ref.parameters(), lr=0.05, momentum=0.9)
    for _ in range(5):
        ropt.zero_grad()
        F.cross_entropy(ref(xs), ys).backward()
        ropt.step()
    ok = all(torch.allclose(a, b, atol=1e-5) for a, b in zip(model.parameters(), ref.parameters()))
    hvd.shutdown()
    return ok


def test_data_parallel_setup_matches_single_process():
    assert all(run_parallel(_data_parallel, np=2))


def test_utils_namespace_without_gpu():
    import horovod_b200.utils as u
    assert isinstance(u.kernel_launch_count(), int)
    assert isinstance(u.gpu_backend(), str)
    topo = u.gpu_topology()
    assert "device_count" in topo
