"""Model-side kernels against plain PyTorch: the fused 3x3/stride-2 max pooling
(outputs and gradients must equal F.max_pool2d exactly, ties and NaN
included) and the multi-tensor SGD kernel (against torch.optim.SGD in fp32)."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def _dev():
    return torch.device("cuda", 0)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(2, 8, 2, 2), (3, 16, 7, 9), (2, 64, 112, 112), (1, 24, 5, 4),
                                   (4, 8, 33, 17)])
def test_max_pool_matches_pytorch(dtype, shape):
    from horovod_b200 import _C
    from horovod_b200.ops.pooling import fused_max_pool_available, max_pool_3x3_s2
    torch.manual_seed(0)
    # relu makes ties (runs of zeros) frequent, as in the ResNet stem
    base = torch.relu(torch.randn(shape, device=_dev())).to(dtype)
    base = base.contiguous(memory_format=torch.channels_last)
    x = base.clone().requires_grad_(True)
    ref_x = base.float().clone().requires_grad_(True)  # plain PyTorch fp32 reference
    assert fused_max_pool_available(x)
    before = _C.kernel_launch_count()
    y = max_pool_3x3_s2(x)
    assert _C.kernel_launch_count() > before, "native kernel did not run"
    ref = F.max_pool2d(ref_x, 3, stride=2, padding=1)
    assert y.shape == ref.shape
    assert torch.equal(y.float(), ref)
    go = torch.randn_like(ref).to(dtype)
    y.backward(go)
    ref.backward(go.float())
    # a position can collect up to four gradients: compare in the 16-bit type
    torch.testing.assert_close(x.grad.float(), ref_x.grad.to(dtype).float(), rtol=1e-2, atol=1e-2)
    # and the set of positions that received gradient must be the same
    assert torch.equal(x.grad != 0, ref_x.grad.to(dtype) != 0)


def test_max_pool_nan_and_fallback():
    from horovod_b200.ops.pooling import fused_max_pool_available, max_pool_3x3_s2
    x = torch.zeros(1, 8, 6, 6, device=_dev(), dtype=torch.bfloat16)
    x[0, 0, 2, 2] = float("nan")
    x[0, 1, 0, 0] = float("-inf")
    x = x.contiguous(memory_format=torch.channels_last)
    y = max_pool_3x3_s2(x)
    ref = F.max_pool2d(x.float(), 3, stride=2, padding=1)
    assert torch.equal(torch.isnan(y), torch.isnan(ref))
    assert torch.equal(torch.nan_to_num(y.float(), nan=7.0), torch.nan_to_num(ref, nan=7.0))
    # NCHW or fp32 inputs take PyTorch's own kernel
    z = torch.randn(2, 8, 9, 9, device=_dev())
    assert not fused_max_pool_available(z)
    assert torch.equal(max_pool_3x3_s2(z), F.max_pool2d(z, 3, stride=2, padding=1))


def _small_net():
    torch.manual_seed(3)
    net = torch.nn.Sequential(
        torch.nn.Conv2d(3, 16, 3, padding=1), torch.nn.ReLU(),
        torch.nn.Conv2d(16, 8, 3, padding=1, bias=False), torch.nn.Flatten(),
        torch.nn.Linear(8 * 8 * 8, 10))
    return net.to(_dev()).to(memory_format=torch.channels_last)


@pytest.mark.parametrize("kwargs", [
    dict(lr=0.1),
    dict(lr=0.05, momentum=0.9),
    dict(lr=0.05, momentum=0.9, weight_decay=1e-2),
    dict(lr=0.05, momentum=0.9, weight_decay=1e-2, nesterov=True),
    dict(lr=0.05, momentum=0.8, dampening=0.3),
    dict(lr=0.05, momentum=0.9, maximize=True),
])
def test_fused_sgd_matches_torch_sgd(kwargs):
    from horovod_b200 import _C
    from horovod_b200.torch.fused_sgd import FusedSGD
    a, b = _small_net(), _small_net()
    b.load_state_dict(a.state_dict())
    ref = torch.optim.SGD(a.parameters(), **kwargs)
    opt = FusedSGD(b.parameters(), **kwargs)
    torch.manual_seed(11)
    before = _C.kernel_launch_count()
    for step in range(5):
        x = torch.randn(4, 3, 8, 8, device=_dev()).contiguous(memory_format=torch.channels_last)
        for net, o in ((a, ref), (b, opt)):
            o.zero_grad()
            net(x).square().mean().backward()
            o.step()
    assert _C.kernel_launch_count() - before >= 5, "the fused kernel did not run"
    for pa, pb in zip(a.parameters(), b.parameters()):
        torch.testing.assert_close(pb, pa, rtol=1e-5, atol=1e-6)
    if kwargs.get("momentum"):
        for pa, pb in zip(a.parameters(), b.parameters()):
            torch.testing.assert_close(opt.state[pb]["momentum_buffer"],
                                       ref.state[pa]["momentum_buffer"], rtol=1e-5, atol=1e-6)


def test_fused_sgd_state_dict_round_trip_and_odd_sizes():
    from horovod_b200.torch.fused_sgd import FusedSGD
    torch.manual_seed(5)
    sizes = [1, 3, 4, 5, 1023, 65536, 65537, 200003]
    ps = [torch.randn(s, device=_dev(), requires_grad=True) for s in sizes]
    # a view that is only 4-byte aligned
    holder = torch.randn(1001, device=_dev())
    odd = holder[1:].detach().requires_grad_(True)
    ps.append(odd)
    qs = [p.detach().clone().requires_grad_(True) for p in ps]
    ref = torch.optim.SGD(qs, lr=0.1, momentum=0.9, weight_decay=1e-3)
    opt = FusedSGD(ps, lr=0.1, momentum=0.9, weight_decay=1e-3)
    for step in range(3):
        for p, q in zip(ps, qs):
            g = torch.randn_like(p)
            p.grad, q.grad = g.clone(), g.clone()
        opt.step()
        ref.step()
        if step == 1:  # reload in the middle: torch.optim.SGD's format
            opt.load_state_dict(opt.state_dict())
    for p, q in zip(ps, qs):
        torch.testing.assert_close(p, q, rtol=1e-5, atol=1e-6)
