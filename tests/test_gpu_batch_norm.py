"""Fused batch norm (+ residual + ReLU) kernels against a plain PyTorch fp32
reference of the same op, forward and backward, and the ResNet blocks built
on them against the unfused PyTorch composition."""
import os

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu

SHAPES = [(8, 64, 14, 14), (4, 256, 7, 7), (2, 8, 9, 9), (3, 2048, 4, 4), (16, 128, 28, 28),
          (5, 16, 3, 3), (2, 512, 1, 1)]


def _reference(x, res, weight, bias, relu, eps):
    xf = x.float().detach().requires_grad_(True)
    rf = res.float().detach().requires_grad_(True) if res is not None else None
    w = weight.detach().clone().requires_grad_(True)
    b = bias.detach().clone().requires_grad_(True)
    rm, rv = torch.zeros_like(w), torch.ones_like(w)
    out = F.batch_norm(xf, rm, rv, w, b, True, 0.1, eps)
    if rf is not None:
        out = out + rf
    if relu:
        out = F.relu(out)
    return xf, rf, w, b, rm, rv, out


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("relu,with_res", [(True, False), (True, True), (False, False),
                                           (False, True)])
@pytest.mark.parametrize("shape", SHAPES)
def test_fused_batch_norm_matches_fp32_reference(shape, relu, with_res, dtype):
    from horovod_b200 import _C
    from horovod_b200.ops.batch_norm import batch_norm_act, fused_batch_norm_available
    dev = torch.device("cuda", 0)
    g = torch.Generator(device="cpu").manual_seed(hash((shape, relu, with_res)) % 1000)
    n, c, h, w_ = shape
    x = (torch.randn(shape, generator=g) * 1.5 + 0.3).to(dev, dtype) \
        .contiguous(memory_format=torch.channels_last).requires_grad_(True)
    res = torch.randn(shape, generator=g).to(dev, dtype) \
        .contiguous(memory_format=torch.channels_last).requires_grad_(True) if with_res else None
    weight = (torch.rand(c, generator=g) + 0.5).to(dev).requires_grad_(True)
    bias = (torch.randn(c, generator=g) * 0.2).to(dev).requires_grad_(True)
    rm, rv = torch.zeros(c, device=dev), torch.ones(c, device=dev)
    assert fused_batch_norm_available(x, 0.1), "fused path not taken"
    before = _C.kernel_launch_count()
    y = batch_norm_act(x, weight, bias, rm, rv, residual=res, training=True, momentum=0.1,
                       eps=1e-5, relu=relu)
    assert _C.kernel_launch_count() == before + 2, "native kernels did not run"
    go = torch.randn(shape, generator=g).to(dev, dtype).contiguous(memory_format=torch.channels_last)
    y.backward(go)
    assert _C.kernel_launch_count() == before + 4

    xf, rf, wr, br, rmr, rvr, out = _reference(x, res, weight, bias, relu, 1e-5)
    out.backward(go.float())
    tol = dict(rtol=2e-2, atol=3e-2) if dtype == torch.bfloat16 else dict(rtol=4e-3, atol=6e-3)
    torch.testing.assert_close(y.float(), out, **tol)
    torch.testing.assert_close(rm, rmr, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(rv, rvr, rtol=1e-4, atol=1e-5)
    m = n * h * w_
    # The ReLU mask is taken from the rounded output, the reference's from the
    # unrounded one: identical except where the pre-activation is within
    # rounding of zero, so gradients are compared with a small outlier budget.
    def close(a, b, what, rel):
        err = (a.float() - b).abs()
        lim = rel * (b.abs() + b.abs().mean() + 1e-3)
        bad = (err > lim).float().mean().item()
        assert bad <= 2e-3, (what, bad, err.max().item())
    close(x.grad, xf.grad, "dx", 4e-2 if dtype == torch.bfloat16 else 1e-2)
    if with_res:
        close(res.grad, rf.grad, "dres", 2e-2)
    scale = max(1.0, m ** 0.5)
    assert (weight.grad - wr.grad).abs().max().item() <= 2e-2 * scale * 0.1 + 2e-2 * wr.grad.abs().max().item()
    assert (bias.grad - br.grad).abs().max().item() <= 2e-2 * scale * 0.1 + 2e-2 * br.grad.abs().max().item()


def test_resnet_blocks_match_unfused_composition(monkeypatch):
    """The network built on the fused op is as close to an fp32 run of the
    plain PyTorch composition as the bf16 run of that composition is."""
    from horovod_b200.models.resnet import resnet_tiny
    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    x = torch.randn(32, 3, 64, 64, device=dev).contiguous(memory_format=torch.channels_last)
    y = torch.randint(0, 10, (32,), device=dev)

    def run(fused, autocast):
        monkeypatch.setenv("HOROVOD_B200_FUSED_BN", "1" if fused else "0")
        torch.manual_seed(1)
        model = resnet_tiny().to(dev).to(memory_format=torch.channels_last)
        # bn3 weights start at zero (identity blocks): give them a value so the
        # fused residual path carries signal
        with torch.no_grad():
            for name, p in model.named_parameters():
                if name.endswith("bn3.weight"):
                    p.fill_(0.5)
        with torch.autocast("cuda", dtype=torch.bfloat16, enabled=autocast):
            loss = F.cross_entropy(model(x), y)
        loss.backward()
        return (loss.item(), {n: p.grad.float().clone() for n, p in model.named_parameters()},
                {n: b.clone() for n, b in model.named_buffers()})

    l_ref, g_ref, b_ref = run(fused=False, autocast=False)
    l_plain, g_plain, _ = run(fused=False, autocast=True)
    l_fused, g_fused, b_fused = run(fused=True, autocast=True)
    assert abs(l_fused - l_ref) <= 2 * abs(l_plain - l_ref) + 2e-2, (l_fused, l_plain, l_ref)

    def rel(a, b):
        return (a - b).norm().item() / (b.norm().item() + 1e-6)

    e_plain = {n: rel(g_plain[n], g_ref[n]) for n in g_ref}
    e_fused = {n: rel(g_fused[n], g_ref[n]) for n in g_ref}
    worse = {n: (e_fused[n], e_plain[n]) for n in g_ref
             if e_fused[n] > 2.0 * e_plain[n] + 0.05}
    assert not worse, worse
    for n in b_ref:
        if b_ref[n].dtype.is_floating_point:
            torch.testing.assert_close(b_fused[n], b_ref[n], rtol=5e-2, atol=5e-2)
        else:
            assert torch.equal(b_fused[n], b_ref[n]), n
