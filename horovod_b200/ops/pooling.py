"""Max pooling 3x3 / stride 2 / padding 1 for channels-last bf16/fp16
activations on this library's CUDA kernels (csrc/kernels/pooling.cu), with
PyTorch's ``F.max_pool2d`` everywhere else.

PyTorch's channels-last max pooling stores an int64 index per output element
and scatters the gradient with atomics; on the ResNet-50 stem (256 x 64 x 112
x 112 in bf16) forward plus backward take 2.5 ms per step on a B200. The
kernels here keep one byte per output element and gather in backward, which
moves a third of the bytes and needs no atomics. Ties and NaN follow PyTorch's
rule, so outputs and gradients are identical. The reference has no
counterpart (it takes pooling from the framework).
"""
import os

import torch
import torch.nn as nn
import torch.nn.functional as F


def _extension():
    from horovod_b200 import _C
    return _C


def fused_max_pool_available(x):
    if os.environ.get("HOROVOD_B200_FUSED_POOL", "1") != "1":
        return False
    if not (x.is_cuda and x.dim() == 4 and x.dtype in (torch.bfloat16, torch.float16)):
        return False
    if not x.is_contiguous(memory_format=torch.channels_last):
        return False
    return x.size(2) >= 2 and x.size(3) >= 2 and _extension().maxpool3s2_supported(x.size(1))


class _MaxPool3s2(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        y, idx = _extension().maxpool3s2_forward(x)
        ctx.save_for_backward(idx)
        ctx.hw = (x.size(2), x.size(3))
        return y

    @staticmethod
    def backward(ctx, dy):
        (idx,) = ctx.saved_tensors
        dy = dy.contiguous(memory_format=torch.channels_last)
        return _extension().maxpool3s2_backward(dy, idx, ctx.hw[0], ctx.hw[1])


def max_pool_3x3_s2(x):
    """``F.max_pool2d(x, 3, stride=2, padding=1)``, fused on the GPU when possible."""
    if fused_max_pool_available(x):
        return _MaxPool3s2.apply(x)
    return F.max_pool2d(x, 3, stride=2, padding=1)


class MaxPool3x3s2(nn.Module):
    """Drop-in for ``nn.MaxPool2d(3, stride=2, padding=1)``."""

    def forward(self, x):
        return max_pool_3x3_s2(x)
