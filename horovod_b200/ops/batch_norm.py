"""Fused training-mode batch normalisation (+ residual add + ReLU) for
channels-last bf16/fp16 activations, backed by this library's CUDA kernels
(csrc/kernels/batch_norm.cu), with a plain PyTorch fallback everywhere else
(CPU, fp32, NCHW, eval mode, channel counts the kernels do not tile).

``BatchNormAct2d`` is a drop-in ``nn.BatchNorm2d`` (same parameters, buffers
and state_dict keys) whose forward takes an optional residual:

    y = relu(batch_norm(x) + residual)

The eager PyTorch sequence batch_norm -> add -> relu makes eight passes over
the activation in forward and nine in backward; the fused kernels make three
and seven. The reference has no counterpart (it takes batch normalisation
from the framework; horovod/torch/sync_batch_norm.py:98-199 composes
torch.batch_norm_stats / batch_norm_elemt / batch_norm_backward_reduce).
"""
import os

import torch
import torch.nn as nn
import torch.nn.functional as F


def _extension():
    from horovod_b200 import _C
    return _C


def fused_batch_norm_available(x, momentum):
    """True when the CUDA kernels can take this input."""
    if os.environ.get("HOROVOD_B200_FUSED_BN", "1") != "1":
        return False
    if not (x.is_cuda and x.dim() == 4 and x.dtype in (torch.bfloat16, torch.float16)):
        return False
    if momentum is None or not x.is_contiguous(memory_format=torch.channels_last):
        return False
    channels = x.size(1)
    return _extension().bn_supported(x.numel() // channels, channels)


class _FusedBatchNormAct(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, residual, weight, bias, running_mean, running_var, momentum, eps, relu):
        y, mean, invstd = _extension().bn_forward(x, residual, weight, bias, running_mean,
                                                  running_var, momentum, eps, relu)
        ctx.save_for_backward(x, y if relu else None, weight, mean, invstd)
        ctx.relu = relu
        ctx.has_residual = residual is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        x, y, weight, mean, invstd = ctx.saved_tensors
        if dy.dtype != x.dtype:
            dy = dy.to(x.dtype)
        dy = dy.contiguous(memory_format=torch.channels_last)
        want_dres = ctx.has_residual and ctx.needs_input_grad[1]
        dx, dres, dweight, dbias = _extension().bn_backward(
            dy, y if ctx.relu else dy, x, weight, mean, invstd, ctx.relu, want_dres)
        if weight is None:
            dweight = None
        return dx, dres, dweight, dbias if ctx.needs_input_grad[3] else None, None, None, None, \
            None, None


def batch_norm_act(x, weight, bias, running_mean, running_var, residual=None, training=True,
                   momentum=0.1, eps=1e-5, relu=True):
    """relu(batch_norm(x) + residual), fused on the GPU when possible."""
    if training and fused_batch_norm_available(x, momentum) and \
            (residual is None or (residual.shape == x.shape and residual.dtype == x.dtype)):
        if residual is not None:
            residual = residual.contiguous(memory_format=torch.channels_last)
        return _FusedBatchNormAct.apply(x, residual, weight, bias, running_mean, running_var,
                                        float(momentum), float(eps), bool(relu))
    out = F.batch_norm(x, running_mean, running_var, weight, bias, training,
                       0.0 if momentum is None else momentum, eps)
    if residual is not None:
        out = out + residual
    return F.relu(out) if relu else out


class BatchNormAct2d(nn.BatchNorm2d):
    """``nn.BatchNorm2d`` followed by an optional residual add and ReLU."""

    def __init__(self, num_features, relu=True, **kwargs):
        super().__init__(num_features, **kwargs)
        self.relu = relu

    def forward(self, x, residual=None):
        self._check_input_dim(x)
        if self.training and self.track_running_stats and self.num_batches_tracked is not None:
            self.num_batches_tracked.add_(1)
        training = self.training or (self.running_mean is None and self.running_var is None)
        momentum = self.momentum
        if momentum is None and self.training and self.track_running_stats:
            momentum = 1.0 / float(self.num_batches_tracked)
        return batch_norm_act(
            x, self.weight, self.bias,
            self.running_mean if not self.training or self.track_running_stats else None,
            self.running_var if not self.training or self.track_running_stats else None,
            residual=residual, training=training, momentum=momentum, eps=self.eps,
            relu=self.relu)
