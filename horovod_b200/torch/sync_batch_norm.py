"""Batch normalisation whose statistics are computed over the whole global
batch instead of each rank's slice.

Forward gathers per-rank (count, mean, inverse std) and merges them;
backward sums the two reductions the input gradient needs across ranks.

Parity: horovod/torch/sync_batch_norm.py:99-218.
"""
import torch
from torch.autograd.function import Function
import torch.nn.functional as F
from torch.nn.modules.batchnorm import _BatchNorm

from horovod_b200.torch.mpi_ops import Sum, allgather_async, allreduce_async, size, synchronize


class SyncBatchNorm(_BatchNorm):
    """Drop-in replacement for ``torch.nn.BatchNorm{1,2,3}d`` in data-parallel
    training. Falls back to local statistics in eval mode or when the job has
    one rank."""

    def __init__(self, num_features, eps=1e-5, momentum=0.1, affine=True,
                 track_running_stats=True):
        super().__init__(num_features, eps, momentum, affine, track_running_stats)

    def _check_input_dim(self, input):
        if input.dim() < 2:
            raise ValueError("expected at least 2D input (got %dD input)" % input.dim())

    def _run_bn(self, input):
        return F.batch_norm(input, self.running_mean, self.running_var, self.weight,
                            self.bias, self.training or not self.track_running_stats,
                            self.momentum, self.eps)

    @torch.jit.unused
    def _maybe_run_sync_bn(self, input):
        if size() == 1:
            return self._run_bn(input)
        return _SyncBatchNorm.apply(input, self.weight, self.bias, self.running_mean,
                                    self.running_var, self.eps, self.momentum)

    def forward(self, input):
        self._check_input_dim(input)
        if self.training and self.track_running_stats and self.num_batches_tracked is not None:
            self.num_batches_tracked = self.num_batches_tracked + 1
        if not self.training and self.track_running_stats:
            return self._run_bn(input)
        return self._maybe_run_sync_bn(input)


def _reduce_dims(x):
    return [0] + list(range(2, x.dim()))


def _bshape(x):
    return [1, -1] + [1] * (x.dim() - 2)


class _SyncBatchNorm(Function):
    @staticmethod
    def forward(ctx, input, weight, bias, running_mean, running_var, eps, momentum):
        x = input.float().contiguous()
        dims = _reduce_dims(x)
        count = x.numel() // x.size(1)
        mean = x.mean(dims)
        var = x.var(dims, unbiased=False)
        invstd = torch.rsqrt(var + eps)

        count_t = torch.full((1,), float(count), dtype=mean.dtype, device=mean.device)
        h_count = allgather_async(count_t.unsqueeze(0), name="sync_batch_norm.count")
        h_mean = allgather_async(mean.unsqueeze(0), name="sync_batch_norm.mean")
        h_invstd = allgather_async(invstd.unsqueeze(0), name="sync_batch_norm.invstd")
        counts = synchronize(h_count).view(-1)
        means = synchronize(h_mean)
        invstds = synchronize(h_invstd)

        # Merge per-rank moments: E[x] and E[x^2] weighted by sample count.
        total = counts.sum()
        w = (counts / total).unsqueeze(1)
        g_mean = (means * w).sum(0)
        vars_ = 1.0 / (invstds * invstds) - eps
        g_var = ((vars_ + means * means) * w).sum(0) - g_mean * g_mean
        g_invstd = torch.rsqrt(g_var + eps)

        if running_mean is not None and running_var is not None:
            unbiased = g_var * (total / (total - 1).clamp(min=1))
            running_mean.mul_(1 - momentum).add_(g_mean.to(running_mean.dtype), alpha=momentum)
            running_var.mul_(1 - momentum).add_(unbiased.to(running_var.dtype), alpha=momentum)

        ctx.save_for_backward(x, weight, g_mean, g_invstd, total)
        ctx.in_dtype = input.dtype
        shape = _bshape(x)
        out = (x - g_mean.view(shape)) * g_invstd.view(shape)
        if weight is not None:
            out = out * weight.float().view(shape)
        if bias is not None:
            out = out + bias.float().view(shape)
        return out.to(input.dtype)

    @staticmethod
    def backward(ctx, grad_output):
        x, weight, mean, invstd, total = ctx.saved_tensors
        dy = grad_output.float().contiguous()
        dims = _reduce_dims(x)
        shape = _bshape(x)
        xmu = x - mean.view(shape)
        sum_dy = dy.sum(dims)
        sum_dy_xmu = (dy * xmu).sum(dims)

        grad_weight = grad_bias = None
        if weight is not None and ctx.needs_input_grad[1]:
            grad_weight = (sum_dy_xmu * invstd).to(weight.dtype)
        if ctx.needs_input_grad[2]:
            grad_bias = sum_dy.clone()

        grad_input = None
        if ctx.needs_input_grad[0]:
            h1 = allreduce_async(sum_dy, op=Sum, name="sync_batch_norm.sum_dy")
            h2 = allreduce_async(sum_dy_xmu, op=Sum, name="sync_batch_norm.sum_dy_xmu")
            g_sum_dy = synchronize(h1)
            g_sum_dy_xmu = synchronize(h2)
            mean_dy = (g_sum_dy / total).view(shape)
            mean_dy_xmu = (g_sum_dy_xmu / total).view(shape)
            w = weight.float().view(shape) if weight is not None else 1.0
            inv = invstd.view(shape)
            grad_input = (dy - mean_dy - xmu * inv * inv * mean_dy_xmu) * inv * w
            grad_input = grad_input.to(ctx.in_dtype)
        return grad_input, grad_weight, grad_bias, None, None, None, None
