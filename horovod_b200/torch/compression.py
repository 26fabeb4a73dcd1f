"""Gradient compression applied around allreduce.

Parity: horovod/torch/compression.py:20-74, plus a bf16 compressor. When
gradients travel through DistributedOptimizer on CUDA, the fp32 <-> 16-bit
casts of these compressors are not run as separate torch kernels: the fused
allreduce kernel reads fp32, puts 16-bit values on the wire and writes fp32
back (see ``wire_dtype``).
"""
import torch


class Compressor:
    """Interface: compress(tensor) -> (tensor, ctx); decompress(tensor, ctx)."""
    # dtype that floating-point gradients take on the wire, or None.
    wire_dtype = None

    @staticmethod
    def compress(tensor):
        raise NotImplementedError

    @staticmethod
    def decompress(tensor, ctx):
        raise NotImplementedError


class NoneCompressor(Compressor):
    @staticmethod
    def compress(tensor):
        return tensor, None

    @staticmethod
    def decompress(tensor, ctx):
        return tensor


class _CastCompressor(Compressor):
    @classmethod
    def compress(cls, tensor):
        ctx = tensor.dtype
        if tensor.dtype.is_floating_point and tensor.dtype != cls.wire_dtype:
            tensor = tensor.to(cls.wire_dtype)
        return tensor, ctx

    @classmethod
    def decompress(cls, tensor, ctx):
        if ctx is not None and ctx.is_floating_point and tensor.dtype != ctx:
            tensor = tensor.to(ctx)
        return tensor


class FP16Compressor(_CastCompressor):
    """Floating-point tensors travel as float16."""
    wire_dtype = torch.float16


class BF16Compressor(_CastCompressor):
    """Floating-point tensors travel as bfloat16 (fp32 range, 8-bit mantissa)."""
    wire_dtype = torch.bfloat16


class Compression:
    none = NoneCompressor
    fp16 = FP16Compressor
    bf16 = BF16Compressor
