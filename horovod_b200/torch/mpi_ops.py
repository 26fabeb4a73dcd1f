"""Collective operations on torch tensors.

Every op exists in an asynchronous form returning a handle (``*_async``),
an in-place form (trailing underscore) and a blocking, autograd-aware form.
All of them accept ``process_set=``. Tensors are identified across ranks by
``name``; unnamed ops get ``<op>.noname.<handle>``, so unnamed ops must be
issued in the same order on every rank.

Parity: horovod/torch/mpi_ops.py:63-903. Extensions: reducescatter, bf16,
Min/Max/Product, process_set on every op.
"""
import os

import torch

from horovod_b200 import _C
from horovod_b200.common.basics import HorovodBasics
from horovod_b200.common.exceptions import HorovodInternalError
from horovod_b200.common.process_sets import _resolve, global_process_set
from horovod_b200.common.util import (get_average_backwards_compatibility_fun,
                                      num_rank_is_power_2)
from horovod_b200.torch.compression import Compression

_basics = HorovodBasics()

init = _basics.init


def shutdown():
    """Stops the background thread and releases its resources; init() may be
    called again afterwards."""
    _barrier_counts.clear()  # survivors and newcomers of an elastic reset agree again
    _basics.shutdown()


is_initialized = _basics.is_initialized
size = _basics.size
local_size = _basics.local_size
cross_size = _basics.cross_size
rank = _basics.rank
local_rank = _basics.local_rank
cross_rank = _basics.cross_rank
is_homogeneous = _basics.is_homogeneous
start_timeline = _basics.start_timeline
stop_timeline = _basics.stop_timeline
mpi_threads_supported = _basics.mpi_threads_supported
mpi_enabled = _basics.mpi_enabled
mpi_built = _basics.mpi_built
gloo_enabled = _basics.gloo_enabled
gloo_built = _basics.gloo_built
nccl_built = _basics.nccl_built
ddl_built = _basics.ddl_built
ccl_built = _basics.ccl_built
cuda_built = _basics.cuda_built
rocm_built = _basics.rocm_built
gpu_backend = _basics.gpu_backend
runtime_params = _basics.runtime_params
topology = _basics.topology


class _ReduceOps:
    Average = 0
    Sum = 1
    Adasum = 2
    Min = 3
    Max = 4
    Product = 5


Average = _ReduceOps.Average
Sum = _ReduceOps.Sum
Adasum = _ReduceOps.Adasum
Min = _ReduceOps.Min
Max = _ReduceOps.Max
Product = _ReduceOps.Product

handle_average_backwards_compatibility = get_average_backwards_compatibility_fun(_ReduceOps)

# handle -> (kind, extra) so that synchronize() knows how to shape the result.
_handle_map = {}


def _enqueue(native_op, *args):
    """Hands an op to the background thread. A runtime failure at this point
    (the job has been shut down, a peer died, a tensor name is already in
    flight) is the same kind of event as one reported at synchronize():
    HorovodInternalError, which elastic jobs catch and recover from
    (horovod/torch/mpi_ops.py:137-138)."""
    try:
        return native_op(*args)
    except RuntimeError as e:
        raise HorovodInternalError(e)


def _is_dense(tensor):
    """Contiguous in some memory format (e.g. channels_last): element-wise
    collectives only need the same dense layout on every rank."""
    return (tensor.is_contiguous()
            or (tensor.dim() == 4 and tensor.is_contiguous(memory_format=torch.channels_last))
            or (tensor.dim() == 5
                and tensor.is_contiguous(memory_format=torch.channels_last_3d)))


def _check_tensor(tensor, dense_ok=False):
    if not isinstance(tensor, torch.Tensor):
        raise ValueError("Horovod collectives need torch tensors, got %s" % type(tensor))
    if tensor.is_sparse:
        raise ValueError("Sparse tensors are not supported by this op; use "
                         "sparse_allreduce_async or sparse_as_dense=True.")
    if not (tensor.is_contiguous() or (dense_ok and _is_dense(tensor))):
        raise ValueError("Horovod collectives need contiguous tensors; "
                         "call .contiguous() first.")


def _check_adasum(op, process_set):
    if op != Adasum:
        return
    ps_size = process_set.size() if process_set is not None else size()
    if not num_rank_is_power_2(ps_size):
        raise NotImplementedError(
            "Running Adasum needs a power-of-two number of ranks; this set has %d." % ps_size)


def _scaled_op(op, prescale_factor, postscale_factor):
    return int(op), float(prescale_factor), float(postscale_factor)


_WIRE_IDS = {torch.float16: 6, torch.bfloat16: 10}


def _wire_id(tensor, wire_dtype):
    """Wire format id for the native call: fp32 CUDA tensors can be cast to a
    16-bit type inside the collective kernel; anything else is sent as is."""
    if wire_dtype is None or not tensor.is_cuda or tensor.dtype != torch.float32:
        return -1
    return _WIRE_IDS.get(wire_dtype, -1)


# ---- shadow check ------------------------------------------------------------
# HOROVOD_SHADOW_CHECK=1: every allreduce of a CUDA tensor is also computed on
# fp64 host copies of the inputs by the CPU data plane (an independent
# implementation: TCP mesh, no kernels of this library), and synchronize()
# compares the two. A debugging aid: it synchronises the stream at every call
# and moves every tensor a second time. "all" shadows CPU tensors as well
# (catches what a narrow accumulation type loses).
_shadow_mode = os.environ.get("HOROVOD_SHADOW_CHECK", "0").lower()
_shadow_map = {}     # handle of the checked op -> (handle of its shadow, dtype, wire dtype)
_shadow_counter = [0]


class ShadowMismatch(RuntimeError):
    """The device result of a collective differs from its host shadow."""


def set_shadow_check(mode):
    """``False`` / ``True`` / ``"all"`` at run time; the same on every rank."""
    global _shadow_mode
    _shadow_mode = {False: "0", True: "1"}.get(mode, str(mode).lower())


def _shadow_wanted(tensor, op):
    if _shadow_mode in ("0", "", "false", "off") or (op is not None and op == Adasum):
        return False
    return tensor.is_cuda or _shadow_mode == "all"


def _shadow_tolerance(dtype, wire_dtype, ranks):
    """(rtol, atol factor of the largest magnitude) for a result of ``dtype``."""
    narrow = dtype in (torch.float16, torch.bfloat16) or wire_dtype in (torch.float16,
                                                                         torch.bfloat16)
    if not dtype.is_floating_point:
        return 0.0, 0.0
    if narrow:
        return 2e-2, 1e-2 * ranks
    return (1e-5, 1e-6 * ranks) if dtype == torch.float32 else (1e-12, 1e-13 * ranks)


_shadow_per_set = {}  # process set id -> shadows of unnamed ops started on that set


def _shadow_name(label, name=None, process_set=None):
    """The shadow of a named op is named after it; shadows of unnamed ops are
    numbered per process set, whose members all issue the same sequence."""
    _shadow_counter[0] += 1
    if name:
        return "hvd.shadow.%s.%s" % (label, name)
    ps_id = _resolve(process_set)
    _shadow_per_set[ps_id] = _shadow_per_set.get(ps_id, 0) + 1
    return "hvd.shadow.%s.noname.%d.%d" % (label, ps_id, _shadow_per_set[ps_id])


def _host_copy(tensor, widen):
    target = torch.float64 if widen and tensor.is_floating_point() else tensor.dtype
    return tensor.detach().to("cpu", target, copy=True).contiguous()


def _start_shadow(handle, tensors, op, prescale_factor, postscale_factor, process_set, wire_dtype,
                  name=None):
    """``tensors``: the inputs of the allreduce behind ``handle`` (one, or the
    list of a grouped op, which is shadowed as one flat vector)."""
    wide = torch.cat([_host_copy(t, True).reshape(-1) for t in tensors]).contiguous()
    shadow = _enqueue(_C.allreduce_async, wide, torch.empty_like(wide),
                      _shadow_name("allreduce", name, process_set),
                      *_scaled_op(op, prescale_factor, postscale_factor), _resolve(process_set), -1)
    narrow = [t.dtype for t in tensors if t.dtype in (torch.float16, torch.bfloat16)]
    _shadow_map[handle] = (shadow, "allreduce", narrow[0] if narrow else tensors[0].dtype,
                           wire_dtype, process_set.size() if process_set is not None else size())


def _start_exact_shadow(handle, label, enqueue_twin, name=None, process_set=None):
    """For the ops that only move data: ``enqueue_twin(name)`` starts the
    same op on host copies; the results must be equal."""
    _shadow_map[handle] = (enqueue_twin(_shadow_name(label, name, process_set)), label, None,
                           None, 1)


def _finish_shadow(handle, results):
    shadow, label, dtype, wire_dtype, ranks = _shadow_map.pop(handle)
    try:
        expected = _C.wait_and_clear(shadow)[0][0]
    except RuntimeError as e:
        raise HorovodInternalError(e)
    flat = [r.detach().reshape(-1) for r in results]
    if len(results) == 1 and label != "allreduce" and tuple(results[0].shape) != tuple(expected.shape):
        raise ShadowMismatch("%s result has shape %s, its host shadow %s"
                             % (label, tuple(results[0].shape), tuple(expected.shape)))
    expected = expected.reshape(-1)
    got = torch.cat([r.to("cpu", expected.dtype) for r in flat])
    rtol, atol_factor = (0.0, 0.0) if dtype is None else _shadow_tolerance(dtype, wire_dtype, ranks)
    scale = float(expected.abs().max()) if expected.numel() and expected.dtype != torch.bool else 0.0
    if expected.dtype == torch.bool:
        bad = got != expected
        worst = float(bad.any())
    else:
        diff = (got - expected).abs()
        bad = diff > rtol * expected.abs() + atol_factor * max(scale, 1e-30)
        worst = float(diff.max()) if diff.numel() else 0.0
    if bool(bad.any()):
        raise ShadowMismatch(
            "%s result differs from its host shadow in %d of %d elements (largest "
            "difference %.3e, largest expected magnitude %.3e, dtype %s)"
            % (label, int(bad.sum()), expected.numel(), worst, scale, dtype or results[0].dtype))


def _shadow_group_ok(tensors, op):
    """A grouped op is shadowed when its tensors can share one flat vector."""
    if not tensors or not _shadow_wanted(tensors[0], op):
        return False
    kinds = {t.is_floating_point() for t in tensors}
    return len(kinds) == 1 and (True in kinds or len({t.dtype for t in tensors}) == 1)


def _allreduce_async(tensor, output, name, op, prescale_factor, postscale_factor, process_set,
                     wire_dtype=None):
    _check_tensor(tensor, dense_ok=True)
    _check_adasum(op, process_set)
    if _shadow_wanted(tensor, op) and (op != Average or tensor.is_floating_point()):
        # the copy comes first: an in-place op overwrites its input
        wide_input = tensor.detach().clone() if tensor is output else tensor
        handle = _allreduce_async_unchecked(tensor, output, name, op, prescale_factor,
                                            postscale_factor, process_set, wire_dtype)
        _start_shadow(handle, [wide_input], op, prescale_factor, postscale_factor, process_set,
                      wire_dtype, name)
        return handle
    return _allreduce_async_unchecked(tensor, output, name, op, prescale_factor, postscale_factor,
                                      process_set, wire_dtype)


def _allreduce_async_unchecked(tensor, output, name, op, prescale_factor, postscale_factor,
                               process_set, wire_dtype=None):
    if op == Average and not (tensor.is_floating_point() or tensor.is_complex()):
        # Integer averaging: sum on the wire, floor-divide afterwards, as the
        # framework's integer division would.
        handle = _enqueue(_C.allreduce_async, tensor, output, name or "", Sum, float(prescale_factor),
                                    float(postscale_factor), _resolve(process_set))
        divisor = process_set.size() if process_set is not None else size()
        _handle_map[handle] = ("allreduce_intavg", divisor)
        return handle
    handle = _enqueue(_C.allreduce_async, tensor, output, name or "", *_scaled_op(
        op, prescale_factor, postscale_factor), _resolve(process_set),
        _wire_id(tensor, wire_dtype) if op in (Average, Sum) else -1)
    _handle_map[handle] = ("allreduce", None)
    return handle


def allreduce_async(tensor, average=None, name=None, op=None, prescale_factor=1.0,
                    postscale_factor=1.0, process_set=global_process_set):
    """Starts an allreduce of ``tensor`` into a new tensor and returns a
    handle for poll() / synchronize()."""
    op = handle_average_backwards_compatibility(op, average)
    output = torch.empty_like(tensor)
    return _allreduce_async(tensor, output, name, op, prescale_factor, postscale_factor,
                            process_set)


class HorovodAllreduce(torch.autograd.Function):
    """Allreduce whose gradient is the allreduce of the incoming gradient."""

    @staticmethod
    def forward(ctx, tensor, average, name, op, prescale_factor, postscale_factor, process_set):
        ctx.average = average
        ctx.op = op
        ctx.prescale_factor = prescale_factor
        ctx.postscale_factor = postscale_factor
        ctx.process_set = process_set
        handle = allreduce_async(tensor, average, name, op, prescale_factor,
                                 postscale_factor, process_set)
        return synchronize(handle)

    @staticmethod
    def backward(ctx, grad_output):
        return (allreduce(grad_output.contiguous(), average=ctx.average, op=ctx.op,
                          prescale_factor=ctx.prescale_factor,
                          postscale_factor=ctx.postscale_factor,
                          process_set=ctx.process_set),
                None, None, None, None, None, None)


def allreduce(tensor, average=None, name=None, compression=Compression.none, op=None,
              prescale_factor=1.0, postscale_factor=1.0, process_set=global_process_set):
    """Reduces ``tensor`` over all ranks of the process set and returns the
    result on every rank. Differentiable. ``op`` is Average (default), Sum,
    Adasum, Min, Max or Product."""
    tensor_compressed, ctx = compression.compress(tensor)
    summed = HorovodAllreduce.apply(tensor_compressed, average, name, op,
                                    prescale_factor, postscale_factor, process_set)
    return compression.decompress(summed, ctx)


def allreduce_async_(tensor, average=None, name=None, op=None, prescale_factor=1.0,
                     postscale_factor=1.0, process_set=global_process_set, wire_dtype=None):
    """In-place asynchronous allreduce. ``wire_dtype`` (torch.float16 or
    torch.bfloat16) makes an fp32 CUDA tensor travel in that format: the
    casts happen inside the collective kernel instead of as separate torch
    kernels, and the tensor itself stays fp32."""
    op = handle_average_backwards_compatibility(op, average)
    return _allreduce_async(tensor, tensor, name, op, prescale_factor, postscale_factor,
                            process_set, wire_dtype)


def allreduce_(tensor, average=None, name=None, op=None, prescale_factor=1.0,
               postscale_factor=1.0, process_set=global_process_set):
    """In-place blocking allreduce."""
    handle = allreduce_async_(tensor, average, name, op, prescale_factor,
                              postscale_factor, process_set)
    return synchronize(handle)


def _grouped_allreduce_async(tensors, outputs, name, op, prescale_factor, postscale_factor,
                             process_set, wire_dtype=None):
    for t in tensors:
        _check_tensor(t, dense_ok=True)
    _check_adasum(op, process_set)
    int_avg = op == Average and any(not t.is_floating_point() for t in tensors)
    wire_op = Sum if int_avg else op
    shadowed = None
    if not int_avg and _shadow_group_ok(tensors, op):
        # copies first: an in-place group overwrites its inputs
        shadowed = [t.detach().clone() if any(t is o for o in outputs) else t for t in tensors]
    handle = _enqueue(_C.grouped_allreduce_async, list(tensors), list(outputs), name or "",
                                        int(wire_op), float(prescale_factor),
                                        float(postscale_factor), _resolve(process_set),
                                        _wire_id(tensors[0], wire_dtype)
                                        if tensors and wire_op in (Average, Sum)
                                        and all(t.dtype == torch.float32 and t.is_cuda
                                                for t in tensors) else -1)
    if int_avg:
        divisor = process_set.size() if process_set is not None else size()
        _handle_map[handle] = ("grouped_intavg", divisor)
    else:
        _handle_map[handle] = ("grouped", None)
    if shadowed is not None:
        _start_shadow(handle, shadowed, op, prescale_factor, postscale_factor, process_set,
                      wire_dtype, name)
    return handle


def grouped_allreduce_async(tensors, average=None, name=None, op=None, prescale_factor=1.0,
                            postscale_factor=1.0, process_set=global_process_set):
    """Allreduce of a list of tensors negotiated and fused as one unit."""
    op = handle_average_backwards_compatibility(op, average)
    outputs = [torch.empty_like(t) for t in tensors]
    return _grouped_allreduce_async(tensors, outputs, name, op, prescale_factor,
                                    postscale_factor, process_set)


class HorovodGroupedAllreduce(torch.autograd.Function):
    @staticmethod
    def forward(ctx, average, name, op, prescale_factor, postscale_factor, process_set,
                *tensors):
        ctx.average = average
        ctx.op = op
        ctx.prescale_factor = prescale_factor
        ctx.postscale_factor = postscale_factor
        ctx.process_set = process_set
        handle = grouped_allreduce_async(list(tensors), average, name, op, prescale_factor,
                                         postscale_factor, process_set)
        return tuple(synchronize(handle))

    @staticmethod
    def backward(ctx, *grad_output):
        grads = grouped_allreduce([g.contiguous() for g in grad_output],
                                  average=ctx.average, op=ctx.op,
                                  prescale_factor=ctx.prescale_factor,
                                  postscale_factor=ctx.postscale_factor,
                                  process_set=ctx.process_set)
        return (None, None, None, None, None, None, *grads)


def grouped_allreduce(tensors, average=None, name=None, compression=Compression.none,
                      op=None, prescale_factor=1.0, postscale_factor=1.0,
                      process_set=global_process_set):
    """Blocking, differentiable grouped allreduce. Returns a list."""
    compressed, ctxs = zip(*[compression.compress(t) for t in tensors]) if tensors else ((), ())
    summed = HorovodGroupedAllreduce.apply(average, name, op, prescale_factor,
                                           postscale_factor, process_set, *compressed)
    return [compression.decompress(t, c) for t, c in zip(summed, ctxs)]


def grouped_allreduce_async_(tensors, average=None, name=None, op=None, prescale_factor=1.0,
                             postscale_factor=1.0, process_set=global_process_set,
                             wire_dtype=None):
    op = handle_average_backwards_compatibility(op, average)
    return _grouped_allreduce_async(tensors, tensors, name, op, prescale_factor,
                                    postscale_factor, process_set, wire_dtype)


def grouped_allreduce_(tensors, average=None, name=None, op=None, prescale_factor=1.0,
                       postscale_factor=1.0, process_set=global_process_set):
    handle = grouped_allreduce_async_(tensors, average, name, op, prescale_factor,
                                      postscale_factor, process_set)
    return synchronize(handle)


def sparse_allreduce_async(tensor, name, op, process_set=global_process_set):
    """Allreduce of a sparse COO tensor as two allgathers (indices, values).
    Returns a function that waits and builds the result."""
    t = tensor.coalesce() if not tensor.is_coalesced() else tensor
    indices_handle = allgather_async(t._indices().transpose(0, 1).contiguous(),
                                     name="%s.indices" % name, process_set=process_set)
    values_handle = allgather_async(t._values(), name="%s.values" % name,
                                    process_set=process_set)

    def handle():
        indices = synchronize(indices_handle)
        values = synchronize(values_handle)
        n = process_set.size() if process_set is not None else size()
        values = values / n if op == Average else values
        if indices.dim() == 0 or values.dim() == 0:
            return t.new_empty(t.shape)
        return torch.sparse_coo_tensor(indices.transpose(0, 1), values, t.shape)

    return handle


def allgather_async(tensor, name=None, process_set=global_process_set):
    """Starts concatenating ``tensor`` from all ranks along dimension 0
    (dimension 0 may differ between ranks)."""
    _check_tensor(tensor)
    handle = _enqueue(_C.allgather_async, tensor, name or "", _resolve(process_set))
    _handle_map[handle] = ("allgather", None)
    if _shadow_wanted(tensor, None):
        twin = _host_copy(tensor, False)
        _start_exact_shadow(handle, "allgather", lambda shadow_name: _enqueue(
            _C.allgather_async, twin, shadow_name, _resolve(process_set)), name, process_set)
    return handle


class HorovodAllgather(torch.autograd.Function):
    @staticmethod
    def forward(ctx, tensor, name, process_set):
        ctx.dim = tensor.shape[0]
        ctx.process_set = process_set
        handle = allgather_async(tensor, name, process_set)
        return synchronize(handle)

    @staticmethod
    def backward(ctx, grad_output):
        ps = ctx.process_set
        grad_reduced = allreduce(grad_output.contiguous(), average=True, process_set=ps)
        dim_t = torch.tensor([ctx.dim], dtype=torch.int64)
        dims = allgather(dim_t, process_set=ps).view(-1)
        r = ps.rank() if ps is not None else rank()
        offset = int(dims[:r].sum().item()) if r != 0 else 0
        return grad_reduced.narrow(0, offset, ctx.dim), None, None


def allgather(tensor, name=None, process_set=global_process_set):
    """Blocking, differentiable allgather."""
    return HorovodAllgather.apply(tensor, name, process_set)


def _broadcast_async(tensor, output, root_rank, name, process_set):
    _check_tensor(tensor, dense_ok=True)
    twin = _host_copy(tensor, False) if _shadow_wanted(tensor, None) else None  # before an in-place op
    handle = _enqueue(_C.broadcast_async, tensor, output, int(root_rank), name or "",
                                _resolve(process_set))
    _handle_map[handle] = ("broadcast", None)
    if twin is not None:
        _start_exact_shadow(handle, "broadcast", lambda shadow_name: _enqueue(
            _C.broadcast_async, twin, twin, int(root_rank), shadow_name, _resolve(process_set)),
            name, process_set)
    return handle


def broadcast_async(tensor, root_rank, name=None, process_set=global_process_set):
    """Starts broadcasting ``tensor`` from global rank ``root_rank``."""
    output = torch.empty_like(tensor)
    return _broadcast_async(tensor, output, root_rank, name, process_set)


class HorovodBroadcast(torch.autograd.Function):
    @staticmethod
    def forward(ctx, tensor, root_rank, name, process_set):
        ctx.root_rank = root_rank
        ctx.process_set = process_set
        handle = broadcast_async(tensor, root_rank, name, process_set)
        return synchronize(handle)

    @staticmethod
    def backward(ctx, grad_output):
        grad_reduced = allreduce(grad_output.contiguous(), average=True,
                                 process_set=ctx.process_set)
        if rank() != ctx.root_rank:
            grad_reduced *= 0
        return grad_reduced, None, None, None


def broadcast(tensor, root_rank, name=None, process_set=global_process_set):
    """Blocking, differentiable broadcast."""
    return HorovodBroadcast.apply(tensor, root_rank, name, process_set)


def broadcast_async_(tensor, root_rank, name=None, process_set=global_process_set):
    return _broadcast_async(tensor, tensor, root_rank, name, process_set)


def broadcast_(tensor, root_rank, name=None, process_set=global_process_set):
    handle = broadcast_async_(tensor, root_rank, name, process_set)
    return synchronize(handle)


def _splits_list(splits):
    if splits is None:
        return []
    if isinstance(splits, torch.Tensor):
        if splits.dim() != 1 or splits.dtype not in (torch.int32, torch.int64):
            raise ValueError("splits must be a 1-D integer tensor")
        return [int(v) for v in splits.cpu().tolist()]
    return [int(v) for v in splits]


def alltoall_async(tensor, splits=None, name=None, process_set=global_process_set):
    """Starts an all-to-all: rows ``splits[i]`` of dimension 0 go to rank i
    (an even split when ``splits`` is None)."""
    _check_tensor(tensor)
    handle = _enqueue(_C.alltoall_async, tensor, _splits_list(splits), name or "",
                               _resolve(process_set))
    _handle_map[handle] = ("alltoall", splits is not None)
    if _shadow_wanted(tensor, None):
        twin = _host_copy(tensor, False)
        _start_exact_shadow(handle, "alltoall", lambda shadow_name: _enqueue(
            _C.alltoall_async, twin, _splits_list(splits), shadow_name, _resolve(process_set)),
            name, process_set)
    return handle


class HorovodAlltoall(torch.autograd.Function):
    @staticmethod
    def forward(ctx, tensor, splits, name, process_set):
        handle = alltoall_async(tensor, splits, name, process_set)
        result = synchronize(handle)
        ctx.process_set = process_set
        if splits is None:
            # Even split both ways.
            ctx.recvsplits = None
            return result
        output, recv = result
        ctx.recvsplits = recv
        ctx.mark_non_differentiable(recv)
        return output, recv

    @staticmethod
    def backward(ctx, grad_output, *dead_gradients):
        out = alltoall(grad_output.contiguous(), splits=ctx.recvsplits,
                       process_set=ctx.process_set)
        grad = out[0] if isinstance(out, tuple) else out
        return grad, None, None, None


def alltoall(tensor, splits=None, name=None, process_set=global_process_set):
    """Blocking, differentiable all-to-all. Returns ``output`` or, when
    ``splits`` was given, ``(output, received_splits)``."""
    return HorovodAlltoall.apply(tensor, splits, name, process_set)


def reducescatter_async(tensor, name=None, op=Average, prescale_factor=1.0,
                        postscale_factor=1.0, process_set=global_process_set):
    """Starts a reduce-scatter: the reduction of ``tensor`` over all ranks is
    split along dimension 0 and rank r keeps chunk r (the first
    ``dim0 % size`` ranks get one extra row)."""
    _check_tensor(tensor)
    if op == Adasum:
        raise ValueError("reducescatter does not support Adasum")
    handle = _enqueue(_C.reducescatter_async, tensor, name or "", int(op), float(prescale_factor),
                                    float(postscale_factor), _resolve(process_set))
    _handle_map[handle] = ("reducescatter", None)
    if _shadow_wanted(tensor, op) and (op != Average or tensor.is_floating_point()):
        wide = _host_copy(tensor, True)
        shadow = _enqueue(_C.reducescatter_async, wide,
                          _shadow_name("reducescatter", name, process_set), int(op),
                          float(prescale_factor), float(postscale_factor), _resolve(process_set))
        _shadow_map[handle] = (shadow, "reducescatter", tensor.dtype, None,
                               process_set.size() if process_set is not None else size())
    return handle


class HorovodReducescatter(torch.autograd.Function):
    @staticmethod
    def forward(ctx, tensor, name, op, prescale_factor, postscale_factor, process_set):
        ctx.op = op
        ctx.process_set = process_set
        ctx.scale = prescale_factor * postscale_factor
        handle = reducescatter_async(tensor, name, op, prescale_factor, postscale_factor,
                                     process_set)
        return synchronize(handle)

    @staticmethod
    def backward(ctx, grad_output):
        ps = ctx.process_set
        n = ps.size() if ps is not None else size()
        grad = allgather(grad_output.contiguous(), process_set=ps) * ctx.scale
        if ctx.op == Average:
            grad = grad / n
        return grad, None, None, None, None, None


def reducescatter(tensor, name=None, compression=Compression.none, op=Average,
                  prescale_factor=1.0, postscale_factor=1.0, process_set=global_process_set):
    """Blocking, differentiable reduce-scatter."""
    tensor_compressed, ctx = compression.compress(tensor)
    out = HorovodReducescatter.apply(tensor_compressed, name, op, prescale_factor,
                                     postscale_factor, process_set)
    return compression.decompress(out, ctx)


def symmetric_empty(*size, dtype=torch.float32):
    """Allocates a CUDA tensor inside the symmetric heap: memory that every
    GPU of the box has mapped, at the same offset on every rank. Collective by
    contract: all ranks must call it with the same sizes in the same order.
    Allreduce on such tensors (in place, whole tensors or 16-byte aligned
    slices) runs without any staging copy: the kernel reduces the ranks'
    tensors directly over NVLink. The memory is never freed individually and
    becomes invalid at hvd.shutdown(). Size the heap with
    HOROVOD_SYMM_HEAP_MB (default 4096)."""
    if len(size) == 1 and isinstance(size[0], (tuple, list, torch.Size)):
        size = tuple(size[0])
    if not gpu_backend().startswith("symm"):
        # The arena is built by the first device collective of the job.
        if not torch.cuda.is_available():
            raise RuntimeError("symmetric memory needs CUDA")
        allreduce_(torch.zeros(1, device="cuda"), op=Sum, name="hvd.symm.bootstrap")
    if not gpu_backend().startswith("symm"):
        raise RuntimeError("symmetric memory is not available: " + gpu_backend())
    return _C.symm_empty([int(s) for s in size], dtype)


def poll(handle):
    """True once the op behind ``handle`` has run (CPU) or been launched
    (GPU); synchronize() will then not block the host."""
    return _C.poll(handle)


def synchronize(handle):
    """Waits for an asynchronous op and returns its result. GPU ops are
    chained onto the current CUDA stream rather than host-synchronised."""
    if handle not in _handle_map:
        return None
    kind, extra = _handle_map.pop(handle)
    try:
        outputs, recv_splits, _ = _C.wait_and_clear(handle)
    except RuntimeError as e:
        raise HorovodInternalError(e)
    if kind == "allreduce":
        if handle in _shadow_map:
            _finish_shadow(handle, [outputs[0]])
        return outputs[0]
    if kind == "allreduce_intavg":
        outputs[0].copy_(torch.div(outputs[0], extra, rounding_mode="floor"))
        return outputs[0]
    if kind == "grouped":
        if handle in _shadow_map:
            _finish_shadow(handle, list(outputs))
        return list(outputs)
    if kind == "grouped_intavg":
        for o in outputs:
            if not o.is_floating_point():
                o.copy_(torch.div(o, extra, rounding_mode="floor"))
            else:
                o.div_(extra)
        return list(outputs)
    if handle in _shadow_map:  # allgather, broadcast, alltoall, reducescatter
        _finish_shadow(handle, [outputs[0]])
    if kind == "alltoall":
        out = outputs[0]
        if extra:
            return out, torch.tensor(recv_splits, dtype=torch.int32)
        return out
    return outputs[0]


_barrier_counts = {}


def barrier(process_set=global_process_set):
    """Returns once every rank of the process set has called it (and every
    collective this rank enqueued before has been negotiated). An extension
    that later releases of the reference also offer."""
    ps_id = _resolve(process_set)
    count = _barrier_counts.get(ps_id, 0)
    _barrier_counts[ps_id] = count + 1
    # Named by a per-set call counter, which is the same on every rank
    # whatever else the ranks have enqueued.
    synchronize(allreduce_async(torch.zeros(1), op=Sum, name="hvd.barrier.%d.%d" % (ps_id, count),
                                process_set=process_set))


def grouped_allgather_async(tensors, name=None, process_set=global_process_set):
    """Starts the allgather of a list of tensors as one group: the controller
    negotiates the members together and fuses them, so tensors of one dtype
    travel in one kernel launch. ``synchronize`` returns the list of gathered
    tensors in order."""
    tensors = list(tensors)
    for t in tensors:
        _check_tensor(t)
    handle = _enqueue(_C.grouped_allgather_async, tensors, name or "", _resolve(process_set))
    _handle_map[handle] = ("grouped", None)
    return handle


def grouped_allgather(tensors, name=None, process_set=global_process_set):
    """Allgathers a list of tensors as one group. Returns the gathered tensors
    in order."""
    return synchronize(grouped_allgather_async(tensors, name, process_set))


def grouped_reducescatter_async(tensors, name=None, op=Average, prescale_factor=1.0,
                                postscale_factor=1.0, process_set=global_process_set):
    """Starts the reduce-scatter of a list of tensors as one group (one fused
    response and, for device tensors of one dtype, one kernel launch).
    ``synchronize`` returns this rank's shards in order."""
    tensors = list(tensors)
    for t in tensors:
        _check_tensor(t)
    if op == Adasum:
        raise ValueError("reducescatter does not support Adasum")
    handle = _enqueue(_C.grouped_reducescatter_async, tensors, name or "", int(op),
                      float(prescale_factor), float(postscale_factor), _resolve(process_set))
    _handle_map[handle] = ("grouped", None)
    return handle


def grouped_reducescatter(tensors, name=None, op=Average, prescale_factor=1.0,
                          postscale_factor=1.0, process_set=global_process_set):
    """Reduce-scatters a list of tensors as one group; returns this rank's
    shards in order."""
    return synchronize(grouped_reducescatter_async(tensors, name, op, prescale_factor,
                                                   postscale_factor, process_set))


def join(device=-1, process_set=global_process_set):
    """Tells the other ranks this rank has no more data. Blocks until every
    rank has joined; meanwhile this rank contributes zeros to their
    allreduces. Returns the rank that joined last."""
    handle = _enqueue(_C.join_async, _resolve(process_set))
    try:
        _, _, last = _C.wait_and_clear(handle)
    except RuntimeError as e:
        raise HorovodInternalError(e)
    return last
