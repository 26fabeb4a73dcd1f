"""DistributedOptimizer: wraps any torch optimizer so that gradients are
averaged (or Adasum-combined) across ranks while backward is still running.

A hook on every parameter fires as soon as that parameter's gradient has been
accumulated and enqueues an asynchronous in-place allreduce; ``step()`` waits
for all of them and then runs the wrapped optimizer.

Parity: horovod/torch/optimizer.py:35-590.
"""
import warnings
from contextlib import contextmanager

import torch

from horovod_b200.common.process_sets import global_process_set
from horovod_b200.common.util import split_list
from horovod_b200.torch.compression import Compression
from horovod_b200.torch.functions import broadcast_object
from horovod_b200.torch.mpi_ops import (Adasum, Average, Sum, allreduce_async_,
                                        grouped_allreduce_async_, rank, size,
                                        sparse_allreduce_async, synchronize)


class _DistributedOptimizer(torch.optim.Optimizer):
    def __init__(self, params, named_parameters, compression, backward_passes_per_step=1,
                 op=Average, gradient_predivide_factor=1.0, groups=None,
                 sparse_as_dense=False, process_set=global_process_set,
                 symmetric_gradients=False):
        super(self.__class__, self).__init__(params)
        self._compression = compression
        self._symm_flats = []
        if named_parameters is not None:
            named_parameters = list(named_parameters)
        else:
            named_parameters = [("allreduce.noname.%s.%s" % (gi, pi), v)
                                for gi, group in enumerate(self.param_groups)
                                for pi, v in enumerate(group["params"])]
        if any(not isinstance(p, tuple) for p in named_parameters):
            raise ValueError("named_parameters should be a sequence of tuples (name, "
                             "parameter), usually produced by model.named_parameters().")
        dups = _find_duplicates([k for k, _ in named_parameters])
        if dups:
            raise ValueError("Parameter names in named_parameters must be unique. "
                             "Found duplicates: %s" % ", ".join(dups))
        all_param_ids = {id(v) for group in self.param_groups for v in group["params"]}
        named_param_ids = {id(v) for _, v in named_parameters}
        unnamed = all_param_ids - named_param_ids
        if unnamed:
            raise ValueError("named_parameters was specified, but one or more model "
                             "parameters were not named. Python object ids: %s"
                             % ", ".join(str(i) for i in unnamed))

        self._parameter_names = {v: k for k, v in sorted(named_parameters)}
        self.backward_passes_per_step = backward_passes_per_step
        self._allreduce_delay = {v: self.backward_passes_per_step
                                 for _, v in sorted(named_parameters)}
        self.op = op
        self.gradient_predivide_factor = gradient_predivide_factor
        self.sparse_as_dense = sparse_as_dense
        self.process_set = process_set
        self._handles = {}
        self._hook_handles = []
        self._requires_update = set()
        self._synchronized = False
        self._should_synchronize = True

        self._groups = None
        self._p_to_group = {}
        self._group_counts = {}
        if groups is not None:
            if not (isinstance(groups, list) or (isinstance(groups, int) and groups > 0)):
                raise ValueError("groups should be a non-negative integer or a list of "
                                 "lists of torch.Tensor.")
            if isinstance(groups, list):
                grouped_ids = set()
                for g in groups:
                    for p in g:
                        if not isinstance(p, torch.Tensor):
                            raise ValueError("groups must consist of torch.Tensor.")
                        if id(p) in grouped_ids:
                            raise ValueError("A parameter can only appear once in groups.")
                        grouped_ids.add(id(p))
                self._groups = [list(g) for g in groups]
            else:
                # Same grouping on every rank: rank 0's parameter order wins.
                names = [self._parameter_names[p] for p in self._parameter_names]
                if process_set.included() and size() > 1:
                    names = broadcast_object(names, 0, name="hvd.optimizer.group_order",
                                             process_set=process_set)
                by_name = {v: k for k, v in self._parameter_names.items()}
                ordered = [by_name[n] for n in names]
                self._groups = split_list(ordered, groups)
            self._groups = [sorted(g, key=lambda p: self._parameter_names[p])
                            for g in self._groups]
            for gi, g in enumerate(self._groups):
                for p in g:
                    self._p_to_group[p] = gi
                self._group_counts[gi] = 0

        if symmetric_gradients and self.process_set.included():
            self._setup_symmetric_gradients()
        if self.process_set.included() and (size() > 1 or _force_hooks()):
            self._register_hooks()

    def _setup_symmetric_gradients(self):
        """Places every dense CUDA gradient in one flat buffer inside the
        symmetric heap (one buffer per dtype) and makes ``p.grad`` a view of
        it, so that the gradient allreduce runs in place over NVLink with no
        staging copies. Same parameter order on every rank (sorted by name)."""
        from horovod_b200.torch.mpi_ops import symmetric_empty
        import warnings
        try:
            symmetric_empty(64)  # builds the arena; fails on the NCCL path
        except RuntimeError as e:
            warnings.warn("symmetric_gradients ignored: %s" % e)
            return
        by_dtype = {}
        for p, name in sorted(self._parameter_names.items(), key=lambda kv: kv[1]):
            if p.requires_grad and p.is_cuda and p.dtype.is_floating_point and \
                    (p.is_contiguous() or _is_dense(p)):
                by_dtype.setdefault(p.dtype, []).append(p)
        from horovod_b200 import _C
        need = sum((p.numel() * p.element_size() + 255) // 256 * 256
                   for plist in by_dtype.values() for p in plist)
        heap = _C.symm_heap_info()
        if need > heap["bytes"] - heap["used"]:
            warnings.warn("symmetric_gradients ignored: gradients need %d MB, the symmetric "
                          "heap has %d MB left (HOROVOD_SYMM_HEAP_MB)"
                          % (need >> 20, (heap["bytes"] - heap["used"]) >> 20))
            return
        for dtype, plist in sorted(by_dtype.items(), key=lambda kv: str(kv[0])):
            es = torch.empty((), dtype=dtype).element_size()
            slot = 256 // es  # every gradient starts on a 256-byte boundary
            offsets, total = [], 0
            for p in plist:
                offsets.append(total)
                total += (p.numel() + slot - 1) // slot * slot
            flat = symmetric_empty(max(total, slot), dtype=dtype)
            flat.zero_()
            for p, off in zip(plist, offsets):
                p.grad = torch.as_strided(flat, p.size(), p.stride(), storage_offset=off)
            self._symm_flats.append(flat)

    def load_state_dict(self, *args, **kwargs):
        self._handles = {}
        self._synchronized = False
        self._should_synchronize = True
        for p in self._allreduce_delay:
            self._allreduce_delay[p] = self.backward_passes_per_step
        super(self.__class__, self).load_state_dict(*args, **kwargs)

    @staticmethod
    def find_duplicates(lst):
        return _find_duplicates(lst)

    def set_backward_passes_per_step(self, passes):
        self.backward_passes_per_step = passes
        for p in self._allreduce_delay:
            self._allreduce_delay[p] = self.backward_passes_per_step

    def _register_hooks(self):
        for group in self.param_groups:
            for p in group["params"]:
                if p.requires_grad:
                    self._requires_update.add(p)
                    self._hook_handles.append(
                        p.register_post_accumulate_grad_hook(self._make_hook(p)))

    def _scale_factors(self):
        if self.op == Average:
            # Split the averaging between before and after the sum.
            pre = 1.0 / self.gradient_predivide_factor
            post = self.gradient_predivide_factor
            return pre, post
        return 1.0, 1.0

    def _allreduce_grad_async(self, p):
        if p.grad is None:
            # Unused this step: other ranks may still reduce it, send zeros.
            p.grad = p.data.new_zeros(p.size())
        name = self._parameter_names.get(p)
        tensor = p.grad
        if p.grad.is_sparse:
            if self.sparse_as_dense:
                tensor = tensor.to_dense()
            else:
                return self._sparse_allreduce_grad_async(p, name)
        pre, post = self._scale_factors()
        wire = getattr(self._compression, "wire_dtype", None)
        if wire is not None and tensor.is_cuda and tensor.dtype == torch.float32 \
                and self.op in (Average, Sum):
            # The cast to the 16-bit wire format and back happens inside the
            # collective kernel; the gradient tensor stays fp32.
            handle = allreduce_async_(tensor, name=name, op=self.op, prescale_factor=pre,
                                      postscale_factor=post, process_set=self.process_set,
                                      wire_dtype=wire)
            return handle, (tensor, None)
        tensor_compressed, ctx = self._compression.compress(tensor)
        handle = allreduce_async_(tensor_compressed, name=name, op=self.op,
                                  prescale_factor=pre, postscale_factor=post,
                                  process_set=self.process_set)
        return handle, (tensor_compressed, ctx)

    def _grouped_allreduce_grad_async(self, ps):
        name = self._parameter_names.get(ps[0])
        pre, post = self._scale_factors()
        tensors, ctxs = [], []
        for p in ps:
            if p.grad is None:
                p.grad = p.data.new_zeros(p.size())
            t = p.grad.to_dense() if (p.grad.is_sparse and self.sparse_as_dense) else p.grad
            tc, ctx = self._compression.compress(t)
            tensors.append(tc)
            ctxs.append(ctx)
        handle = grouped_allreduce_async_(tensors, name=name, op=self.op,
                                          prescale_factor=pre, postscale_factor=post,
                                          process_set=self.process_set)
        return handle, (tensors, ctxs)

    def _sparse_allreduce_grad_async(self, p, name):
        handle = sparse_allreduce_async(p.grad, name=name, op=self.op,
                                        process_set=self.process_set)
        return handle, None

    def _make_hook(self, p):
        def hook(*ignore):
            if p in self._handles and self._handles[p][0] is not None:
                if self._allreduce_delay[p] <= 0:
                    raise AssertionError(
                        "Gradients were computed more than backward_passes_per_step "
                        "times before call to step(). Increase "
                        "backward_passes_per_step to accumulate gradients locally.")
            assert not p.grad.requires_grad
            assert self._allreduce_delay[p] > 0
            handle, ctx = None, None
            self._allreduce_delay[p] -= 1
            if self._allreduce_delay[p] == 0:
                if self._groups is not None and p in self._p_to_group:
                    gi = self._p_to_group[p]
                    self._group_counts[gi] += 1
                    if self._group_counts[gi] == len(self._groups[gi]):
                        handle, ctxs = self._grouped_allreduce_grad_async(self._groups[gi])
                        self._handles[p] = (handle, ctxs)
                        # The other members share the group's handle.
                        for gp in self._groups[gi]:
                            if gp is not p:
                                self._handles[gp] = (handle, ctxs)
                        self._group_counts[gi] = 0
                        return
                    self._handles[p] = (None, None)
                    return
                handle, ctx = self._allreduce_grad_async(p)
            self._handles[p] = (handle, ctx)
        return hook

    def synchronize(self):
        """Waits for every outstanding gradient reduction and writes the
        results into ``p.grad``. Called by step(); call it yourself before
        gradient clipping and then run step() inside skip_synchronize()."""
        if not self.process_set.included():
            self._synchronized = True
            return
        grouped = self._p_to_group if self._groups is not None else {}
        # Groups that were never launched this step (some member's hook did
        # not fire): launch them whole now.
        if self._groups is not None:
            for gi, g in enumerate(self._groups):
                launched = all(p in self._handles and self._handles[p][0] is not None
                               for p in g)
                if launched or not any(p in self._requires_update for p in g):
                    continue
                handle, ctxs = self._grouped_allreduce_grad_async(g)
                for gp in g:
                    self._handles[gp] = (handle, ctxs)
                self._group_counts[gi] = 0
        # Ungrouped parameters whose hook never fired, or which are still
        # accumulating locally.
        for p in self._requires_update:
            if p in grouped:
                continue
            if p not in self._handles or self._handles[p][0] is None:
                self._handles[p] = self._allreduce_grad_async(p)

        done_handles = {}
        for p, (handle, ctx) in self._handles.items():
            if callable(handle):  # sparse: function that waits and rebuilds
                p.grad = handle()
                self._allreduce_delay[p] = self.backward_passes_per_step
                continue
            if isinstance(ctx, tuple) and isinstance(ctx[0], list):
                # grouped: ctx = (tensors, ctxs)
                if handle not in done_handles:
                    done_handles[handle] = synchronize(handle)
                outputs = done_handles[handle]
                gi = self._p_to_group[p]
                idx = next(i for i, q in enumerate(self._groups[gi]) if q is p)
                tensors, ctxs = ctx
                self._allreduce_delay[p] = self.backward_passes_per_step
                out = outputs[idx] if outputs is not None else tensors[idx]
                self._set_grad(p, self._compression.decompress(out, ctxs[idx]))
                continue
            output = synchronize(handle)
            self._allreduce_delay[p] = self.backward_passes_per_step
            tensor_compressed, cctx = ctx
            out = output if output is not None else tensor_compressed
            self._set_grad(p, self._compression.decompress(out, cctx))
        self._handles.clear()
        self._synchronized = True

    @staticmethod
    def _set_grad(p, value):
        if p.grad is value:
            return
        if p.grad.is_sparse or p.grad.shape != value.shape or p.grad.dtype != value.dtype:
            p.grad = value
        elif p.grad.data_ptr() != value.data_ptr():
            p.grad.copy_(value)

    @contextmanager
    def skip_synchronize(self):
        """Inside this context step() does not synchronize (use after an
        explicit synchronize(), e.g. for gradient clipping)."""
        self._should_synchronize = False
        try:
            yield
        finally:
            self._should_synchronize = True

    def step(self, closure=None):
        if self._should_synchronize:
            if self._synchronized:
                warnings.warn("optimizer.step() called without "
                              "optimizer.skip_synchronize() context after "
                              "optimizer.synchronize(). This can cause training "
                              "slowdown. You may want to consider using "
                              "optimizer.skip_synchronize() context if you use "
                              "optimizer.synchronize() in your code.")
            self.synchronize()
        self._synchronized = False
        return super(self.__class__, self).step(closure)

    def _hvd_base_step(self):
        """The wrapped optimizer's step without any communication."""
        return super(self.__class__, self).step()

    def zero_grad(self, *args, **kwargs):
        if self._handles:
            raise AssertionError(
                "optimizer.zero_grad() was called after loss.backward() but before "
                "optimizer.step() or optimizer.synchronize(). This is prohibited as it "
                "can cause a race condition.")
        if self._symm_flats:
            # Gradients are views of the flat symmetric buffers: clear those
            # (one memset each) and keep the views, whatever set_to_none says.
            for flat in self._symm_flats:
                flat.zero_()
            in_flat = set()
            for group in self.param_groups:
                for p in group["params"]:
                    if p.grad is not None and any(
                            p.grad.untyped_storage().data_ptr() == f.untyped_storage().data_ptr()
                            for f in self._symm_flats):
                        in_flat.add(p)
                    elif p.grad is not None:
                        p.grad = None if kwargs.get("set_to_none", True) else p.grad.zero_()
            return None
        return super(self.__class__, self).zero_grad(*args, **kwargs)


def _is_dense(t):
    return (t.dim() == 4 and t.is_contiguous(memory_format=torch.channels_last)) or \
        (t.dim() == 5 and t.is_contiguous(memory_format=torch.channels_last_3d))


def _force_hooks():
    """Gradient hooks although the job has one rank now: asked for
    (HOROVOD_FORCE_HOOKS, benchmarks at N=1), or an elastic job, which may
    grow later while this optimizer object lives on
    (horovod/torch/optimizer.py:128-131)."""
    import os
    return os.environ.get("HOROVOD_FORCE_HOOKS", "0") == "1" or \
        os.environ.get("HOROVOD_ELASTIC", "0") == "1"


def _find_duplicates(lst):
    seen, dups = set(), set()
    for el in lst:
        if el in seen:
            dups.add(el)
        seen.add(el)
    return sorted(dups)


class _DistributedAdasumOptimizer(torch.optim.Optimizer):
    """Adasum variant: each parameter's *update* (not its gradient) is
    combined across ranks, and step() applies the combined delta to the value
    the parameter had at the start of the step.

    Two schedules compute the same per-parameter deltas:
      * fused (default): step() runs the wrapped optimizer once on all
        parameters, forms all deltas with multi-tensor ops and reduces them
        in one grouped Adasum allreduce (few large fused kernels);
      * per parameter (HOROVOD_ADASUM_PER_PARAMETER=1, the reference's
        schedule): when a gradient is ready the wrapped optimizer steps that
        one parameter alone and its delta is reduced asynchronously, which
        overlaps with backward but costs one optimizer step() call and one
        negotiation per parameter.

    Parity: horovod/torch/optimizer.py:335-503.
    """
    _instances = 0

    def __init__(self, params, named_parameters, compression, backward_passes_per_step=1,
                 process_set=global_process_set):
        super(self.__class__, self).__init__(params)
        self._compression = compression
        if named_parameters is not None:
            named_parameters = list(named_parameters)
        else:
            named_parameters = [("allreduce.noname.%s.%s" % (gi, pi), v)
                                for gi, group in enumerate(self.param_groups)
                                for pi, v in enumerate(group["params"])]
        dups = _find_duplicates([k for k, _ in named_parameters])
        if dups:
            raise ValueError("Parameter names in named_parameters must be unique. "
                             "Found duplicates: %s" % ", ".join(dups))
        self._parameter_names = {v: k for k, v in sorted(named_parameters)}
        self.backward_passes_per_step = backward_passes_per_step
        self._allreduce_delay = {v: self.backward_passes_per_step
                                 for _, v in sorted(named_parameters)}
        self.process_set = process_set
        self._handles = {}
        self._requires_update = set()
        self._synchronized = False
        self._should_synchronize = True
        self._starting_models = {
            p: torch.zeros_like(p, requires_grad=False)
            for _, p in named_parameters
        }
        self._hook_handles = []
        import os
        self._fused = os.environ.get("HOROVOD_ADASUM_PER_PARAMETER", "0") != "1"
        cls = self.__class__
        self._group_name = "DistributedAdasumOptimizer.%d" % cls._instances
        cls._instances += 1
        if self.process_set.included() and (size() > 1 or _force_hooks()):
            for group in self.param_groups:
                for p in group["params"]:
                    if p.requires_grad:
                        self._requires_update.add(p)
                        self._hook_handles.append(
                            p.register_post_accumulate_grad_hook(self._make_hook(p)))

    def set_backward_passes_per_step(self, passes):
        self.backward_passes_per_step = passes
        for p in self._allreduce_delay:
            self._allreduce_delay[p] = self.backward_passes_per_step

    def _fused_step(self):
        """One local optimizer step on everything, all deltas at once."""
        params = [p for group in self.param_groups for p in group["params"]
                  if p in self._requires_update]
        for p in params:
            if p.grad is None:
                p.grad = p.data.new_zeros(p.size())
        datas = [p.data for p in params]
        starts = [self._starting_models[p].data for p in params]
        torch._foreach_copy_(starts, datas)
        super(self.__class__, self).step()
        torch._foreach_sub_(datas, starts)  # every parameter now holds its local delta
        by_kind = {}
        for i, d in enumerate(datas):
            by_kind.setdefault((d.dtype, d.device), []).append(i)
        pending = []
        for k, (kind, idx) in enumerate(sorted(by_kind.items(), key=lambda kv: str(kv[0]))):
            comp = [self._compression.compress(datas[i]) for i in idx]
            handle = grouped_allreduce_async_([c[0] for c in comp],
                                              name="%s.%d" % (self._group_name, k), op=Adasum,
                                              process_set=self.process_set)
            pending.append((idx, comp, handle))
        for idx, comp, handle in pending:
            outs = synchronize(handle)
            for i, (tensor_compressed, cctx), out in zip(idx, comp, outs):
                delta = self._compression.decompress(out, cctx)
                if delta.data_ptr() != datas[i].data_ptr():
                    datas[i].copy_(delta)
        torch._foreach_add_(starts, datas)
        torch._foreach_copy_(datas, starts)
        for p in params:
            self._allreduce_delay[p] = self.backward_passes_per_step
        self._handles.clear()

    def _allreduce_grad_async(self, p):
        # Run the wrapped optimizer on this parameter alone to get its delta.
        name = self._parameter_names.get(p)
        start = self._starting_models[p]
        stashed = []
        for group in self.param_groups:
            stashed.append(group["params"])
            group["params"] = [q for q in group["params"] if q is p]
        start.data.copy_(p.data)
        super(self.__class__, self).step()
        for group, params in zip(self.param_groups, stashed):
            group["params"] = params
        p.data.sub_(start)  # p now holds the local delta
        tensor_compressed, ctx = self._compression.compress(p.data)
        handle = allreduce_async_(tensor_compressed, name=name, op=Adasum,
                                  process_set=self.process_set)
        return handle, (tensor_compressed, ctx)

    def _make_hook(self, p):
        def hook(*ignore):
            if p in self._handles and self._handles[p][0] is not None:
                if self._allreduce_delay[p] <= 0:
                    raise AssertionError(
                        "Gradients were computed more than backward_passes_per_step "
                        "times before call to step(). Increase "
                        "backward_passes_per_step to accumulate gradients locally.")
            assert not p.grad.requires_grad
            handle, ctx = None, None
            self._allreduce_delay[p] -= 1
            if self._allreduce_delay[p] == 0 and not self._fused:
                handle, ctx = self._allreduce_grad_async(p)
            self._handles[p] = (handle, ctx)
        return hook

    def synchronize(self):
        pass

    @contextmanager
    def skip_synchronize(self):
        raise AssertionError("Skipping synchronization is not supported when using "
                             "Adasum optimizer.")
        yield  # pragma: no cover

    def step(self, closure=None):
        loss = None
        if closure is not None:
            loss = closure()
        if not self.process_set.included():
            return super(self.__class__, self).step()
        if self._fused:
            self._fused_step()
            return loss
        missing = self._requires_update - set(self._handles.keys())
        for p in missing:
            if p.grad is None:
                p.grad = p.data.new_zeros(p.size())
            self._handles[p] = self._allreduce_grad_async(p)
        for p, (handle, ctx) in list(self._handles.items()):
            if handle is None:
                self._handles[p] = self._allreduce_grad_async(p)
        for p, (handle, ctx) in self._handles.items():
            output = synchronize(handle)
            tensor_compressed, cctx = ctx
            delta = self._compression.decompress(
                output if output is not None else tensor_compressed, cctx)
            start = self._starting_models[p]
            start.data.add_(delta.data)
            p.data.copy_(start)
            self._allreduce_delay[p] = self.backward_passes_per_step
        self._handles.clear()
        return loss

    def zero_grad(self, *args, **kwargs):
        if self._handles:
            raise AssertionError(
                "optimizer.zero_grad() was called after loss.backward() but before "
                "optimizer.step() or optimizer.synchronize(). This is prohibited as it "
                "can cause a race condition.")
        return super(self.__class__, self).zero_grad(*args, **kwargs)


def DistributedOptimizer(optimizer, named_parameters=None, compression=Compression.none,
                         backward_passes_per_step=1, op=Average,
                         gradient_predivide_factor=1.0, num_groups=0, groups=None,
                         sparse_as_dense=False, process_set=global_process_set,
                         symmetric_gradients=None):
    """Returns an optimizer of the same class as ``optimizer`` whose step()
    first combines gradients across the ranks of ``process_set``.

    Arguments:
        optimizer: the torch optimizer to wrap.
        named_parameters: ``model.named_parameters()``; names identify
            gradients across ranks.
        compression: ``hvd.Compression.none|fp16|bf16`` wire format.
        backward_passes_per_step: local backward passes accumulated before a
            reduction.
        op: ``hvd.Average`` (default), ``hvd.Sum`` or ``hvd.Adasum``.
        gradient_predivide_factor: with Average, gradients are scaled by
            1/factor before and factor/size after the sum.
        num_groups / groups: fuse gradients into explicit groups (an int for
            that many equal groups, or a list of lists of parameters).
        sparse_as_dense: densify sparse gradients before reduction.
        symmetric_gradients: keep gradients in the symmetric heap (one flat
            buffer, ``p.grad`` are views) so that their allreduce runs in
            place over NVLink without staging copies. Default: the value of
            HOROVOD_SYMMETRIC_GRADIENTS (off). Not available in elastic jobs
            (the heap does not survive a reset) or with Adasum.
    """
    import os
    if symmetric_gradients is None:
        symmetric_gradients = os.environ.get("HOROVOD_SYMMETRIC_GRADIENTS", "0") == "1"
    if os.environ.get("HOROVOD_ELASTIC") == "1" or not torch.cuda.is_available():
        symmetric_gradients = False
    if gradient_predivide_factor != 1.0 and op != Average:
        raise ValueError("gradient_predivide_factor not supported with op != Average")
    if num_groups != 0:
        warnings.warn("Parameter `num_groups` has been replaced by `groups` "
                      "and will be removed", DeprecationWarning)
        if groups is None:
            groups = num_groups
    if op != Adasum or size() == 1:
        cls = type(optimizer.__class__.__name__, (optimizer.__class__,),
                   dict(_DistributedOptimizer.__dict__))
        return cls(optimizer.param_groups, named_parameters, compression,
                   backward_passes_per_step, op, gradient_predivide_factor, groups,
                   sparse_as_dense, process_set,
                   symmetric_gradients and size() > 1 and op != Adasum)
    if groups is not None:
        raise ValueError("groups are not supported with op == Adasum")
    cls = type(optimizer.__class__.__name__, (optimizer.__class__,),
               dict(_DistributedAdasumOptimizer.__dict__))
    return cls(optimizer.param_groups, named_parameters, compression,
               backward_passes_per_step, process_set)
