"""Broadcast of model parameters, optimizer state and arbitrary objects, and
allgather of objects.

Parity: horovod/torch/functions.py:29-266.
"""
import collections
import io

import cloudpickle
import torch

from horovod_b200.common.process_sets import global_process_set
from horovod_b200.torch.mpi_ops import (allgather, broadcast_, broadcast_async_, rank,
                                        size, synchronize)


def broadcast_parameters(params, root_rank, process_set=global_process_set):
    """Overwrites ``params`` on every rank with the values held by
    ``root_rank``. Accepts ``model.state_dict()``, ``model.named_parameters()``
    or a list of (name, tensor) pairs. All broadcasts are launched before any
    is waited for, so the runtime can batch them into few launches."""
    if isinstance(params, dict):
        params = sorted(params.items())
    elif isinstance(params, list):
        params = [p if isinstance(p, tuple) else (None, p) for p in params]
    else:
        params = list(params)
        if params and not isinstance(params[0], tuple):
            raise ValueError("invalid params of type: %s" % type(params))
    handles = []
    for name, p in params:
        if p is None or not isinstance(p, torch.Tensor):
            continue
        handles.append(broadcast_async_(p.data if p.requires_grad else p, root_rank,
                                        name="broadcast.%s" % name if name else None,
                                        process_set=process_set))
    for h in handles:
        synchronize(h)


def broadcast_object(obj, root_rank=0, name=None, process_set=global_process_set):
    """Pickles ``obj`` on ``root_rank`` and returns the copy on every rank."""
    if name is None:
        name = type(obj).__name__
    if rank() == root_rank:
        buf = io.BytesIO()
        cloudpickle.dump(obj, buf)
        t = torch.frombuffer(bytearray(buf.getvalue()), dtype=torch.uint8)
        sz = torch.tensor([t.shape[0]], dtype=torch.int64)
        broadcast_(sz, root_rank, name + ".sz", process_set=process_set)
    else:
        sz = torch.zeros(1, dtype=torch.int64)
        broadcast_(sz, root_rank, name + ".sz", process_set=process_set)
        t = torch.empty(int(sz.item()), dtype=torch.uint8)
    broadcast_(t, root_rank, name + ".t", process_set=process_set)
    if rank() != root_rank:
        obj = cloudpickle.load(io.BytesIO(t.numpy().tobytes()))
    return obj


def allgather_object(obj, name=None, process_set=global_process_set):
    """Returns the list of every rank's ``obj`` (ordered by rank)."""
    if name is None:
        name = type(obj).__name__
    buf = io.BytesIO()
    cloudpickle.dump(obj, buf)
    t = torch.frombuffer(bytearray(buf.getvalue()), dtype=torch.uint8)
    sz = torch.tensor([t.shape[0]], dtype=torch.int64)
    sizes = allgather(sz, name=name + ".sz", process_set=process_set)
    gathered = allgather(t, name=name + ".t", process_set=process_set)
    out, pos = [], 0
    raw = gathered.numpy().tobytes()
    for n in sizes.tolist():
        out.append(cloudpickle.load(io.BytesIO(raw[pos:pos + n])))
        pos += n
    return out


def broadcast_optimizer_state(optimizer, root_rank, process_set=global_process_set):
    """Makes the optimizer on every rank identical to the one on
    ``root_rank``: state tensors are broadcast in place, scalars and
    param_group options travel as one pickled object."""
    if isinstance(optimizer, torch.optim.LBFGS):
        raise ValueError("cannot broadcast torch.optim.LBFGS state")
    state_dict = optimizer.state_dict()

    # Ranks that have not stepped yet have no state: create it with a step on
    # zero gradients, using the plain optimizer class so that no allreduce
    # is triggered, then put the parameters back.
    if len(state_dict["state"]) == 0:
        saved = []
        for group in optimizer.param_groups:
            for p in group["params"]:
                saved.append((p, p.data.clone(), p.grad))
                if p.requires_grad and p.grad is None:
                    p.grad = p.data.new_zeros(p.size())
        base = getattr(optimizer, "_hvd_base_step", None)
        if base is not None:
            base()
        else:
            optimizer.step()
        for p, data, grad in saved:
            p.data.copy_(data)
            p.grad = grad
        state_dict = optimizer.state_dict()
    if len(state_dict["state"]) == 0:
        # Stateless optimizer (plain SGD): only options need to agree.
        pass

    tensors = {}
    scalars = collections.OrderedDict()
    for gi, group in enumerate(state_dict["param_groups"]):
        for key, value in group.items():
            if key == "params":
                continue
            scalars["group.%d.%s" % (gi, key)] = value
    for pid, pstate in sorted(state_dict["state"].items(), key=lambda kv: str(kv[0])):
        for key, value in sorted(pstate.items()):
            full = "state.%s.%s" % (pid, key)
            if isinstance(value, torch.Tensor):
                tensors[full] = value
            else:
                scalars[full] = value

    broadcast_parameters(tensors, root_rank, process_set=process_set)
    scalars = broadcast_object(scalars, root_rank, name="optimizer.scalars",
                               process_set=process_set)
    for full, value in scalars.items():
        kind, idx, key = full.split(".", 2)
        if kind == "group":
            state_dict["param_groups"][int(idx)][key] = value
        else:
            pid = int(idx) if idx.lstrip("-").isdigit() else idx
            state_dict["state"][pid][key] = value
    optimizer.load_state_dict(state_dict)
