"""Elastic state for PyTorch.

``TorchState(model=..., optimizer=..., sampler=..., epoch=0, batch=0)`` keeps
an in-memory checkpoint of everything a training loop needs to continue after
the set of workers changed: ``commit()`` snapshots it, ``restore()`` rolls
back to the last snapshot, ``sync()`` makes every rank adopt rank 0's values.
How a value is snapshotted and synchronised depends on its type: modules,
optimizers and ElasticSamplers go through their ``state_dict``; anything else
is a plain picklable attribute handled by ``ObjectState``.

Behaviour follows horovod/torch/elastic/state.py:27-179; the type-to-handler
registry (``get_handler_registry`` / ``set_handler_registry``) is kept so that
users can add their own kinds of state.
"""
import torch

from horovod_b200.common.elastic import ObjectState
from horovod_b200.torch.elastic.sampler import ElasticSampler
from horovod_b200.torch.functions import (allgather_object, broadcast_object,
                                          broadcast_optimizer_state, broadcast_parameters)
from horovod_b200.torch.mpi_ops import rank


def _snapshot(obj):
    """A private copy of a (nested) state_dict: tensors are cloned where they
    live, containers are rebuilt, everything else is kept as it is (numbers,
    strings, None are immutable)."""
    if isinstance(obj, torch.Tensor):
        return obj.detach().clone()
    if isinstance(obj, dict):
        return type(obj)((k, _snapshot(v)) for k, v in obj.items())
    if isinstance(obj, (list, tuple, set, frozenset)):
        return type(obj)(_snapshot(v) for v in obj)
    return obj


class StateHandler:
    """Knows how to save, restore and synchronise one kind of value."""

    def __init__(self, value):
        self.value = value

    def save(self):
        raise NotImplementedError()

    def restore(self):
        raise NotImplementedError()

    def sync(self):
        raise NotImplementedError()

    def set_value(self, value):
        """The attribute was re-assigned: track the new object from now on."""
        self.value = value
        self.save()


class _StateDictHandler(StateHandler):
    """For anything with ``state_dict()`` / ``load_state_dict()``: the
    checkpoint is a private copy of the state_dict."""

    def __init__(self, value):
        super().__init__(value)
        self._checkpoint = None
        self.save()

    def save(self):
        self._checkpoint = _snapshot(self.value.state_dict())

    def restore(self):
        # load_state_dict may keep references to what it is given (optimizers
        # do), so hand out a copy and keep the checkpoint pristine.
        self.value.load_state_dict(_snapshot(self._checkpoint))


class ModelStateHandler(_StateDictHandler):
    def sync(self):
        broadcast_parameters(self.value.state_dict(), root_rank=0)


class OptimizerStateHandler(_StateDictHandler):
    def sync(self):
        broadcast_optimizer_state(self.value, root_rank=0)


class SamplerStateHandler(_StateDictHandler):
    def sync(self):
        # What any rank has processed is processed for everybody; then all
        # ranks take rank 0's view and repartition the rest.
        mine = self.value.state_dict()
        done = set()
        for part in allgather_object(mine["processed_indices"], name="hvd.elastic.sampler"):
            done.update(part)
        mine["processed_indices"] = done
        self.value.load_state_dict(
            broadcast_object(mine, 0, name="hvd.elastic.sampler_state"))


_handler_registry = [
    (torch.nn.Module, ModelStateHandler),
    (torch.optim.Optimizer, OptimizerStateHandler),
    (ElasticSampler, SamplerStateHandler),
]


def get_handler_registry():
    return _handler_registry


def set_handler_registry(registry):
    global _handler_registry
    _handler_registry = registry


def _handler_for(value):
    for kind, factory in _handler_registry:
        if isinstance(value, kind):
            return factory(value)
    return None


class TorchState(ObjectState):
    def __init__(self, model=None, optimizer=None, **kwargs):
        # Only the two named arguments are optional; a user attribute that
        # happens to be None stays an attribute.
        named = {k: v for k, v in (("model", model), ("optimizer", optimizer)) if v is not None}
        self._handlers = {}
        plain = {}
        for name, value in {**kwargs, **named}.items():
            handler = _handler_for(value)
            if handler is None:
                plain[name] = value
            else:
                self._handlers[name] = handler
                object.__setattr__(self, name, value)
        super().__init__(bcast_object=broadcast_object, get_rank=rank, **plain)

    def save(self):
        for handler in self._handlers.values():
            handler.save()
        super().save()

    def restore(self):
        for handler in self._handlers.values():
            handler.restore()
        super().restore()

    def sync(self):
        for handler in self._handlers.values():
            handler.sync()
            # what rank 0 sent is the new rollback point, on a worker that has
            # just joined as much as on the others
            handler.save()
        super().sync()

    def __setattr__(self, name, value):
        handlers = self.__dict__.get("_handlers")
        if handlers and name in handlers:
            handlers[name].set_value(value)
        super().__setattr__(name, value)
