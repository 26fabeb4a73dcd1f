"""Elastic state for PyTorch: model, optimizer, sampler and plain attributes.

Parity: horovod/torch/elastic/state.py:27-179.
"""
import copy

import torch

from horovod_b200.common.elastic import ObjectState
from horovod_b200.torch.elastic.sampler import ElasticSampler
from horovod_b200.torch.functions import (broadcast_object, broadcast_optimizer_state,
                                          broadcast_parameters)
from horovod_b200.torch.mpi_ops import rank


class StateHandler:
    """Knows how to save/restore/sync one kind of value."""

    def __init__(self, value):
        self.value = value

    def save(self):
        raise NotImplementedError()

    def restore(self):
        raise NotImplementedError()

    def sync(self):
        raise NotImplementedError()

    def set_value(self, value):
        self.value = value
        self.save()


class ModelStateHandler(StateHandler):
    def __init__(self, model):
        super().__init__(model)
        self._saved = copy.deepcopy(model.state_dict())

    def save(self):
        self._saved = copy.deepcopy(self.value.state_dict())

    def restore(self):
        self.value.load_state_dict(self._saved)

    def sync(self):
        broadcast_parameters(self.value.state_dict(), root_rank=0)


class OptimizerStateHandler(StateHandler):
    def __init__(self, optimizer):
        super().__init__(optimizer)
        self._saved = copy.deepcopy(optimizer.state_dict())

    def save(self):
        self._saved = copy.deepcopy(self.value.state_dict())

    def restore(self):
        self.value.load_state_dict(self._saved)

    def sync(self):
        broadcast_optimizer_state(self.value, root_rank=0)


class SamplerStateHandler(StateHandler):
    def __init__(self, sampler):
        super().__init__(sampler)
        self._saved = copy.deepcopy(sampler.state_dict())

    def save(self):
        self._saved = copy.deepcopy(self.value.state_dict())

    def restore(self):
        self.value.load_state_dict(self._saved)

    def sync(self):
        # Union of what every rank processed, then repartition.
        from horovod_b200.torch.functions import allgather_object
        state = self.value.state_dict()
        all_processed = allgather_object(state["processed_indices"],
                                         name="hvd.elastic.sampler")
        merged = set()
        for s in all_processed:
            merged |= set(s)
        state["processed_indices"] = merged
        state = broadcast_object(state, 0, name="hvd.elastic.sampler_state")
        self.value.load_state_dict(state)


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


def _get_handler(v):
    for handler_type, handler_cls in _handler_registry:
        if isinstance(v, handler_type):
            return handler_cls(v)
    return None


def _get_handlers(kwargs):
    handlers, remainder = {}, {}
    for k, v in kwargs.items():
        h = _get_handler(v)
        if h is not None:
            handlers[k] = h
        else:
            remainder[k] = v
    return handlers, remainder


class TorchState(ObjectState):
    """``TorchState(model=..., optimizer=..., sampler=..., epoch=0, batch=0)``.
    Modules, optimizers and ElasticSamplers get dedicated handlers; everything
    else is treated as a picklable attribute."""

    def __init__(self, model=None, optimizer=None, **kwargs):
        kwargs.update(dict(model=model, optimizer=optimizer))
        kwargs = {k: v for k, v in kwargs.items() if v is not None}
        self._handlers, kwargs = _get_handlers(kwargs)
        for name, handler in self._handlers.items():
            setattr(self, name, handler.value)
        super().__init__(bcast_object=broadcast_object, get_rank=rank, **kwargs)

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
        super().sync()

    def __setattr__(self, name, value):
        if hasattr(self, name) and name in getattr(self, "_handlers", {}):
            self._handlers[name].set_value(value)
        super().__setattr__(name, value)
