"""Framework-independent half of elastic training: the State object that can
be committed / restored / synced, and the retry loop around the user's
training function.

Parity: horovod/common/elastic.py:26-175.
"""
import functools
import queue

from horovod_b200.common.exceptions import (HorovodInternalError, HostsUpdatedInterrupt,
                                             WorkerRemovedError)


class HostUpdateResult:
    no_update = 0
    removed = 1
    added = 2
    mixed = 3


class _NotificationManager:
    """Fan-out of host-change messages from the elastic driver to the State
    objects of this process. The worker-side notification service (started by
    the launcher glue) calls handle_hosts_updated()."""

    def __init__(self):
        self._listeners = set()
        self._service = None

    def init(self):
        if self._service is not None:
            return
        try:
            from horovod_b200.runner.elastic.worker import start_notification_service
            self._service = start_notification_service(self)
        except Exception:
            self._service = None

    def register_listener(self, listener):
        self._listeners.add(listener)

    def remove_listener(self, listener):
        self._listeners.discard(listener)

    def handle_hosts_updated(self, timestamp, update_res):
        for listener in list(self._listeners):
            listener.on_hosts_updated(timestamp, update_res)


notification_manager = _NotificationManager()


class State:
    """State that must survive a change of membership.

    ``commit()`` saves a copy and checks for host changes; ``restore()`` goes
    back to the last commit after a failure; ``sync()`` makes every rank equal
    to rank 0 after a reset.
    """

    def __init__(self, bcast_object, get_rank):
        self._bcast_object = bcast_object
        self._rank = get_rank
        self._host_messages = queue.Queue()
        self._last_updated_timestamp = 0
        self._reset_callbacks = []

    def register_reset_callbacks(self, callbacks):
        """Functions called after every reset, e.g. to rescale the learning
        rate to the new world size."""
        self._reset_callbacks.extend(callbacks)

    def on_reset(self):
        self._host_messages = queue.Queue()
        self.reset()
        for cb in self._reset_callbacks:
            cb()

    def on_hosts_updated(self, timestamp, update_res):
        self._host_messages.put((timestamp, update_res))

    def commit(self):
        self.save()
        self.check_host_updates()

    def check_host_updates(self):
        """Raises HostsUpdatedInterrupt on all ranks at the same commit if the
        driver has reported a host change since the last check. Rank 0's view
        is the one that counts (the driver notifies rank 0 only): it is
        broadcast, so no rank runs ahead of the others."""
        seen_before = self._last_updated_timestamp
        newest, combined = seen_before, HostUpdateResult.no_update
        try:
            while True:
                stamp, change = self._host_messages.get_nowait()
                if stamp > seen_before:
                    newest = max(newest, stamp)
                    combined |= change
        except queue.Empty:
            pass
        seen_before, newest, combined = self._bcast_object(
            (seen_before, newest, combined), name="hvd.elastic.host_updates")
        self._last_updated_timestamp = newest
        if newest > seen_before:
            # Only removals: the survivors are already in sync with each other.
            raise HostsUpdatedInterrupt(skip_sync=combined == HostUpdateResult.removed)

    def save(self):
        raise NotImplementedError()

    def restore(self):
        raise NotImplementedError()

    def sync(self):
        raise NotImplementedError()

    def reset(self):
        pass


class ObjectState(State):
    """State made of plain picklable attributes given as keyword arguments:
    ``ObjectState(..., epoch=0, batch=0)`` has ``.epoch`` and ``.batch``."""

    def __init__(self, bcast_object, get_rank, **kwargs):
        self._committed = dict(kwargs)
        self._apply_committed()
        super().__init__(bcast_object=bcast_object, get_rank=get_rank)

    def save(self):
        self._committed = {name: getattr(self, name) for name in self._committed}

    def _apply_committed(self):
        for name, value in self._committed.items():
            setattr(self, name, value)

    def restore(self):
        self._apply_committed()

    def sync(self):
        if not self._committed:
            return
        self._committed = self._bcast_object(self._committed, name="hvd.elastic.object_state")
        # Only the attributes: restore() of a subclass would also roll back
        # what the subclass has just synchronised by other means.
        self._apply_committed()


def run_fn(func, reset):
    """Wraps ``func(state, ...)`` in the elastic retry loop."""

    @functools.wraps(func)
    def wrapper(state, *args, **kwargs):
        # listener first: the driver may answer the registration with a host
        # change that it could not deliver earlier
        notification_manager.register_listener(state)
        notification_manager.init()
        skip_sync = False
        try:
            while True:
                if not skip_sync:
                    state.sync()
                try:
                    return func(state, *args, **kwargs)
                except HorovodInternalError:
                    state.restore()
                    skip_sync = False
                except HostsUpdatedInterrupt as e:
                    skip_sync = e.skip_sync
                try:
                    reset()
                except WorkerRemovedError as e:
                    # Nothing is left for this process to do; its exit is not
                    # part of the job's outcome.
                    import sys
                    print(str(e), file=sys.stderr, flush=True)
                    raise SystemExit(0)
                state.on_reset()
        finally:
            notification_manager.remove_listener(state)

    return wrapper
