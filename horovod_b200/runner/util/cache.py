"""Small on-disk cache of launcher checks (e.g. "ssh to host X works") that
expires after a staleness threshold and is invalidated when the launch
parameters change.

Parity: horovod/runner/util/cache.py:23-129.
"""
import datetime
import os
import pickle
import threading


class Cache:
    def __init__(self, cache_folder, cache_staleness_threshold_in_minutes, parameters_hash):
        self._file = os.path.join(cache_folder, "cache.bin")
        self._threshold = datetime.timedelta(minutes=cache_staleness_threshold_in_minutes)
        self._lock = threading.Lock()
        self._content = {}
        try:
            os.makedirs(cache_folder, exist_ok=True)
            if os.path.isfile(self._file):
                with open(self._file, "rb") as f:
                    content = pickle.load(f)
                if content.get("parameters_hash") == parameters_hash:
                    self._content = content
        except Exception:
            self._content = {}
        self._content["parameters_hash"] = parameters_hash

    def get(self, key):
        with self._lock:
            item = self._content.get(key)
            if item is None:
                return None
            timestamp, value = item
            if datetime.datetime.now() - timestamp > self._threshold:
                return None
            return value

    def put(self, key, value):
        with self._lock:
            self._content[key] = (datetime.datetime.now(), value)
            try:
                with open(self._file, "wb") as f:
                    pickle.dump(self._content, f)
            except OSError:
                pass


def use_cache():
    """Decorator: caches the wrapped function's result in ``fn_cache=``."""
    def wrap(func):
        def wrapped(*args, **kwargs):
            fn_cache = kwargs.get("fn_cache")
            if fn_cache is None:
                return func(*args, **kwargs)
            key = (func.__name__, tuple(args), frozenset(
                (k, v) for k, v in kwargs.items() if k != "fn_cache"))
            hit = fn_cache.get(key)
            if hit is not None:
                return hit
            result = func(*args, **kwargs)
            fn_cache.put(key, result)
            return result
        return wrapped
    return wrap
