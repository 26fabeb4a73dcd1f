"""Where an estimator runs its training function: ``Backend.run(fn, args,
kwargs, env)`` runs ``fn`` once per rank of one job and returns the results
ordered by rank; ``num_processes()`` is the number of ranks.

``SparkBackend`` runs the ranks inside Spark tasks (horovod_b200.spark.run);
``LocalBackend`` runs them as processes of the launcher on this machine or on
the given hosts, for estimators that are fitted outside a Spark session.
Parity: horovod/spark/common/backend.py:30-91 (Backend, SparkBackend).
"""


class Backend:
    """Interface of an estimator's execution backend."""

    def run(self, fn, args=(), kwargs=None, env=None):
        raise NotImplementedError()

    def num_processes(self):
        raise NotImplementedError()


class SparkBackend(Backend):
    """One rank per Spark task of a barrier stage. ``num_proc`` defaults to
    ``spark.default.parallelism`` of the active context; ``env`` is added to
    every rank's environment; the other keyword arguments go to
    ``horovod_b200.spark.run`` unchanged."""

    def __init__(self, num_proc=None, env=None, **run_kwargs):
        self._num_proc = num_proc
        self._env = dict(env or {})
        self._run_kwargs = run_kwargs

    def _resolved(self):
        if self._num_proc is None:
            from horovod_b200.spark.runner import _require_pyspark
            context = _require_pyspark().SparkContext._active_spark_context
            if context is None:
                raise Exception("Could not find an active SparkContext, are you running in a "
                                "PySpark session?")
            self._num_proc = context.defaultParallelism
        return self._num_proc

    def run(self, fn, args=(), kwargs=None, env=None):
        from horovod_b200.spark.runner import run
        merged = dict(self._env)
        merged.update(env or {})
        return run(fn, args=args, kwargs=kwargs or {}, num_proc=self._resolved(),
                   extra_env=merged, **self._run_kwargs)

    def num_processes(self):
        return self._resolved()


class LocalBackend(Backend):
    """The ranks are processes started by this package's launcher:
    ``num_proc`` of them on this machine, or spread over ``hosts``
    (``"host1:2,host2:2"``)."""

    def __init__(self, num_proc=1, hosts=None, env=None, **run_kwargs):
        self._num_proc = int(num_proc)
        self._hosts = hosts
        self._env = dict(env or {})
        self._run_kwargs = run_kwargs

    def run(self, fn, args=(), kwargs=None, env=None):
        from horovod_b200.runner import run
        merged = dict(self._env)
        merged.update(env or {})
        return run(fn, args=args, kwargs=kwargs or {}, np=self._num_proc, hosts=self._hosts,
                   env=merged or None, **self._run_kwargs)

    def num_processes(self):
        return self._num_proc
