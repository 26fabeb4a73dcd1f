"""What a training function can ask about the Spark task it runs in.

``get_available_devices()`` returns the GPU addresses Spark's resource
scheduling gave this task (``spark.task.resource.gpu.amount``), as strings,
or an empty list when the task has none; a training function picks its
device from it instead of from its local rank:

    devices = horovod_b200.spark.task.get_available_devices()
    if devices:
        torch.cuda.set_device(int(devices[0]))

Parity: horovod/spark/task/task_info.py:25-32 (get_available_devices,
set_resources).
"""

_resources = {}


def set_resources(resources):
    """Called by the task wrapper of ``spark.run`` / ``run_elastic`` with
    ``TaskContext.resources()`` before the training function starts."""
    global _resources
    _resources = dict(resources or {})


def get_available_devices():
    gpu = _resources.get("gpu")
    if gpu is None:
        return []
    return [str(a) for a in getattr(gpu, "addresses", gpu)]


def resources_of(context):
    """``context.resources()`` where the Spark version has it, else {}."""
    try:
        return dict(context.resources() or {})
    except Exception:  # noqa: BLE001 - Spark < 3.0, or no resource scheduling
        return {}
