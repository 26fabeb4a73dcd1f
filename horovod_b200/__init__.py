"""horovod_b200: a Blackwell-native data-parallel training library with
Horovod's public API. ``import horovod_b200.torch as hvd`` is the entry point;
``horovod_b200.run`` launches a function on several ranks programmatically.
"""
__version__ = "0.1.0"


def run(*args, **kwargs):
    """Programmatic launcher (see horovod_b200.runner.run)."""
    from horovod_b200.runner import run as _run
    return _run(*args, **kwargs)
