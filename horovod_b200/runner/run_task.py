"""Worker side of ``horovod_b200.run``: fetches the pickled function from the
launcher's key-value server, runs it and stores the result under this rank.

Parity: horovod/runner/run_task.py:22, task_fn.py:23.
"""
import os
import sys
import traceback
import urllib.request

import cloudpickle


def main(addr, port):
    base = "http://%s:%s" % (addr, port)
    with urllib.request.urlopen(base + "/runfunc/func", timeout=60) as r:
        func, args, kwargs = cloudpickle.loads(r.read())
    rank = int(os.environ.get("HOROVOD_RANK", "0"))
    try:
        result = (True, func(*args, **kwargs), None)
    except SystemExit as e:
        if e.code in (0, None):
            # e.g. an elastic worker whose host left the job: it has no rank
            # any more and nothing to report
            return 0
        result = (False, traceback.format_exc(), None)
    except BaseException:
        result = (False, traceback.format_exc(), None)
    # Rank and world size can change in elastic jobs (every re-initialisation
    # rewrites the environment): report under the final ones.
    rank = int(os.environ.get("HOROVOD_RANK", rank))
    size = int(os.environ.get("HOROVOD_SIZE", "1"))
    try:
        import horovod_b200.torch as hvd
        if hvd.is_initialized():
            rank, size = hvd.rank(), hvd.size()
    except Exception:
        pass
    blob = cloudpickle.dumps((result[0], result[1], size))
    req = urllib.request.Request("%s/runfunc_result/%d" % (base, rank), data=blob, method="PUT")
    with urllib.request.urlopen(req, timeout=60):
        pass
    return 0 if result[0] else 1


if __name__ == "__main__":
    sys.exit(main(sys.argv[1], sys.argv[2]))
