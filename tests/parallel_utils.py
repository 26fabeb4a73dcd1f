"""Runs a function on several ranks as child processes of the test, wired
together through the launcher's rendezvous server on 127.0.0.1."""
import multiprocessing as mp
import os
import queue
import traceback

from horovod_b200.runner.http.http_server import RendezvousServer


def _plain(obj):
    """Tensors travel back as numpy arrays (no shared-memory handles that die
    with the child)."""
    import torch
    if isinstance(obj, torch.Tensor):
        t = obj.detach().cpu()
        return t.float().numpy() if t.dtype in (torch.bfloat16, torch.float16) else t.numpy()
    if isinstance(obj, (list, tuple)):
        return type(obj)(_plain(o) for o in obj)
    if isinstance(obj, dict):
        return {k: _plain(v) for k, v in obj.items()}
    return obj


def _child(fn, rank, size, port, env, args, q):
    try:
        os.environ.update({
            "HOROVOD_RANK": str(rank), "HOROVOD_SIZE": str(size),
            "HOROVOD_LOCAL_RANK": str(rank), "HOROVOD_LOCAL_SIZE": str(size),
            "HOROVOD_CROSS_RANK": "0", "HOROVOD_CROSS_SIZE": "1",
            "HOROVOD_GLOO_RENDEZVOUS_ADDR": "127.0.0.1",
            "HOROVOD_GLOO_RENDEZVOUS_PORT": str(port),
            "HOROVOD_HOSTNAME": "127.0.0.1",
        })
        os.environ.update(env or {})
        import torch
        torch.set_num_threads(1)
        result = fn(rank, size, *args)
        q.put((rank, "ok", _plain(result)))
    except BaseException:
        q.put((rank, "error", traceback.format_exc()))


def run_parallel(fn, np=2, env=None, args=(), timeout=180):
    """Runs ``fn(rank, size, *args)`` on ``np`` ranks; returns the list of
    results ordered by rank. Any rank's exception fails the test."""
    server = RendezvousServer()
    port = server.start()
    server.init([None] * np)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_child, args=(fn, r, np, port, env, args, q))
             for r in range(np)]
    for p in procs:
        p.start()
    results, errors = {}, []
    try:
        for _ in range(np):
            try:
                rank, status, payload = q.get(timeout=timeout)
            except queue.Empty:
                errors.append("timed out waiting for ranks %s"
                              % sorted(set(range(np)) - set(results)))
                break
            if status == "ok":
                results[rank] = payload
            else:
                errors.append("rank %d failed:\n%s" % (rank, payload))
                results[rank] = None
    finally:
        for p in procs:
            p.join(timeout=10 if not errors else 2)
            if p.is_alive():
                p.kill()
        server.stop()
    if errors:
        raise AssertionError("\n".join(errors))
    return [results[r] for r in range(np)]
