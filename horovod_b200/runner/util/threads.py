"""Thread helpers for the launcher.

Parity: horovod/runner/util/threads.py.
"""
import queue
import threading


def execute_function_multithreaded(fn, args_list, block_until_all_done=True, max_concurrent=0):
    """Calls ``fn(*args)`` for every args tuple on its own thread. Returns
    {index: result} (when blocking). An exception in a thread is re-raised in
    the caller."""
    results, errors = {}, queue.Queue()
    sem = threading.Semaphore(max_concurrent) if max_concurrent else None

    def run(i, args):
        try:
            if sem:
                sem.acquire()
            results[i] = fn(*args)
        except BaseException as e:  # noqa: BLE001 - forwarded to the caller
            errors.put(e)
        finally:
            if sem:
                sem.release()

    threads = [threading.Thread(target=run, args=(i, a), daemon=True)
               for i, a in enumerate(args_list)]
    for t in threads:
        t.start()
    if block_until_all_done:
        for t in threads:
            t.join()
        if not errors.empty():
            raise errors.get()
        return results
    return threads


def in_thread(target, args=(), name=None, daemon=True):
    t = threading.Thread(target=target, args=args, name=name, daemon=daemon)
    t.start()
    return t


def on_event(event, func, args=(), stop=None, check_interval_seconds=0.2):
    """Runs ``func(*args)`` once ``event`` is set, unless ``stop`` is set first."""
    def wait():
        while not event.is_set():
            if stop is not None and stop.is_set():
                return
            event.wait(check_interval_seconds)
        func(*args)
    return in_thread(wait)
