"""Runs a shell command so that nothing it starts can outlive the launcher.

The command runs in its own session (process group). Its stdout/stderr are
forwarded line by line, optionally prefixed with ``[index]<stdout>:`` and a
timestamp. The whole group is terminated (SIGTERM, then SIGKILL after a grace
period) when one of the given events fires or when the launcher itself dies.

Parity: horovod/runner/common/util/safe_shell_exec.py:33-270. The reference
forks a "middleman" process to watch its parent; here a watcher thread in the
launcher plus PR_SET_PDEATHSIG in the child cover the same two cases.
"""
import ctypes
import datetime
import os
import signal
import subprocess
import sys
import threading
import time

GRACEFUL_TERMINATION_TIME_S = 5


def _set_pdeathsig():
    # New session so that killpg reaches every descendant; die with the parent.
    os.setsid()
    try:
        libc = ctypes.CDLL("libc.so.6", use_errno=True)
        libc.prctl(1, signal.SIGTERM)  # PR_SET_PDEATHSIG
    except OSError:
        pass


def terminate_process_group(pid, grace=GRACEFUL_TERMINATION_TIME_S):
    """SIGTERM to the group led by ``pid``; SIGKILL if it is still there after
    ``grace`` seconds."""
    try:
        os.killpg(pid, signal.SIGTERM)
    except (ProcessLookupError, PermissionError):
        return
    deadline = time.time() + grace
    while time.time() < deadline:
        try:
            os.killpg(pid, 0)
        except (ProcessLookupError, PermissionError):
            return
        time.sleep(0.1)
    try:
        os.killpg(pid, signal.SIGKILL)
    except (ProcessLookupError, PermissionError):
        pass


def prefix_stream(src, dst, prefix, index, prefix_timestamp):
    """Copies lines from ``src`` to ``dst`` adding ``[index]<prefix>:``."""
    for raw in iter(src.readline, b""):
        line = raw.decode("utf-8", errors="replace")
        head = ""
        if prefix_timestamp:
            head += datetime.datetime.now().strftime("%a %b %d %H:%M:%S %Y")
        if index is not None and prefix is not None:
            head += "[%s]<%s>:" % (index, prefix)
        try:
            dst.write(head + line if head else line)
            dst.flush()
        except ValueError:  # destination closed
            break
    src.close()


def execute(command, env=None, stdout=None, stderr=None, index=None, events=None,
            prefix_output_with_timestamp=False):
    """Runs ``command`` through the shell and returns its exit code. ``events``
    is a list of threading.Event; when any is set the process tree is killed."""
    stdout = stdout if stdout is not None else sys.stdout
    stderr = stderr if stderr is not None else sys.stderr
    proc = subprocess.Popen(command, shell=True, env=env, stdout=subprocess.PIPE,
                            stderr=subprocess.PIPE, preexec_fn=_set_pdeathsig,
                            executable="/bin/bash")
    pumps = [
        threading.Thread(target=prefix_stream, daemon=True,
                         args=(proc.stdout, stdout, "stdout", index,
                               prefix_output_with_timestamp)),
        threading.Thread(target=prefix_stream, daemon=True,
                         args=(proc.stderr, stderr, "stderr", index,
                               prefix_output_with_timestamp)),
    ]
    for t in pumps:
        t.start()

    stop_watch = threading.Event()

    def watch():
        while not stop_watch.is_set():
            if any(e.is_set() for e in (events or [])):
                terminate_process_group(proc.pid)
                return
            stop_watch.wait(0.1)

    watcher = threading.Thread(target=watch, daemon=True)
    watcher.start()
    try:
        code = proc.wait()
    except BaseException:
        terminate_process_group(proc.pid)
        raise
    finally:
        stop_watch.set()
    watcher.join()
    for t in pumps:
        t.join(timeout=2)
    # Stragglers the command left behind in its group.
    terminate_process_group(proc.pid, grace=1)
    return code if code >= 0 else 128 - code
