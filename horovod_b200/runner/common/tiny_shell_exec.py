"""Runs a short command and hands back what it printed.
Parity: horovod/runner/common/util/tiny_shell_exec.py."""
import io
import sys
import traceback

from horovod_b200.runner.common import safe_shell_exec


def execute(command, env=None):
    """(combined stdout and stderr, exit code), or None when the command could
    not be run at all."""
    captured = io.StringIO()
    try:
        code = safe_shell_exec.execute(command, env=env, stdout=captured, stderr=captured)
        return captured.getvalue(), code
    except Exception:  # noqa: BLE001 - reported to the caller as "could not run"
        print(traceback.format_exc(), file=sys.stderr)
        return None
    finally:
        captured.close()
