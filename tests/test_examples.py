"""The examples run under the launcher as smoke tests, as the reference's CI
does (.buildkite/gen-pipeline.sh:173-225): 2 CPU ranks on this machine."""
import os
import re
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _launch(np, script_args, timeout=300):
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""),
               CUDA_VISIBLE_DEVICES="")
    cmd = [sys.executable, "-m", "horovod_b200.runner.launch", "-np", str(np),
           sys.executable] + script_args
    proc = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=timeout)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-2000:]
    return proc.stdout


def test_mnist_example_trains(tmp_path):
    ckpt = str(tmp_path / "mnist.pt")
    out = _launch(2, ["examples/pytorch_mnist.py", "--epochs", "2", "--batch-size", "128",
                      "--checkpoint", ckpt])
    accs = [float(a) for a in re.findall(r"acc(?:uracy)?[ =:]+([0-9.]+)", out)]
    losses = [float(a) for a in re.findall(r"loss[ =:]+([0-9.]+)", out)]
    assert len(accs) == 2 and len(losses) == 2, out[-1500:]
    assert losses[1] < losses[0] and accs[1] > accs[0], out[-1500:]
    assert os.path.exists(ckpt)


def test_synthetic_benchmark_example():
    out = _launch(2, ["examples/pytorch_synthetic_benchmark.py", "--no-cuda", "--batch-size", "1",
                      "--num-warmup-batches", "1", "--num-batches-per-iter", "1",
                      "--num-iters", "1"])
    assert "Total img/sec on 2 rank(s)" in out
