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


def test_imagenet_style_example_trains_checkpoints_and_resumes(tmp_path):
    fmt = str(tmp_path / "ckpt-{epoch}.pt")
    common = ["examples/pytorch_imagenet_resnet50.py", "--no-cuda", "--model", "tiny",
              "--image-size", "32", "--num-classes", "10", "--synthetic-samples", "64",
              "--batch-size", "8", "--batches-per-allreduce", "2", "--warmup-epochs", "1",
              "--checkpoint-format", fmt]
    out = _launch(2, common + ["--epochs", "2"], timeout=600)
    assert len(re.findall(r"epoch \d+ train loss", out)) == 2, out[-1500:]
    assert len(re.findall(r"epoch \d+ val loss", out)) == 2
    assert os.path.exists(fmt.format(epoch=2))
    # a second run with more epochs starts from the newest checkpoint
    out = _launch(2, common + ["--epochs", "3"], timeout=600)
    assert re.findall(r"epoch (\d+) train loss", out) == ["3"], out[-1500:]


def test_adasum_example_runs_both_reductions():
    out = _launch(2, ["examples/pytorch_adasum.py", "--no-cuda", "--steps", "30"])
    rows = dict(re.findall(r"(average|adasum) \(.*?\)\s+first loss ([0-9.]+) last loss [0-9.]+", out))
    assert set(rows) == {"average", "adasum"}, out[-1500:]
    last = {k: float(v) for k, v in re.findall(r"(average|adasum) .*? last loss ([0-9.]+)", out)}
    first = {k: float(v) for k, v in rows.items()}
    assert all(last[k] < first[k] for k in last), out[-1500:]


def test_elastic_synthetic_benchmark_example():
    out = _launch(2, ["examples/pytorch_synthetic_benchmark_elastic.py", "--no-cuda", "--model",
                      "tiny", "--image-size", "32", "--batch-size", "2", "--num-warmup-batches",
                      "1", "--num-batches-per-iter", "1", "--num-iters", "2"])
    assert len(re.findall(r"Iter #\d+: [0-9.]+ img/sec per rank, 2 rank\(s\)", out)) == 2, out[-1500:]
    assert "Total img/sec over 2 iteration(s)" in out


def test_ray_and_spark_examples_are_importable_without_their_frameworks():
    """Their bodies need ray / pyspark; importing them (what a user's editor
    and the launcher do first) must not."""
    import importlib.util
    for name in ("ray_basic", "spark_basic"):
        spec = importlib.util.spec_from_file_location(name, os.path.join(ROOT, "examples",
                                                                         name + ".py"))
        module = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(module)
        assert callable(module.train)


def test_estimator_example_on_pandas(tmp_path):
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""),
               CUDA_VISIBLE_DEVICES="")
    proc = subprocess.run([sys.executable, "examples/spark_torch_estimator.py", "--num-proc", "2",
                           "--rows", "512", "--epochs", "3", "--no-cuda", "--work-dir",
                           str(tmp_path)], cwd=ROOT, env=env, capture_output=True, text=True,
                          timeout=600)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-2000:]
    losses = [float(v) for v in re.findall(r"epoch \d+: train loss ([0-9.]+)", proc.stdout)]
    assert len(losses) == 3 and losses[-1] < losses[0], proc.stdout[-1500:]
    assert "label__output" in proc.stdout


def test_elastic_mnist_example_trains():
    out = _launch(2, ["examples/pytorch_mnist_elastic.py", "--epochs", "2", "--samples", "1024",
                      "--batch-size", "64", "--no-cuda"])
    rows = re.findall(r"epoch (\d+): loss ([0-9.]+) accuracy ([0-9.]+) on 2 rank\(s\)", out)
    assert [r[0] for r in rows] == ["0", "1"], out[-1500:]
    assert float(rows[1][1]) < float(rows[0][1]) and float(rows[1][2]) > float(rows[0][2])


def test_elastic_example_through_the_command_line_with_a_discovery_script(tmp_path):
    """horovodrun --min-np/--max-np --host-discovery-script: the elastic
    driver behind the command line, on one "host" with two slots."""
    script = tmp_path / "discover.sh"
    script.write_text("#!/bin/bash\necho localhost:2\n")
    script.chmod(0o755)
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""),
               CUDA_VISIBLE_DEVICES="")
    proc = subprocess.run([sys.executable, "-m", "horovod_b200.runner.launch", "-np", "2",
                           "--min-np", "1", "--max-np", "2", "--host-discovery-script",
                           str(script), sys.executable, "examples/pytorch_mnist_elastic.py",
                           "--epochs", "2", "--samples", "512", "--no-cuda"],
                          cwd=ROOT, env=env, capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-2000:]
    assert len(re.findall(r"epoch \d+: loss [0-9.]+ accuracy [0-9.]+ on 2 rank\(s\)",
                          proc.stdout)) == 2, proc.stdout[-1500:]


def _elastic_sum(tag):
    import torch
    import horovod_b200.torch as hvd
    hvd.init()

    @hvd.elastic.run
    def train(state):
        for state.step in range(state.step, 5):
            state.total += float(hvd.allreduce(torch.ones(1), op=hvd.Sum, name="s"))
            state.commit()
        return state.total

    total = train(hvd.elastic.ObjectState(hvd.broadcast_object, hvd.rank, step=0, total=0.0))
    result = (tag, hvd.rank(), hvd.size(), total)
    hvd.shutdown()
    return result


def test_programmatic_run_with_elastic_arguments(tmp_path):
    import cloudpickle
    import horovod_b200.runner as runner
    cloudpickle.register_pickle_by_value(sys.modules[__name__])
    script = tmp_path / "discover.sh"
    script.write_text("#!/bin/bash\necho localhost:2\n")
    script.chmod(0o755)
    results = runner.run(_elastic_sum, args=("x",), np=2, min_np=1, max_np=2,
                         host_discovery_script=str(script),
                         env={"CUDA_VISIBLE_DEVICES": "", "PYTHONPATH": ROOT})
    assert results == [("x", 0, 2, 10.0), ("x", 1, 2, 10.0)]


def _elastic_sizes():
    import time
    import torch
    import horovod_b200.torch as hvd
    hvd.init()

    @hvd.elastic.run
    def train(state):
        for state.step in range(state.step, 60):
            size_now = int(hvd.allreduce(torch.ones(1), op=hvd.Sum, name="s"))
            time.sleep(0.2)
            state.sizes.append(size_now)
            state.commit()
        return state.sizes

    sizes = train(hvd.elastic.ObjectState(hvd.broadcast_object, hvd.rank, step=0, sizes=[]))
    result = (hvd.rank(), hvd.size(), sizes[-1], len(sizes) >= 60)
    hvd.shutdown()
    return result


def test_programmatic_elastic_run_reports_the_ranks_of_the_last_round(tmp_path):
    """A host disappears while run() is under way: its worker leaves quietly,
    the survivor finishes, and the results are those of the ranks that
    existed at the end (the survivor under its new rank 0)."""
    import time
    import cloudpickle
    import horovod_b200.runner as runner
    cloudpickle.register_pickle_by_value(sys.modules[__name__])
    script = tmp_path / "discover.sh"
    script.write_text("#!/bin/bash\necho localhost:1\n"
                      "if [ $(( $(date +%%s) - %d )) -lt 10 ]; then echo 127.0.0.1:1; fi\n"
                      % int(time.time()))
    script.chmod(0o755)
    results = runner.run(_elastic_sizes, np=2, min_np=1, max_np=2,
                         host_discovery_script=str(script),
                         env={"CUDA_VISIBLE_DEVICES": "", "PYTHONPATH": ROOT})
    assert results == [(0, 1, 1, True)]
