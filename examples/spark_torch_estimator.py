"""Fitting a PyTorch model to a DataFrame with ``TorchEstimator`` and scoring
the DataFrame with the ``TorchModel`` that comes back.

    python examples/spark_torch_estimator.py --num-proc 2 --work-dir /tmp/est

With ``--spark`` the DataFrame is a Spark DataFrame and the ranks run as Spark
tasks (needs ``pyspark`` and a session); without it the same estimator is
fitted to a pandas DataFrame and the ranks are processes of this package's
launcher on this machine.

Counterpart of the reference's examples/spark/pytorch/pytorch_spark_mnist.py,
on synthetic regression data since no dataset can be downloaded here.
"""
import argparse
import tempfile

import numpy as np
import pandas as pd
import torch

from horovod_b200.spark.common.backend import LocalBackend, SparkBackend
from horovod_b200.spark.common.store import Store
from horovod_b200.spark.torch import TorchEstimator


class Regressor(torch.nn.Module):
    def __init__(self, width):
        super().__init__()
        self.net = torch.nn.Sequential(torch.nn.Linear(width, 32), torch.nn.ReLU(),
                                       torch.nn.Linear(32, 1))

    def forward(self, features):
        return self.net(features)


def synthetic_frame(rows, width, seed=0):
    rng = np.random.RandomState(seed)
    x = rng.randn(rows, width).astype(np.float32)
    y = np.sin(x[:, 0]) + 0.5 * x[:, 1] * x[:, 2] + 0.05 * rng.randn(rows).astype(np.float32)
    return pd.DataFrame({"features": list(x), "label": y.astype(np.float32)})


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--num-proc", type=int, default=2)
    parser.add_argument("--rows", type=int, default=4096)
    parser.add_argument("--width", type=int, default=8)
    parser.add_argument("--epochs", type=int, default=5)
    parser.add_argument("--batch-size", type=int, default=64)
    parser.add_argument("--work-dir", default=None, help="store prefix (default: a temp dir)")
    parser.add_argument("--spark", action="store_true", help="run the ranks as Spark tasks")
    parser.add_argument("--no-cuda", action="store_true")
    args = parser.parse_args()

    frame = synthetic_frame(args.rows, args.width)
    if args.spark:
        from pyspark.sql import SparkSession
        spark = SparkSession.builder.appName("torch estimator").getOrCreate()
        frame = spark.createDataFrame(frame.assign(features=frame["features"].map(list)))
        backend = SparkBackend(num_proc=args.num_proc)
    else:
        backend = LocalBackend(num_proc=args.num_proc)

    model = Regressor(args.width)
    estimator = TorchEstimator(
        backend=backend, store=Store.create(args.work_dir or tempfile.mkdtemp(prefix="hvd_est_")),
        model=model, optimizer=torch.optim.Adam(model.parameters(), lr=3e-3),
        loss=torch.nn.MSELoss(), feature_cols=["features"], label_cols=["label"],
        input_shapes=[[-1, args.width]], batch_size=args.batch_size, epochs=args.epochs,
        validation=0.1, verbose=1, no_cuda=args.no_cuda)
    fitted = estimator.fit(frame)
    for entry in fitted.getHistory():
        print("epoch %d: train loss %.4f, validation loss %.4f"
              % (entry["epoch"], entry["train"]["loss"], entry["validation"]["loss"]))
    scored = fitted.transform(frame)
    if args.spark:
        scored.select("label", "label__output").show(5)
    else:
        print(scored[["label", "label__output"]].head())


if __name__ == "__main__":
    main()
