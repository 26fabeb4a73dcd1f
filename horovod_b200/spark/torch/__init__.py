"""Estimator API for PyTorch models: ``TorchEstimator.fit(df)`` trains on the
ranks of a backend and returns a ``TorchModel`` that adds predictions to a
DataFrame."""
from horovod_b200.spark.torch.estimator import TorchEstimator, TorchModel  # noqa: F401
