"""Loaders that feed an estimator's trainer from the Parquet data in a store."""
from horovod_b200.spark.data_loaders.pytorch_data_loaders import (  # noqa: F401
    AsyncParquetDataLoader, ParquetDataLoader)
