"""Running a job inside Spark tasks (needs ``pyspark`` at call time) and the
filesystem store used for intermediate data, checkpoints and logs."""
from horovod_b200.spark.runner import run  # noqa: F401
from horovod_b200.spark.elastic import run_elastic  # noqa: F401
from horovod_b200.spark.common.store import (ArrowFilesystemStore, DBFSLocalStore,  # noqa: F401
                                             FilesystemStore, HDFSStore, LocalStore, Store)
