"""Where a training run keeps its intermediate datasets, checkpoints and
logs. ``Store.create(prefix_path)`` picks the implementation from the path;
only plain filesystem paths (local disk, NFS, FUSE mounts) are built here:
HDFS / DBFS / S3 URLs are refused with a clear message.
Parity: horovod/spark/common/store.py:36-536 (Store, AbstractFilesystemStore,
LocalStore)."""
import contextlib
import os
import shutil
import tempfile


class Store:
    """Abstract layout: <prefix>/intermediate_train_data[.idx], .../runs/<run_id>/
    {checkpoint, logs}."""

    def is_parquet_dataset(self, path):
        raise NotImplementedError()

    def get_train_data_path(self, idx=None):
        raise NotImplementedError()

    def get_val_data_path(self, idx=None):
        raise NotImplementedError()

    def get_test_data_path(self, idx=None):
        raise NotImplementedError()

    def saving_runs(self):
        raise NotImplementedError()

    def get_runs_path(self):
        raise NotImplementedError()

    def get_run_path(self, run_id):
        raise NotImplementedError()

    def get_checkpoint_path(self, run_id):
        raise NotImplementedError()

    def get_logs_path(self, run_id):
        raise NotImplementedError()

    def get_checkpoint_filename(self):
        raise NotImplementedError()

    def get_logs_subdir(self):
        raise NotImplementedError()

    def exists(self, path):
        raise NotImplementedError()

    def read(self, path):
        raise NotImplementedError()

    def write_text(self, path, text):
        raise NotImplementedError()

    def sync_fn(self, run_id):
        """Returns fn(local_run_path) that publishes a worker's local run
        directory (checkpoint, logs) into the store."""
        raise NotImplementedError()

    def to_remote(self, run_id, dataset_idx):
        """A picklable view with the paths a remote trainer needs."""
        attrs = self._remote_attrs(run_id, dataset_idx)

        class RemoteStore:
            def __init__(self):
                self.__dict__.update(attrs)

        return RemoteStore()

    def _remote_attrs(self, run_id, dataset_idx):
        return {
            "train_data_path": self.get_train_data_path(dataset_idx),
            "val_data_path": self.get_val_data_path(dataset_idx),
            "test_data_path": self.get_test_data_path(dataset_idx),
            "saving_runs": self.saving_runs(),
            "runs_path": self.get_runs_path(),
            "run_path": self.get_run_path(run_id),
            "checkpoint_path": self.get_checkpoint_path(run_id),
            "logs_path": self.get_logs_path(run_id),
            "checkpoint_filename": self.get_checkpoint_filename(),
            "logs_subdir": self.get_logs_subdir(),
            "sync": self.sync_fn(run_id),
        }

    @staticmethod
    def create(prefix_path, *args, **kwargs):
        for scheme in ("hdfs://", "dbfs:/", "s3://", "s3a://", "gs://", "abfs://"):
            if prefix_path.startswith(scheme):
                raise ValueError(
                    "Only filesystem paths are supported by this build (got %r); mount the "
                    "remote filesystem and pass the mount point." % prefix_path)
        return LocalStore(prefix_path, *args, **kwargs)


class FilesystemStore(Store):
    """Store over anything the operating system presents as a directory tree."""

    def __init__(self, prefix_path, train_path=None, val_path=None, test_path=None,
                 runs_path=None, save_runs=True):
        self.prefix_path = self._strip(prefix_path)
        self._train_path = train_path or self._join("intermediate_train_data")
        self._val_path = val_path or self._join("intermediate_val_data")
        self._test_path = test_path or self._join("intermediate_test_data")
        self._runs_path = runs_path or self._join("runs")
        self._save_runs = save_runs

    @staticmethod
    def _strip(path):
        return path[len("file://"):] if path.startswith("file://") else path

    def _join(self, *parts):
        return os.path.join(self.prefix_path, *parts)

    @staticmethod
    def _indexed(path, idx):
        return "%s.%s" % (path, idx) if idx is not None else path

    def is_parquet_dataset(self, path):
        path = self._strip(path)
        if not os.path.isdir(path):
            return False
        return any(f.endswith(".parquet") or f == "_metadata" or f == "_common_metadata"
                   for f in os.listdir(path))

    def get_train_data_path(self, idx=None):
        return self._indexed(self._train_path, idx)

    def get_val_data_path(self, idx=None):
        return self._indexed(self._val_path, idx)

    def get_test_data_path(self, idx=None):
        return self._indexed(self._test_path, idx)

    def saving_runs(self):
        return self._save_runs

    def get_runs_path(self):
        return self._runs_path

    def get_run_path(self, run_id):
        return os.path.join(self._runs_path, run_id)

    def get_checkpoint_path(self, run_id):
        return os.path.join(self.get_run_path(run_id), self.get_checkpoint_filename()) \
            if self._save_runs else None

    def get_logs_path(self, run_id):
        return os.path.join(self.get_run_path(run_id), self.get_logs_subdir()) \
            if self._save_runs else None

    def get_checkpoint_filename(self):
        return "checkpoint"

    def get_logs_subdir(self):
        return "logs"

    def exists(self, path):
        return os.path.exists(self._strip(path))

    def read(self, path):
        with open(self._strip(path), "rb") as f:
            return f.read()

    def write_text(self, path, text):
        path = self._strip(path)
        os.makedirs(os.path.dirname(path), exist_ok=True)
        with open(path, "w") as f:
            f.write(text)

    def get_local_output_dir_fn(self, run_id):
        @contextlib.contextmanager
        def local_run_path():
            path = tempfile.mkdtemp(prefix="hvd_run_%s_" % run_id)
            try:
                yield path
            finally:
                shutil.rmtree(path, ignore_errors=True)
        return local_run_path

    def sync_fn(self, run_id):
        run_path = self.get_run_path(run_id)

        def fn(local_run_path):
            for root, _dirs, files in os.walk(local_run_path):
                rel = os.path.relpath(root, local_run_path)
                dst_dir = run_path if rel == "." else os.path.join(run_path, rel)
                os.makedirs(dst_dir, exist_ok=True)
                for name in files:
                    shutil.copy2(os.path.join(root, name), os.path.join(dst_dir, name))
        return fn


class LocalStore(FilesystemStore):
    """Local disk (or any mounted filesystem)."""

    def __init__(self, prefix_path, *args, **kwargs):
        super().__init__(prefix_path, *args, **kwargs)
        os.makedirs(self.prefix_path, exist_ok=True)
