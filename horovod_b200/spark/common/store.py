"""Where a training run keeps intermediate datasets, checkpoints and logs.

A store is a directory tree:

    <prefix>/intermediate_{train,val,test}_data[.<idx>]   datasets (Parquet)
    <prefix>/runs/<run_id>/checkpoint                      model checkpoint
    <prefix>/runs/<run_id>/logs/                           training logs

``Store.create(prefix_path)`` picks the implementation from the path:
``LocalStore`` for paths the operating system can open (local disk, NFS, FUSE
mounts), ``DBFSLocalStore`` for ``dbfs:/`` paths (Databricks mounts DBFS at
``/dbfs``), ``HDFSStore`` for ``hdfs://`` URLs (through ``pyarrow.fs``, which
needs libhdfs at run time); other object stores are refused with a message
saying so. Workers write into a private local directory and publish it with
``sync_fn``.

The method names are those of horovod/spark/common/store.py:36-536 (Store,
AbstractFilesystemStore, LocalStore), which estimators and remote trainers
call; the layout is data-driven here instead of one method body per path.
"""
import contextlib
import os
import shutil
import tempfile

_REMOTE_SCHEMES = ("s3://", "s3a://", "gs://", "abfs://")
_DATASETS = {"train": "intermediate_train_data", "val": "intermediate_val_data",
             "test": "intermediate_test_data"}
_CHECKPOINT_FILE, _LOGS_DIR = "checkpoint", "logs"


def _local(path):
    """file:// URLs and plain paths name the same thing."""
    return path[len("file://"):] if path.startswith("file://") else path


class Store:
    """Interface. ``FilesystemStore`` is the one implementation built here."""

    @staticmethod
    def create(prefix_path, *args, **kwargs):
        if prefix_path.startswith(_REMOTE_SCHEMES):
            raise ValueError(
                "Only filesystem paths, dbfs:/ and hdfs:// are supported by this build (got "
                "%r); mount the remote filesystem and pass the mount point." % prefix_path)
        if DBFSLocalStore.matches(prefix_path):
            return DBFSLocalStore(prefix_path, *args, **kwargs)
        if prefix_path.startswith("hdfs://"):
            return HDFSStore(prefix_path, *args, **kwargs)
        return LocalStore(prefix_path, *args, **kwargs)

    def to_remote(self, run_id, dataset_idx):
        """A small picklable object with just the paths (and the sync
        function) a trainer on another machine needs."""
        view = _RemoteView()
        view.train_data_path = self.get_train_data_path(dataset_idx)
        view.val_data_path = self.get_val_data_path(dataset_idx)
        view.test_data_path = self.get_test_data_path(dataset_idx)
        view.saving_runs = self.saving_runs()
        view.runs_path = self.get_runs_path()
        view.run_path = self.get_run_path(run_id)
        view.checkpoint_path = self.get_checkpoint_path(run_id)
        view.logs_path = self.get_logs_path(run_id)
        view.checkpoint_filename = self.get_checkpoint_filename()
        view.logs_subdir = self.get_logs_subdir()
        view.sync = self.sync_fn(run_id)
        return view


class _RemoteView:
    pass


class FilesystemStore(Store):
    def __init__(self, prefix_path, train_path=None, val_path=None, test_path=None,
                 runs_path=None, save_runs=True):
        self.prefix_path = _local(prefix_path)
        given = {"train": train_path, "val": val_path, "test": test_path}
        self._data = {kind: given[kind] or os.path.join(self.prefix_path, name)
                      for kind, name in _DATASETS.items()}
        self._runs = runs_path or os.path.join(self.prefix_path, "runs")
        self._save_runs = save_runs

    # ---- datasets -----------------------------------------------------------
    def _dataset(self, kind, idx):
        base = self._data[kind]
        return base if idx is None else "%s.%s" % (base, idx)

    def get_train_data_path(self, idx=None):
        return self._dataset("train", idx)

    def get_val_data_path(self, idx=None):
        return self._dataset("val", idx)

    def get_test_data_path(self, idx=None):
        return self._dataset("test", idx)

    def is_parquet_dataset(self, path):
        path = _local(path)
        try:
            names = os.listdir(path)
        except (FileNotFoundError, NotADirectoryError):
            return False
        return any(n.endswith(".parquet") or n in ("_metadata", "_common_metadata")
                   for n in names)

    # ---- runs -----------------------------------------------------------------
    def saving_runs(self):
        return self._save_runs

    def get_runs_path(self):
        return self._runs

    def get_run_path(self, run_id):
        return os.path.join(self._runs, run_id)

    def get_checkpoint_filename(self):
        return _CHECKPOINT_FILE

    def get_logs_subdir(self):
        return _LOGS_DIR

    def _in_run(self, run_id, leaf):
        return os.path.join(self.get_run_path(run_id), leaf) if self._save_runs else None

    def get_checkpoint_path(self, run_id):
        return self._in_run(run_id, _CHECKPOINT_FILE)

    def get_logs_path(self, run_id):
        return self._in_run(run_id, _LOGS_DIR)

    # ---- file access ----------------------------------------------------------
    def exists(self, path):
        return os.path.exists(_local(path))

    def read(self, path):
        with open(_local(path), "rb") as f:
            return f.read()

    def write_text(self, path, text):
        path = _local(path)
        os.makedirs(os.path.dirname(path), exist_ok=True)
        with open(path, "w") as f:
            f.write(text)

    def get_local_output_dir_fn(self, run_id):
        """A context manager factory: a scratch directory for one worker's
        checkpoint and logs, removed afterwards."""
        @contextlib.contextmanager
        def scratch():
            with tempfile.TemporaryDirectory(prefix="hvd_run_%s_" % run_id) as path:
                yield path
        return scratch

    def sync_fn(self, run_id):
        """fn(local_dir): merges a worker's scratch directory into the run's
        directory in the store."""
        target = self.get_run_path(run_id)

        def publish(local_dir):
            shutil.copytree(local_dir, target, dirs_exist_ok=True)
        return publish


class LocalStore(FilesystemStore):
    """A store on local disk (or any mounted filesystem); creates the prefix."""

    def __init__(self, prefix_path, *args, **kwargs):
        super().__init__(prefix_path, *args, **kwargs)
        os.makedirs(self.prefix_path, exist_ok=True)


class DBFSLocalStore(LocalStore):
    """Databricks File System through its local mount: ``dbfs:/a/b`` and
    ``/dbfs/a/b`` name the same directory; everything is stored under the
    ``/dbfs`` form (horovod/spark/common/store.py DBFSLocalStore). ``root``
    replaces ``/dbfs`` (for tests and unusual mounts)."""

    def __init__(self, prefix_path, *args, root="/dbfs", **kwargs):
        self._root = root.rstrip("/")
        kwargs = {k: (self.normalize(v) if k.endswith("_path") and v else v)
                  for k, v in kwargs.items()}
        super().__init__(self.normalize(prefix_path), *args, **kwargs)

    @staticmethod
    def matches(path):
        return path.startswith(("dbfs:/", "/dbfs/", "file:///dbfs/"))

    def normalize(self, path):
        path = _local(path)
        if path.startswith("dbfs:///"):
            return self._root + "/" + path[len("dbfs:///"):]
        if path.startswith("dbfs:/"):
            return self._root + "/" + path[len("dbfs:/"):]
        if path.startswith("/dbfs/") and self._root != "/dbfs":
            return self._root + path[len("/dbfs"):]
        return path

    def exists(self, path):
        return super().exists(self.normalize(path))

    def read(self, path):
        return super().read(self.normalize(path))


class ArrowFilesystemStore(FilesystemStore):
    """The same layout on any ``pyarrow.fs.FileSystem``: paths are plain
    strings inside that filesystem; files are read, written and published
    through its API instead of the operating system's."""

    def __init__(self, filesystem, prefix_path, *args, **kwargs):
        super().__init__(prefix_path, *args, **kwargs)
        self.fs = filesystem
        self.fs.create_dir(self.prefix_path, recursive=True)

    def _info(self, path):
        return self.fs.get_file_info(path)

    def exists(self, path):
        from pyarrow.fs import FileType
        return self._info(path).type != FileType.NotFound

    def is_parquet_dataset(self, path):
        from pyarrow.fs import FileSelector, FileType
        if self._info(path).type != FileType.Directory:
            return False
        names = [os.path.basename(i.path) for i in self.fs.get_file_info(FileSelector(path))]
        return any(n.endswith(".parquet") or n in ("_metadata", "_common_metadata")
                   for n in names)

    def read(self, path):
        with self.fs.open_input_stream(path) as f:
            return f.read()

    def write_text(self, path, text):
        self.fs.create_dir(os.path.dirname(path), recursive=True)
        with self.fs.open_output_stream(path) as f:
            f.write(text.encode())

    def sync_fn(self, run_id):
        target = self.get_run_path(run_id)
        fs = self.fs

        def publish(local_dir):
            for root, _dirs, files in os.walk(local_dir):
                rel = os.path.relpath(root, local_dir)
                dest = target if rel == "." else target + "/" + rel.replace(os.sep, "/")
                fs.create_dir(dest, recursive=True)
                for name in files:
                    with open(os.path.join(root, name), "rb") as src, \
                            fs.open_output_stream(dest + "/" + name) as dst:
                        shutil.copyfileobj(src, dst)
        return publish


class HDFSStore(ArrowFilesystemStore):
    """``hdfs://namenode:port/path`` through ``pyarrow.fs.HadoopFileSystem``
    (needs libhdfs and a Hadoop client configuration on every machine that
    touches the store; horovod/spark/common/store.py HDFSStore)."""

    def __init__(self, prefix_path, *args, **kwargs):
        try:
            from pyarrow.fs import FileSystem
            filesystem, path = FileSystem.from_uri(prefix_path)
        except Exception as e:  # noqa: BLE001 - libhdfs missing, bad URL, no cluster
            raise RuntimeError("Cannot open %s through pyarrow's HDFS driver: %s"
                               % (prefix_path, e)) from e
        super().__init__(filesystem, path, *args, **kwargs)
