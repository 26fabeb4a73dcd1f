"""Training data of an estimator: a DataFrame becomes Parquet files in the
store, and every rank reads its own share of them in batches.

``prepare_data`` writes the selected columns of a Spark or pandas DataFrame
as a train (and, when asked for, a validation) dataset with enough files that
every rank gets several, and returns the row counts and a description of the
columns. ``ParquetShardReader`` is what a rank iterates over: the row groups
are dealt out to the ranks in turn, read with pyarrow, shuffled and cut into
batches of numpy arrays; it never ends, so that every rank can take the same
number of steps per epoch whatever its share of the rows.

The reference prepares the data the same way (horovod/spark/common/util.py
prepare_data / get_simple_meta_from_parquet) and reads it through Petastorm
(horovod/spark/torch/remote.py:37-416, horovod/spark/data_loaders/
pytorch_data_loaders.py); here the reader is built on pyarrow alone.
"""
import contextlib

import numpy as np


def _is_pandas(df):
    try:
        import pandas
    except ImportError:  # pragma: no cover
        return False
    return isinstance(df, pandas.DataFrame)


def _filesystem(store):
    """(pyarrow filesystem, path -> path inside that filesystem) of a store."""
    if hasattr(store, "fs"):
        return store.fs, (lambda p: p)
    from pyarrow import fs
    normalize = getattr(store, "normalize", None)

    def local(path):
        path = path[len("file://"):] if path.startswith("file://") else path
        return normalize(path) if normalize else path
    return fs.LocalFileSystem(), local


def _parquet_files(filesystem, path):
    from pyarrow.fs import FileSelector, FileType
    if filesystem.get_file_info(path).type != FileType.Directory:
        return []
    infos = filesystem.get_file_info(FileSelector(path, recursive=True))
    return sorted(i.path for i in infos
                  if i.type == FileType.File and i.path.endswith(".parquet"))


def list_row_groups(store, path):
    """[(file, row group index, rows)] of the dataset at ``path``, in a
    stable order (the same on every rank)."""
    import pyarrow.parquet as pq
    filesystem, to_fs = _filesystem(store)
    pieces = []
    for name in _parquet_files(filesystem, to_fs(path)):
        with filesystem.open_input_file(name) as f:
            meta = pq.ParquetFile(f).metadata
            for g in range(meta.num_row_groups):
                rows = meta.row_group(g).num_rows
                if rows:
                    pieces.append((name, g, rows))
    return pieces


def _column_to_numpy(column):
    """A pyarrow (chunked) array as one numpy array: scalars as (n,), lists
    of one length as (n, length)."""
    import pyarrow as pa
    array = column.combine_chunks() if isinstance(column, pa.ChunkedArray) else column
    if pa.types.is_list(array.type) or pa.types.is_large_list(array.type) \
            or pa.types.is_fixed_size_list(array.type):
        n = len(array)
        flat = _column_to_numpy(array.flatten())
        if n and flat.shape[0] % n == 0:
            width = flat.shape[0] // n
            if pa.types.is_fixed_size_list(array.type) or \
                    bool((np.diff(array.offsets.to_numpy()) == width).all()):
                return flat.reshape((n, width) + flat.shape[1:])
        return np.stack([np.asarray(v) for v in array.to_pylist()]) if n else flat
    return array.to_numpy(zero_copy_only=False)


def read_piece(store, piece, columns):
    """{column: numpy array} of one row group."""
    import pyarrow.parquet as pq
    filesystem, _ = _filesystem(store)
    name, group, _rows = piece
    with filesystem.open_input_file(name) as f:
        table = pq.ParquetFile(f).read_row_group(group, columns=list(columns))
    return {c: _column_to_numpy(table.column(c)) for c in columns}


def read_metadata(store, path, columns=None):
    """(rows, {column: {"dtype": numpy dtype name, "shape": per-row shape}},
    average bytes per row) of the dataset at ``path``."""
    pieces = list_row_groups(store, path)
    if not pieces:
        raise ValueError("no Parquet data found at %s" % path)
    import pyarrow.parquet as pq
    filesystem, _ = _filesystem(store)
    with filesystem.open_input_file(pieces[0][0]) as f:
        names = pq.ParquetFile(f).schema_arrow.names
    columns = list(columns) if columns else names
    missing = [c for c in columns if c not in names]
    if missing:
        raise ValueError("columns %s are not in the dataset at %s (it has %s)"
                         % (missing, path, names))
    first = read_piece(store, pieces[0], columns)
    meta, row_bytes = {}, 0
    for c in columns:
        a = first[c]
        meta[c] = {"dtype": a.dtype.name, "shape": tuple(a.shape[1:])}
        row_bytes += a.dtype.itemsize * int(np.prod(a.shape[1:], dtype=np.int64))
    return sum(p[2] for p in pieces), meta, row_bytes


def _write_pandas(store, pdf, path, files):
    import pyarrow as pa
    import pyarrow.parquet as pq
    filesystem, to_fs = _filesystem(store)
    path = to_fs(path)
    from pyarrow.fs import FileType
    if filesystem.get_file_info(path).type != FileType.NotFound:
        filesystem.delete_dir(path)
    filesystem.create_dir(path, recursive=True)
    files = max(1, min(files, len(pdf)))
    bounds = np.linspace(0, len(pdf), files + 1).astype(int)
    for i in range(files):
        part = pdf.iloc[bounds[i]:bounds[i + 1]]
        if len(part) == 0:
            continue
        table = pa.Table.from_pandas(part, preserve_index=False)
        with filesystem.open_output_stream("%s/part-%05d.parquet" % (path, i)) as out:
            pq.write_table(table, out)


def _spark_vectors_to_arrays(df, columns):
    """pyspark.ml vectors are stored as arrays of doubles."""
    vector_columns = [f.name for f in df.schema.fields
                      if f.name in columns and f.dataType.typeName() == "vector"]
    if not vector_columns:
        return df
    from pyspark.ml.functions import vector_to_array
    for c in vector_columns:
        df = df.withColumn(c, vector_to_array(df[c]))
    return df


def _split(df, validation, seed):
    """(train, val or None). ``validation`` is a fraction of the rows picked at
    random or the name of a column that is true for validation rows."""
    if validation is None or validation == 0:
        return df, None
    if isinstance(validation, str):
        if _is_pandas(df):
            mask = df[validation].astype(bool)
            return df[~mask].drop(columns=[validation]), df[mask].drop(columns=[validation])
        flag = df[validation]
        return (df.filter(~flag.cast("boolean")).drop(validation),
                df.filter(flag.cast("boolean")).drop(validation))
    fraction = float(validation)
    if not 0 < fraction < 1:
        raise ValueError("validation must be a column name or a fraction in (0, 1), got %r"
                         % (validation,))
    if _is_pandas(df):
        picked = np.random.RandomState(seed).rand(len(df)) < fraction
        return df[~picked], df[picked]
    train, val = df.randomSplit([1.0 - fraction, fraction], seed=seed)
    return train, val


_prepared = {}  # cache key -> (train_rows, val_rows, metadata, row_bytes)
_prepared_frames = {}  # cache key -> weak reference to the pandas frame it was made from


def clear_training_cache():
    """Forgets which DataFrames are already in a store, so that the next fit
    writes its data again (horovod/spark/common/util.py clear_training_cache)."""
    _prepared.clear()
    _prepared_frames.clear()


def _frame_key(df):
    """Identifies the content of a DataFrame cheaply: Spark's hash of the
    logical plan, or the object and shape of a pandas frame."""
    if _is_pandas(df):
        return ("pandas", id(df), df.shape, tuple(df.columns))
    plan_hash = getattr(df, "semanticHash", None)
    return ("spark", plan_hash() if callable(plan_hash) else id(df))


def _same_frame(key, df):
    """An object id can be handed out again after its frame was collected."""
    if not _is_pandas(df):
        return True
    ref = _prepared_frames.get(key)
    return ref is not None and ref() is df


@contextlib.contextmanager
def prepare_data(num_proc, store, df, label_columns, feature_columns, validation=None,
                 sample_weight_col=None, partitions_per_process=10, dataset_idx=None,
                 seed=0, verbose=0):
    """Writes ``df`` into the store as Parquet and yields
    ``(train_rows, val_rows, metadata, avg_row_size)``."""
    columns = list(feature_columns) + list(label_columns)
    if sample_weight_col:
        columns.append(sample_weight_col)
    keep = columns + ([validation] if isinstance(validation, str) else [])
    files = max(1, int(num_proc) * int(partitions_per_process))
    train_path = store.get_train_data_path(dataset_idx)
    val_path = store.get_val_data_path(dataset_idx)
    # The same DataFrame prepared the same way is not written twice (repeated
    # fits of a parameter search); the files must still be there.
    key = (_frame_key(df), tuple(keep), repr(validation), files, train_path, seed)
    if key in _prepared and _same_frame(key, df) and dataset_exists(store, train_path):
        if verbose:
            print("using the training data already at %s" % train_path)
        yield _prepared[key]
        return
    if _is_pandas(df):
        absent = [c for c in keep if c not in df.columns]
        if absent:
            raise ValueError("columns %s are not in the DataFrame" % absent)
        train, val = _split(df[keep], validation, seed)
        _write_pandas(store, train, train_path, files)
        if val is not None and len(val):
            _write_pandas(store, val, val_path, files)
        else:
            val = None
    else:
        prepared = _spark_vectors_to_arrays(df.select(*keep), columns)
        train, val = _split(prepared, validation, seed)
        train.repartition(files).write.mode("overwrite").parquet(train_path)
        if val is not None:
            val.repartition(files).write.mode("overwrite").parquet(val_path)
    train_rows, metadata, row_bytes = read_metadata(store, train_path, columns)
    val_rows = 0
    if val is not None:
        with contextlib.suppress(ValueError):  # an empty validation split
            val_rows = read_metadata(store, val_path, columns)[0]
    if verbose:
        print("train_rows=%d val_rows=%d avg_row_size=%d" % (train_rows, val_rows, row_bytes))
    for stale in [k for k in _prepared if k[4] == train_path]:
        del _prepared[stale]  # the path now holds this data
    _prepared[key] = (train_rows, val_rows, metadata, row_bytes)
    if _is_pandas(df):
        import weakref
        _prepared_frames[key] = weakref.ref(df)
    yield _prepared[key]


class ParquetShardReader:
    """Endless iterator over this rank's share of a Parquet dataset in
    batches of ``{column: numpy array}``.

    Row groups are dealt out in turn (piece ``i`` goes to rank ``i % size``);
    when there are fewer row groups than ranks every rank reads all of them
    and keeps the rows ``rank, rank + size, ...``. Each pass over the share
    visits the pieces and the rows inside a piece in a new random order when
    ``shuffle`` is set; rows left over at the end of a piece open the next
    batch. ``cache`` keeps the decoded pieces in memory after the first pass.
    """

    def __init__(self, store, path, columns, batch_size, rank=0, size=1, shuffle=True, seed=0,
                 cache=False, transform=None):
        self._store, self._columns = store, list(columns)
        self._batch = int(batch_size)
        self._shuffle, self._cache, self._transform = shuffle, ({} if cache else None), transform
        self._rng = np.random.RandomState((seed * 1000003 + rank) % (2 ** 31))
        pieces = list_row_groups(store, path)
        if not pieces:
            raise ValueError("no Parquet data found at %s" % path)
        if len(pieces) >= size:
            self._pieces, self._stride = pieces[rank::size], None
        else:
            self._pieces, self._stride = pieces, (rank, size)
        self.rows = sum(self._rows_of(p) for p in self._pieces)
        if self.rows == 0:
            raise ValueError("rank %d of %d has no rows of %s to read" % (rank, size, path))

    def _rows_of(self, piece):
        if self._stride is None:
            return piece[2]
        rank, size = self._stride
        return len(range(rank, piece[2], size))

    def _load(self, index):
        if self._cache is not None and index in self._cache:
            return self._cache[index]
        data = read_piece(self._store, self._pieces[index], self._columns)
        if self._stride is not None:
            rank, size = self._stride
            data = {c: a[rank::size] for c, a in data.items()}
        if self._cache is not None:
            self._cache[index] = data
        return data

    def __iter__(self):
        carry = None
        while True:
            order = self._rng.permutation(len(self._pieces)) if self._shuffle \
                else range(len(self._pieces))
            for index in order:
                data = self._load(int(index))
                n = len(next(iter(data.values())))
                if n == 0:
                    continue
                if self._shuffle:
                    rows = self._rng.permutation(n)
                    data = {c: a[rows] for c, a in data.items()}
                if carry is not None:
                    data = {c: np.concatenate([carry[c], a]) for c, a in data.items()}
                    n = len(next(iter(data.values())))
                full = n - n % self._batch
                for start in range(0, full, self._batch):
                    batch = {c: a[start:start + self._batch] for c, a in data.items()}
                    yield self._transform(batch) if self._transform else batch
                carry = {c: a[full:] for c, a in data.items()} if full < n else None


def steps_per_epoch(rows, batch_size, size, limit=None):
    """How many batches every rank takes per epoch so that together they see
    about ``rows`` rows; ``limit`` caps it (for quick trial runs)."""
    steps = max(1, int(np.ceil(rows / float(batch_size * size))))
    return min(steps, int(limit)) if limit else steps


def dataset_exists(store, path):
    return bool(list_row_groups(store, path)) if store.exists(path) else False
