"""TorchEstimator / TorchModel: data preparation into the store, the sharded
Parquet reader, training on 2 CPU ranks through LocalBackend, prediction, and
the Spark-facing paths against small stand-ins (pyspark is not installed
here). The reference tests its estimators end to end on a local Spark
session (test/integration/test_spark_torch.py); the same checks are made
here on pandas DataFrames."""
import os
import sys

import cloudpickle
import numpy as np
import pandas as pd
import pytest
import torch

from horovod_b200.spark.common import dataset
from horovod_b200.spark.common.backend import Backend, LocalBackend, SparkBackend
from horovod_b200.spark.common.store import LocalStore
from horovod_b200.spark.torch import TorchEstimator, TorchModel

# the model classes below live in this file, which the worker processes cannot import
cloudpickle.register_pickle_by_value(sys.modules[__name__])


def _frame(rows=256, seed=0):
    rng = np.random.RandomState(seed)
    x = rng.randn(rows, 4).astype(np.float32)
    z = rng.randn(rows).astype(np.float64)
    w = np.array([1.0, -2.0, 0.5, 3.0], dtype=np.float32)
    y = x @ w + 0.5 * z.astype(np.float32)
    return pd.DataFrame({"features": list(x), "z": z, "y": y, "row": np.arange(rows),
                         "is_val": (np.arange(rows) % 8 == 0)})


class _Net(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.a = torch.nn.Linear(4, 1)
        self.b = torch.nn.Linear(1, 1, bias=False)

    def forward(self, features, z):
        return self.a(features) + self.b(z)


def test_prepare_data_writes_shards_and_describes_columns(tmp_path):
    store = LocalStore(str(tmp_path))
    df = _frame(100)
    with dataset.prepare_data(2, store, df, ["y"], ["features", "z"], validation="is_val",
                              partitions_per_process=3) as (train_rows, val_rows, meta, row_bytes):
        assert (train_rows, val_rows) == (87, 13)
        assert meta["features"] == {"dtype": "float32", "shape": (4,)}
        assert meta["z"] == {"dtype": "float64", "shape": ()}
        assert row_bytes == 4 * 4 + 8 + 4
    assert len(dataset.list_row_groups(store, store.get_train_data_path())) == 6
    assert store.is_parquet_dataset(store.get_train_data_path())
    # a fraction picks about that share of the rows; writing again replaces the data
    with dataset.prepare_data(1, store, df, ["y"], ["z"], validation=0.25, seed=3) as (tr, va, _m, _b):
        assert tr + va == 100 and 10 <= va <= 40
    # the same frame prepared the same way again is served from the cache: no file is rewritten
    def stamp():
        path = store.get_train_data_path()
        return sorted((n, os.stat(os.path.join(path, n)).st_mtime_ns) for n in os.listdir(path))
    with dataset.prepare_data(1, store, df, ["y"], ["z"], validation=0.25, seed=3) as first:
        written = stamp()
    with dataset.prepare_data(1, store, df, ["y"], ["z"], validation=0.25, seed=3) as second:
        assert second == first and stamp() == written
    dataset.clear_training_cache()
    with dataset.prepare_data(1, store, df, ["y"], ["z"], validation=0.25, seed=3) as third:
        assert third == first and stamp() != written
    with pytest.raises(ValueError, match="not in the DataFrame"):
        with dataset.prepare_data(1, store, df, ["nope"], ["z"]):
            pass
    with pytest.raises(ValueError, match="fraction"):
        with dataset.prepare_data(1, store, df, ["y"], ["z"], validation=1.5):
            pass


@pytest.mark.parametrize("files,size", [(6, 2), (6, 4), (1, 3)])
def test_reader_shares_cover_every_row_once_per_pass(tmp_path, files, size):
    store = LocalStore(str(tmp_path))
    df = _frame(120)
    dataset._write_pandas(store, df[["row", "features"]], store.get_train_data_path(), files)
    seen = []
    for rank in range(size):
        reader = dataset.ParquetShardReader(store, store.get_train_data_path(), ["row", "features"],
                                            batch_size=5, rank=rank, size=size, seed=1)
        batches = iter(reader)
        mine = []
        for _ in range(reader.rows // 5):
            batch = next(batches)
            assert batch["features"].shape == (5, 4) and batch["features"].dtype == np.float32
            mine.extend(batch["row"].tolist())
        assert len(set(mine)) == len(mine)  # no row twice within a pass
        # the features still belong to their rows after shuffling
        assert np.allclose(batch["features"], np.stack(df["features"].iloc[batch["row"]].to_numpy()))
        seen.extend(mine)
    assert len(set(seen)) == len(seen)  # the shares are disjoint
    assert len(seen) >= 120 - 5 * size  # and cover all rows but the last partial batches


def test_reader_is_endless_ordered_without_shuffle_and_cached(tmp_path):
    store = LocalStore(str(tmp_path))
    dataset._write_pandas(store, _frame(10)[["row"]], store.get_train_data_path(), 2)
    reader = dataset.ParquetShardReader(store, store.get_train_data_path(), ["row"], batch_size=4,
                                        shuffle=False, cache=True,
                                        transform=lambda b: {"row": b["row"] + 100})
    it = iter(reader)
    got = [next(it)["row"].tolist() for _ in range(5)]
    # 10 rows in batches of 4: the rest of one pass opens the first batch of the next
    assert got == [[100, 101, 102, 103], [104, 105, 106, 107], [108, 109, 100, 101],
                   [102, 103, 104, 105], [106, 107, 108, 109]]
    assert dataset.steps_per_epoch(10, 4, 1) == 3 and dataset.steps_per_epoch(10, 4, 2) == 2
    assert dataset.steps_per_epoch(1000, 4, 2, limit=7) == 7
    with pytest.raises(ValueError, match="no Parquet data"):
        dataset.ParquetShardReader(store, str(tmp_path / "missing"), ["row"], 4)


def test_settings_accessors_and_argument_checks(tmp_path):
    est = TorchEstimator(model=_Net(), batch_size=16)
    assert est.getBatchSize() == 16 and est.getEpochs() == 1 and est.getFeatureCols() is None
    assert est.setEpochs(3).setLabelCols(["y"]).getEpochs() == 3 and est.getLabelCols() == ["y"]
    with pytest.raises(AttributeError):
        est.getNothing()
    with pytest.raises(TypeError, match="unexpected"):
        TorchEstimator(modle=None)
    with pytest.raises(ValueError, match="num_proc or backend"):
        TorchEstimator(num_proc=2, backend=LocalBackend(2))
    with pytest.raises(ValueError, match="needs optimizer"):
        est.fit(_frame(8))
    net = _Net()
    est = TorchEstimator(model=net, optimizer=torch.optim.SGD(net.parameters(), lr=0.1),
                         loss=torch.nn.MSELoss(), feature_cols=["features", "z"], label_cols=["y"],
                         input_shapes=[[-1, 5], [-1, 1]], store=LocalStore(str(tmp_path)),
                         backend=LocalBackend(1))
    with pytest.raises(ValueError, match="4 values per row"):
        est.fit(_frame(8))
    assert isinstance(LocalBackend(3), Backend) and LocalBackend(3).num_processes() == 3


def _mae(output, label):
    return (output - label).abs().mean()


def test_fit_on_two_ranks_then_transform_save_and_refit_on_parquet(tmp_path):
    torch.manual_seed(0)
    store = LocalStore(str(tmp_path / "store"))
    net = _Net()
    before = {k: v.clone() for k, v in net.state_dict().items()}
    est = TorchEstimator(model=net, optimizer=torch.optim.SGD(net.parameters(), lr=0.1, momentum=0.5),
                         loss=torch.nn.MSELoss(), metrics=[_mae], feature_cols=["features", "z"],
                         label_cols=["y"], input_shapes=[[-1, 4], [-1, 1]], batch_size=16, epochs=6,
                         validation="is_val", store=store, backend=LocalBackend(2), verbose=0,
                         run_id="run1", random_seed=7, partitions_per_process=2, no_cuda=True)
    df = _frame(256)
    fitted = est.fit(df)
    assert isinstance(fitted, TorchModel) and fitted.getRunId() == "run1"
    history = fitted.getHistory()
    assert [h["epoch"] for h in history] == [0, 1, 2, 3, 4, 5]
    assert set(history[0]["train"]) == {"loss", "_mae"} and "validation" in history[0]
    assert history[-1]["train"]["loss"] < 0.2 * history[0]["train"]["loss"]
    assert history[-1]["validation"]["loss"] < history[0]["validation"]["loss"]
    # the estimator's own model is untouched; the fitted copy carries the trained weights
    assert all(torch.equal(before[k], v) for k, v in net.state_dict().items())
    trained = fitted.getModel()
    assert not torch.equal(trained.a.weight, net.a.weight)
    assert torch.allclose(trained.a.weight, torch.tensor([[1.0, -2.0, 0.5, 3.0]]), atol=0.2)
    # the optimizer that comes back is tied to the fitted model and has its momentum
    opt = fitted.getOptimizer()
    assert opt.param_groups[0]["params"][0] is next(trained.parameters())
    assert len(opt.state) == 3
    # rank 0 wrote the checkpoint and the log into the store
    assert store.exists(store.get_checkpoint_path("run1"))
    assert os.path.exists(os.path.join(store.get_logs_path("run1"), "history.jsonl"))
    state = est._load_checkpoint("run1")
    assert torch.equal(state["model"]["a.weight"], trained.a.weight)

    scored = fitted.transform(df)
    assert list(scored.columns)[-1] == "y__output" and len(scored) == len(df)
    assert float(np.mean((scored["y__output"] - scored["y"]) ** 2)) < 0.1
    assert "y__output" not in df.columns
    path = str(tmp_path / "model.bin")
    fitted.save(path)
    again = TorchModel.load(path).setOutputCols(["pred"]).transform(df.iloc[:10])
    assert np.allclose(again["pred"], scored["y__output"].iloc[:10])

    # the data is still in the store: one more epoch from the trained weights
    more = TorchEstimator(model=trained, optimizer=opt, loss=torch.nn.MSELoss(),
                          feature_cols=["features", "z"], label_cols=["y"], batch_size=16,
                          input_shapes=[[-1, 4], [-1, 1]], store=store, backend=LocalBackend(2),
                          verbose=0, no_cuda=True, train_steps_per_epoch=3)
    refit = more.fit_on_parquet(params={"epochs": 2})
    assert more.getEpochs() == 1 and len(refit.getHistory()) == 2
    assert refit.getHistory()[0]["train"]["loss"] < history[0]["train"]["loss"]
    assert "validation" in refit.getHistory()[0]


def test_two_outputs_with_loss_weights_and_sample_weights(tmp_path):
    class Two(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.body = torch.nn.Linear(4, 2)

        def forward(self, features):
            out = self.body(features)
            return out[:, :1], out[:, 1:]

    df = _frame(64)
    df["y2"] = -df["y"]
    df["w"] = np.where(np.arange(64) % 2 == 0, 1.0, 0.0)
    net = Two()
    est = TorchEstimator(model=net, optimizer=torch.optim.Adam(net.parameters(), lr=0.05),
                         loss_constructors=[lambda: torch.nn.MSELoss(reduction="none"),
                                            lambda: torch.nn.L1Loss(reduction="none")],
                         loss_weights=[0.7, 0.3], sample_weight_col="w", feature_cols=["features"],
                         label_cols=["y", "y2"], batch_size=8, epochs=3,
                         store=LocalStore(str(tmp_path)), backend=LocalBackend(1), verbose=0,
                         no_cuda=True, shuffle=False)
    fitted = est.fit(df)
    losses = [h["train"]["loss"] for h in fitted.getHistory()]
    assert losses[-1] < losses[0]
    scored = fitted.transform(df)
    assert {"y__output", "y2__output"} <= set(scored.columns)
    # a loss that already averaged over the batch cannot be weighted per row
    bad = TorchEstimator(model=net, optimizer=torch.optim.Adam(net.parameters()),
                         loss=torch.nn.MSELoss(), sample_weight_col="w", feature_cols=["features"],
                         label_cols=["y", "y2"], store=LocalStore(str(tmp_path)),
                         backend=LocalBackend(1), verbose=0, no_cuda=True)
    with pytest.raises(ValueError, match="reduction='none'"):
        bad.fit(df)


class _Type:
    def __init__(self, name):
        self.name = name

    def typeName(self):
        return self.name

    def simpleString(self):
        return self.name


class _Field:
    def __init__(self, name, kind):
        self.name, self.dataType = name, _Type(kind)


class _FakeSparkFrame:
    """The few DataFrame calls the estimator makes, over a pandas frame."""

    def __init__(self, pdf, log):
        self.pdf, self.log = pdf, log

    @property
    def schema(self):
        kinds = {"float64": "double", "float32": "float", "int64": "bigint", "bool": "boolean"}
        fields = [_Field(c, kinds.get(str(t), "array<float>")) for c, t in self.pdf.dtypes.items()]
        return type("Schema", (), {"fields": fields})()

    def select(self, *cols):
        return _FakeSparkFrame(self.pdf[list(cols)], self.log)

    def randomSplit(self, weights, seed=None):
        self.log.append(("randomSplit", [round(w, 3) for w in weights], seed))
        cut = int(len(self.pdf) * weights[0])
        return (_FakeSparkFrame(self.pdf.iloc[:cut], self.log),
                _FakeSparkFrame(self.pdf.iloc[cut:], self.log))

    def repartition(self, n):
        self.log.append(("repartition", n))
        self.parts = n
        return self

    @property
    def write(self):
        frame = self

        class Writer:
            def mode(self, how):
                frame.log.append(("mode", how))
                return self

            def parquet(self, path):
                dataset._write_pandas(LocalStore(os.path.dirname(path)), frame.pdf, path,
                                      frame.parts)
        return Writer()

    def limit(self, n):
        return _FakeSparkFrame(self.pdf.iloc[:n], self.log)

    def toPandas(self):
        return self.pdf.copy()

    def mapInPandas(self, fn, schema):
        self.log.append(("mapInPandas", schema))
        halves = [self.pdf.iloc[:len(self.pdf) // 2], self.pdf.iloc[len(self.pdf) // 2:]]
        return _FakeSparkFrame(pd.concat(list(fn(iter(halves)))), self.log)


def test_spark_paths_against_stand_ins(tmp_path, monkeypatch):
    """A Spark DataFrame is written with repartition().write.parquet(), split
    with randomSplit, scored with mapInPandas under a schema that names the
    new column; SparkBackend hands the trainer to horovod_b200.spark.run."""
    import horovod_b200.spark.runner as spark_runner
    calls = []

    def fake_spark_run(fn, args=(), kwargs=None, num_proc=None, extra_env=None, verbose=1):
        calls.append((num_proc, extra_env, verbose))
        from horovod_b200.runner import run
        return run(fn, args=args, kwargs=kwargs, np=num_proc, env=extra_env or None)

    monkeypatch.setattr(spark_runner, "run", fake_spark_run)
    log = []
    df = _FakeSparkFrame(_frame(96)[["features", "z", "y"]], log)
    net = _Net()
    est = TorchEstimator(num_proc=2, model=net, optimizer=torch.optim.SGD(net.parameters(), lr=0.05),
                         loss=torch.nn.MSELoss(), feature_cols=["features", "z"], label_cols=["y"],
                         batch_size=8, epochs=2, validation=0.25, store=LocalStore(str(tmp_path)),
                         verbose=0, partitions_per_process=1, no_cuda=True, random_seed=5)
    fitted = est.fit(df)
    assert calls == [(2, {}, 0)]
    assert ("randomSplit", [0.75, 0.25], 5) in log and ("repartition", 2) in log
    assert ("mode", "overwrite") in log
    assert len(fitted.getHistory()) == 2 and "validation" in fitted.getHistory()[0]
    scored = fitted.transform(df)
    schema = [entry[1] for entry in log if entry[0] == "mapInPandas"][0]
    assert schema == "features array<float>, z double, y float, y__output double"
    assert len(scored.pdf) == 96 and scored.pdf["y__output"].dtype == np.float64
    backend = SparkBackend(num_proc=3, env={"A": "1"})
    assert backend.num_processes() == 3
    with pytest.raises(ImportError, match="pyspark"):
        SparkBackend().num_processes()


def test_epoch_loaders_continue_where_the_last_epoch_stopped(tmp_path):
    from horovod_b200.spark.data_loaders import AsyncParquetDataLoader, ParquetDataLoader
    store = LocalStore(str(tmp_path))
    dataset._write_pandas(store, _frame(10)[["row"]], store.get_train_data_path(), 2)
    plain = ParquetDataLoader(store, store.get_train_data_path(), ["row"], 4, total_rows=10,
                              shuffle=False, to_tensors=lambda b: b["row"].tolist())
    assert len(plain) == 3
    assert list(plain) == [[0, 1, 2, 3], [4, 5, 6, 7], [8, 9, 0, 1]]
    assert list(plain) == [[2, 3, 4, 5], [6, 7, 8, 9], [0, 1, 2, 3]]
    ahead = AsyncParquetDataLoader(store, store.get_train_data_path(), ["row"], 4, total_rows=10,
                                   shuffle=False, limit_step_per_epoch=2,
                                   async_loader_queue_size=2)
    assert [b["row"].tolist() for b in ahead] == [[0, 1, 2, 3], [4, 5, 6, 7]]
    assert [b["row"].tolist() for b in ahead] == [[8, 9, 0, 1], [2, 3, 4, 5]]
    ahead.close_async_loader()
