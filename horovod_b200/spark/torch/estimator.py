"""``TorchEstimator``: fits a PyTorch model to a DataFrame on the ranks of a
backend; ``TorchModel``: the fitted model as a transformer of DataFrames.

    store = Store.create("/mnt/work")
    est = TorchEstimator(num_proc=4, model=net, optimizer=opt, loss=torch.nn.MSELoss(),
                         feature_cols=["features"], label_cols=["y"], input_shapes=[[-1, 8]],
                         batch_size=64, epochs=3, validation=0.1, store=store)
    fitted = est.fit(df)                 # a Spark or a pandas DataFrame
    scored = fitted.transform(df)        # adds the column y__output

``fit`` writes the selected columns as Parquet into the store, runs the
trainer of horovod_b200/spark/torch/remote.py on every rank and loads rank
0's final checkpoint into a copy of the model. ``fit_on_parquet`` trains on
data that is already in the store. Settings are read and changed with
``getX()`` / ``setX(value)`` (``getBatchSize()``, ``setEpochs(5)``, ...), as
with Spark ML parameters; the classes themselves do not depend on pyspark, so
an estimator can also be fitted to a pandas DataFrame through
``LocalBackend``.

Parity: horovod/spark/torch/estimator.py:91-327 (TorchEstimator), :329-470
(TorchModel); horovod/spark/common/estimator.py:25-110 (fit / fit_on_parquet
/ transform); horovod/spark/common/params.py (parameter names).
"""
import copy
import io
import re
import time

from horovod_b200.spark.common import dataset
from horovod_b200.spark.common.backend import SparkBackend


class _Settings:
    """Named settings with generated ``getSomeName`` / ``setSomeName``."""

    _defaults = {}

    def __init__(self, **given):
        unknown = sorted(set(given) - set(self._defaults))
        if unknown:
            raise TypeError("%s got unexpected settings %s" % (type(self).__name__, unknown))
        self._values = dict(self._defaults)
        self._values.update(given)

    def setParams(self, **given):
        unknown = sorted(set(given) - set(self._defaults))
        if unknown:
            raise TypeError("%s has no settings %s" % (type(self).__name__, unknown))
        self._values.update(given)
        return self

    def __getattr__(self, name):
        match = re.fullmatch(r"(get|set)([A-Z]\w*)", name)
        if match and "_values" in self.__dict__:
            key = re.sub(r"(?<!^)(?=[A-Z])", "_", match.group(2)).lower()
            if key in self._defaults:
                if match.group(1) == "get":
                    return lambda: self._values[key]

                def setter(value):
                    self._values[key] = value
                    return self
                return setter
        raise AttributeError("%s has no attribute %r" % (type(self).__name__, name))


class TorchEstimator(_Settings):
    _defaults = dict(
        num_proc=None, model=None, backend=None, store=None, optimizer=None, loss=None,
        loss_constructors=None, metrics=None, loss_weights=None, sample_weight_col=None,
        gradient_compression=None, feature_cols=None, input_shapes=None, validation=None,
        label_cols=None, label_shapes=None, callbacks=None, batch_size=32, val_batch_size=None,
        epochs=1, verbose=1, shuffle=True, partitions_per_process=10, run_id=None,
        train_minibatch_fn=None, train_steps_per_epoch=None, validation_steps_per_epoch=None,
        transformation_fn=None, inmemory_cache_all=False, async_loader_queue_size=8,
        random_seed=None, no_cuda=False)

    def __init__(self, **settings):
        super().__init__(**settings)
        if self._values["num_proc"] is not None and self._values["backend"] is not None:
            raise ValueError("give either num_proc or backend, not both")

    # ---- checks ---------------------------------------------------------------
    def _backend(self):
        return self._values["backend"] or SparkBackend(self._values["num_proc"],
                                                      verbose=self._values["verbose"])

    def _check(self):
        v = self._values
        for needed in ("model", "optimizer", "store", "feature_cols", "label_cols"):
            if not v[needed]:
                raise ValueError("TorchEstimator needs %s" % needed)
        if not v["loss"] and not v["loss_constructors"]:
            raise ValueError("TorchEstimator needs loss or loss_constructors")
        if v["sample_weight_col"]:
            for fn in (v["loss"] if isinstance(v["loss"], (list, tuple)) else [v["loss"]]):
                if getattr(fn, "reduction", "none") != "none":
                    raise ValueError("with sample_weight_col the losses must return one value per "
                                     "row (reduction='none'); %r averages over the batch" % (fn,))
        if v["input_shapes"] and len(v["input_shapes"]) != len(v["feature_cols"]):
            raise ValueError("input_shapes needs one shape per feature column")
        if v["label_shapes"] and len(v["label_shapes"]) != len(v["label_cols"]):
            raise ValueError("label_shapes needs one shape per label column")

    def _check_metadata(self, metadata):
        """The shapes asked for must hold exactly the values a row has."""
        v = self._values
        if not v["input_shapes"]:
            return
        for col, shape in zip(v["feature_cols"], v["input_shapes"]):
            per_row = 1
            for d in metadata[col]["shape"]:
                per_row *= d
            wanted = 1
            for d in list(shape)[1:] if list(shape)[0] == -1 else list(shape):
                wanted *= d
            if list(shape)[0] == -1 and wanted != per_row:
                raise ValueError("feature column %r has %d values per row, input shape %s needs %d"
                                 % (col, per_row, list(shape), wanted))

    # ---- fitting ----------------------------------------------------------------
    def fit(self, df, params=None):
        """Trains on ``df``; ``params`` (a dict) overrides settings for this
        call only. Returns a TorchModel."""
        if params:
            return copy.copy(self)._with(params).fit(df)
        self._check()
        v = self._values
        backend = self._backend()
        with dataset.prepare_data(backend.num_processes(), v["store"], df,
                                  label_columns=v["label_cols"], feature_columns=v["feature_cols"],
                                  validation=v["validation"],
                                  sample_weight_col=v["sample_weight_col"],
                                  partitions_per_process=v["partitions_per_process"],
                                  seed=v["random_seed"] or 0,
                                  verbose=v["verbose"]) as (train_rows, val_rows, metadata, _size):
            return self._fit_on_prepared_data(backend, train_rows, val_rows, metadata)

    def _with(self, params):
        self._values = dict(self._values)
        return self.setParams(**params)

    def fit_on_parquet(self, params=None, dataset_idx=None):
        """Trains on the Parquet data already at the store's train (and
        validation) path."""
        if params:
            return copy.copy(self)._with(params).fit_on_parquet(dataset_idx=dataset_idx)
        self._check()
        v = self._values
        store = v["store"]
        columns = list(v["feature_cols"]) + list(v["label_cols"]) + \
            ([v["sample_weight_col"]] if v["sample_weight_col"] else [])
        train_rows, metadata, _ = dataset.read_metadata(
            store, store.get_train_data_path(dataset_idx), columns)
        val_rows = 0
        val_path = store.get_val_data_path(dataset_idx)
        if dataset.dataset_exists(store, val_path):
            val_rows = dataset.read_metadata(store, val_path, columns)[0]
        return self._fit_on_prepared_data(self._backend(), train_rows, val_rows, metadata,
                                          dataset_idx)

    def _fit_on_prepared_data(self, backend, train_rows, val_rows, metadata, dataset_idx=None):
        import cloudpickle
        from horovod_b200.spark.torch.remote import make_trainer
        self._check_metadata(metadata)
        v = self._values
        store = v["store"]
        run_id = v["run_id"] or "pytorch_%d" % int(time.time() * 1000)
        spec = {k: v[k] for k in (
            "store", "feature_cols", "label_cols", "sample_weight_col", "loss",
            "loss_constructors", "loss_weights", "metrics", "input_shapes", "label_shapes",
            "gradient_compression", "batch_size", "val_batch_size", "epochs", "verbose",
            "shuffle", "train_minibatch_fn", "train_steps_per_epoch",
            "validation_steps_per_epoch", "transformation_fn", "inmemory_cache_all",
            "random_seed", "callbacks", "no_cuda", "async_loader_queue_size")}
        spec.update(run_id=run_id, metadata=metadata, train_rows=train_rows, val_rows=val_rows,
                    train_path=store.get_train_data_path(dataset_idx),
                    val_path=store.get_val_data_path(dataset_idx))
        blob = cloudpickle.dumps((v["model"], v["optimizer"]))
        results = backend.run(make_trainer(spec), args=(blob,))
        history, checkpoint = results[0]
        return self._create_model(history, checkpoint, run_id, metadata)

    def _create_model(self, history, checkpoint, run_id, metadata):
        import cloudpickle
        import torch
        v = self._values
        # a copy of both, still tied to each other, with the trained state loaded
        model, optimizer = cloudpickle.loads(cloudpickle.dumps((v["model"], v["optimizer"])))
        state = torch.load(io.BytesIO(checkpoint), map_location="cpu", weights_only=False)
        model.load_state_dict(state["model"])
        optimizer.load_state_dict(state["optimizer"])
        return TorchModel(history=history, model=model, feature_columns=v["feature_cols"],
                          input_shapes=v["input_shapes"], label_columns=v["label_cols"],
                          optimizer=optimizer, run_id=run_id, _metadata=metadata,
                          loss=v["loss"], loss_constructors=v["loss_constructors"])

    def _load_checkpoint(self, run_id):
        """The model state rank 0 last wrote into the store for ``run_id``."""
        import torch
        store = self._values["store"]
        data = store.read(store.get_checkpoint_path(run_id))
        return torch.load(io.BytesIO(data), map_location="cpu", weights_only=False)


class TorchModel(_Settings):
    _defaults = dict(history=None, model=None, feature_columns=None, input_shapes=None,
                     label_columns=None, optimizer=None, run_id=None, _metadata=None, loss=None,
                     loss_constructors=None, output_cols=None, batch_size=1024)

    def __init__(self, **settings):
        super().__init__(**settings)
        if self._values["output_cols"] is None and self._values["label_columns"]:
            self._values["output_cols"] = [c + "__output" for c in self._values["label_columns"]]

    def getFeatureColumns(self):
        return self._values["feature_columns"]

    def getLabelColumns(self):
        return self._values["label_columns"]

    # ---- prediction ---------------------------------------------------------------
    def _predict_pandas(self, pdf, model=None):
        v = self._values
        return _predict(pdf, model or v["model"], v["feature_columns"], v["input_shapes"],
                        v["output_cols"], v["batch_size"])

    def transform(self, df, params=None):
        """Returns ``df`` with one prediction column per label column
        (``<label>__output``): a number when the model emits one value per
        row, else an array."""
        if params:
            return copy.copy(self)._with(params).transform(df)
        if dataset._is_pandas(df):
            return self._predict_pandas(df)
        import cloudpickle
        v = self._values
        blob = cloudpickle.dumps(v["model"])
        sample = self._predict_pandas(df.limit(1).toPandas())
        kinds = []
        for name in v["output_cols"]:
            first = sample[name].iloc[0] if len(sample) else 0.0
            kinds.append("%s %s" % (name, "array<double>" if hasattr(first, "__len__") else "double"))
        schema = ", ".join(["%s %s" % (f.name, f.dataType.simpleString())
                            for f in df.schema.fields] + kinds)
        # only what scoring needs travels to the executors
        features, shapes = v["feature_columns"], v["input_shapes"]
        outputs, batch = v["output_cols"], v["batch_size"]

        def score(frames):
            model = cloudpickle.loads(blob)
            for pdf in frames:
                scored = _predict(pdf, model, features, shapes, outputs, batch)
                for name in outputs:
                    scored[name] = [x.astype("float64").tolist() if hasattr(x, "__len__")
                                    else float(x) for x in scored[name]]
                yield scored
        return df.mapInPandas(score, schema=schema)

    def _with(self, params):
        self._values = dict(self._values)
        return self.setParams(**params)

    # ---- persistence ----------------------------------------------------------------
    def save(self, path):
        import cloudpickle
        with open(path, "wb") as f:
            cloudpickle.dump(self._values, f)

    @classmethod
    def load(cls, path):
        import cloudpickle
        with open(path, "rb") as f:
            return cls(**cloudpickle.load(f))


def _predict(pdf, model, feature_columns, input_shapes, output_cols, batch_size):
    """``pdf`` plus the model's outputs as new columns, computed in batches."""
    import numpy as np
    import torch
    model.eval()
    outputs = [[] for _ in output_cols]
    for start in range(0, len(pdf), batch_size):
        part = pdf.iloc[start:start + batch_size]
        inputs = []
        for i, col in enumerate(feature_columns):
            values = part[col].to_numpy()
            if values.dtype == object:
                values = np.stack([np.asarray(x) for x in values])
            t = torch.tensor(np.asarray(values), dtype=torch.float32)
            if input_shapes:
                t = t.reshape(list(input_shapes[i]))
            elif t.dim() == 1:
                t = t.unsqueeze(1)
            inputs.append(t)
        with torch.no_grad():
            result = model(*inputs)
        result = list(result) if isinstance(result, (tuple, list)) else [result]
        for sink, value in zip(outputs, result):
            sink.append(value.reshape(len(part), -1).cpu().numpy())
    scored = pdf.copy()
    for name, chunks in zip(output_cols, outputs):
        joined = np.concatenate(chunks) if chunks else np.zeros((0, 1), dtype=np.float32)
        scored[name] = joined[:, 0] if joined.shape[1] == 1 else list(joined)
    return scored
