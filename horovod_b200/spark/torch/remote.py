"""The function an estimator runs on every rank: reads this rank's share of
the prepared Parquet data, trains the model under ``DistributedOptimizer``,
validates, averages the epoch's figures over the ranks, and has rank 0 write
a checkpoint into the store after every epoch. Rank 0 returns the history and
the final checkpoint as bytes.

Covers what horovod/spark/torch/remote.py:37-416 (RemoteTrainer) does for the
reference's estimator; the data comes from ParquetShardReader instead of
Petastorm.
"""
import io
import os


def _as_list(value):
    if value is None:
        return []
    return list(value) if isinstance(value, (list, tuple)) else [value]


def make_trainer(spec):
    """``spec`` holds plain settings only (column names, sizes, the store,
    functions); the model and the optimizer travel as the one argument of the
    returned function, pickled together so that the optimizer still refers to
    the model's parameters after loading."""

    def train(model_and_optimizer_blob):
        import cloudpickle
        import numpy as np
        import torch
        import horovod_b200.torch as hvd
        from horovod_b200.spark.common import dataset

        hvd.init()
        try:
            return _train(spec, model_and_optimizer_blob, cloudpickle, np, torch, hvd, dataset)
        finally:
            hvd.shutdown()

    return train


def _train(spec, blob, cloudpickle, np, torch, hvd, dataset):
    store, run_id = spec["store"], spec["run_id"]
    feature_cols, label_cols = spec["feature_cols"], spec["label_cols"]
    weight_col = spec.get("sample_weight_col")
    metadata = spec["metadata"]
    verbose = spec.get("verbose", 0) if hvd.rank() == 0 else 0
    seed = spec.get("random_seed")
    if seed is not None:
        torch.manual_seed(seed)
        np.random.seed(seed)

    model, optimizer = cloudpickle.loads(blob)
    use_cuda = torch.cuda.is_available() and hvd.cuda_built() and not spec.get("no_cuda")
    device = torch.device("cpu")
    if use_cuda:
        # a GPU that Spark's resource scheduling gave this task, else one per local rank
        from horovod_b200.spark.task import get_available_devices
        assigned = get_available_devices()
        index = int(assigned[0]) if assigned else hvd.local_rank()
        torch.cuda.set_device(index)
        device = torch.device("cuda", index)
        model.to(device)
        for state in optimizer.state.values():
            for key, value in state.items():
                if torch.is_tensor(value):
                    state[key] = value.to(device)

    losses = [make() for make in _as_list(spec.get("loss_constructors"))] or _as_list(spec["loss"])
    if len(losses) == 1 and len(label_cols) > 1:
        losses = losses * len(label_cols)
    if len(losses) != len(label_cols):
        raise ValueError("need one loss per label column: %d losses, %d label columns"
                         % (len(losses), len(label_cols)))
    weights = _as_list(spec.get("loss_weights")) or [1.0 / len(label_cols)] * len(label_cols)
    if len(weights) != len(label_cols):
        raise ValueError("loss_weights needs one entry per label column")
    metrics = _as_list(spec.get("metrics"))
    input_shapes, label_shapes = spec.get("input_shapes"), spec.get("label_shapes")

    hvd.broadcast_parameters(model.state_dict(), root_rank=0)
    hvd.broadcast_optimizer_state(optimizer, root_rank=0)
    compression = spec.get("gradient_compression") or hvd.Compression.none
    optimizer = hvd.DistributedOptimizer(optimizer, named_parameters=model.named_parameters(),
                                         compression=compression)

    columns = list(feature_cols) + list(label_cols) + ([weight_col] if weight_col else [])
    transformation = spec.get("transformation_fn")

    def loader(path, rows, batch, shuffle, limit):
        from horovod_b200.spark.data_loaders import AsyncParquetDataLoader
        return AsyncParquetDataLoader(
            store, path, columns, batch, rows, rank=hvd.rank(), size=hvd.size(), shuffle=shuffle,
            seed=seed or 0, cache=spec.get("inmemory_cache_all", False), transform=transformation,
            limit_step_per_epoch=limit, to_tensors=tensors,
            async_loader_queue_size=spec.get("async_loader_queue_size", 8))

    batch_size = spec["batch_size"]
    val_batch_size = spec.get("val_batch_size") or batch_size
    validate = spec.get("val_rows", 0) > 0

    def from_numpy(array):
        array = np.ascontiguousarray(array)
        return torch.from_numpy(array if array.flags.writeable else array.copy())

    def tensors(batch):
        def feature(i, col):
            t = from_numpy(batch[col]).float()
            if input_shapes:
                t = t.reshape(list(input_shapes[i]))
            elif t.dim() == 1 and metadata[col]["shape"] == ():
                t = t.unsqueeze(1)
            return t.to(device)

        def label(col):
            t = from_numpy(batch[col])
            return (t.float() if t.dtype == torch.float64 else t).to(device)

        sample_weights = from_numpy(batch[weight_col]).float().to(device) if weight_col else None
        return ([feature(i, c) for i, c in enumerate(feature_cols)],
                [label(c) for c in label_cols], sample_weights)

    def transform_outputs(outputs, labels):
        outputs = list(outputs) if isinstance(outputs, (tuple, list)) else [outputs]
        shaped = []
        for i, (output, target) in enumerate(zip(outputs, labels)):
            if label_shapes:
                target = target.reshape(list(label_shapes[i]))
            elif hasattr(output, "shape") and target.numel() == output.numel():
                # same number of values: the label takes the output's shape and type
                target = target.reshape(output.shape).to(output.dtype)
            shaped.append(target)
        return outputs, shaped

    def loss_fn(outputs, labels, sample_weights):
        total = 0
        for output, target, fn, w in zip(outputs, labels, losses, weights):
            value = fn(output, target)
            if sample_weights is not None:
                if value.dim() == 0:
                    raise ValueError("with sample_weight_col the losses must return one value per "
                                     "row (reduction='none')")
                per_row = value.reshape(value.shape[0], -1).mean(dim=1)
                value = (per_row * sample_weights).sum() / sample_weights.sum().clamp_min(1e-12)
            elif value.dim() > 0:
                value = value.mean()
            total = total + w * value
        return total

    def default_minibatch(model, optimizer, transform_outputs, loss_fn, inputs, labels, weights_):
        optimizer.zero_grad()
        outputs, labels = transform_outputs(model(*inputs), labels)
        loss = loss_fn(outputs, labels, weights_)
        loss.backward()
        optimizer.step()
        return outputs, loss

    minibatch = spec.get("train_minibatch_fn") or default_minibatch

    def metric_names():
        return [getattr(m, "__name__", None) or type(m).__name__.lower() for m in metrics]

    def summarize(sums, steps):
        """Mean over the steps of this rank, then over the ranks, in one allreduce."""
        from horovod_b200.parallel.data_parallel import average_metrics
        return average_metrics({k: v / max(steps, 1) for k, v in sums.items()})

    def run_epoch(batches, training):
        sums = {"loss": 0.0}
        sums.update({n: 0.0 for n in metric_names()})
        model.train(training)
        for inputs, labels, sample_weights in batches:
            if training:
                outputs, loss = minibatch(model, optimizer, transform_outputs, loss_fn, inputs,
                                          labels, sample_weights)
                _, labels = transform_outputs(outputs, labels)
            else:
                with torch.no_grad():
                    outputs, labels = transform_outputs(model(*inputs), labels)
                    loss = loss_fn(outputs, labels, sample_weights)
            sums["loss"] += float(loss.detach())
            with torch.no_grad():
                for name, fn in zip(metric_names(), metrics):
                    sums[name] += float(fn(*[o.detach() for o in outputs], *labels)
                                        if len(outputs) > 1 else fn(outputs[0].detach(), labels[0]))
        return summarize(sums, len(batches))

    def checkpoint_bytes():
        buffer = io.BytesIO()
        torch.save({"model": {k: v.cpu() for k, v in model.state_dict().items()},
                    "optimizer": optimizer.state_dict()}, buffer)
        return buffer.getvalue()

    train_batches = loader(spec["train_path"], spec["train_rows"], batch_size,
                           spec.get("shuffle", True), spec.get("train_steps_per_epoch"))
    if validate:
        val_batches = loader(spec["val_path"], spec["val_rows"], val_batch_size, False,
                             spec.get("validation_steps_per_epoch"))
    history = []
    callbacks = _as_list(spec.get("callbacks"))
    scratch = store.get_local_output_dir_fn(run_id)
    try:
        with scratch() as out_dir:
            log_path = os.path.join(out_dir, store.get_logs_subdir(), "history.jsonl")
            os.makedirs(os.path.dirname(log_path), exist_ok=True)
            for epoch in range(spec["epochs"]):
                entry = {"epoch": epoch, "train": run_epoch(train_batches, True)}
                if validate:
                    entry["validation"] = run_epoch(val_batches, False)
                history.append(entry)
                if verbose:
                    print("epoch %d: %s" % (epoch, entry), flush=True)
                for callback in callbacks:
                    callback(epoch, entry, model, optimizer)
                if hvd.rank() == 0 and store.saving_runs():
                    import json
                    with open(os.path.join(out_dir, store.get_checkpoint_filename()), "wb") as f:
                        f.write(checkpoint_bytes())
                    with open(log_path, "a") as f:
                        f.write(json.dumps(entry) + "\n")
                    store.sync_fn(run_id)(out_dir)
            if hvd.rank() == 0:
                return history, checkpoint_bytes()
    finally:
        # an error in the middle of an epoch must not leave a reader thread behind
        train_batches.close_async_loader()
        if validate:
            val_batches.close_async_loader()
    return None
