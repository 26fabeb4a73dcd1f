"""Flagship benchmark: ResNet-50 v1.5 synthetic training throughput with
hvd.DistributedOptimizer (per-GPU batch 256, bf16 autocast, fp32 master
weights, SGD momentum 0.9 + weight decay 1e-4), one rank per GPU.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 \
        --master-addr 127.0.0.1 --master-port 29500 bench.py --gpus 8

Protocol follows the reference's synthetic benchmark
(examples/pytorch/pytorch_synthetic_benchmark.py:59-118: fixed random batch,
DistributedOptimizer, broadcast of parameters and optimizer state, warm-up
then timed steps) with device timing: CUDA events around exactly K steps,
barrier + synchronize on both sides, maximum over ranks. A second timed pass
measures the same steps end to end (pinned-host input copy and loss read-back
every step). Rank 0 prints one JSON line.

Other models: --model bert-large | gpt2-medium (the other training configs).
Unless --secondary 0 is given, the BERT-large configuration is measured in the
same job after the flagship and reported under "secondary" in the same line.

With more than one rank the line also carries correctness evidence:
"collective_checks" (one allreduce per algorithm, reducescatter, allgather,
broadcast and alltoall against fp64 sums computed from every rank's seeded
inputs, before the timed region), "params_in_sync" (fp64 checksums of every
parameter after the timed steps, equal on all ranks) and "loss_vs_single" (a
small language model trained for a few steps on rank-specific batches through
the same gradient path, against plain SGD on the concatenated batch in one
process). Any mismatch makes the exit code non-zero. "allreduce_bus" is the
bus bandwidth of a 256 MB fp32 allreduce (in place on the symmetric heap and
staged), the third metric of record.

--impl ddp runs the same model, batch and autocast through
torch.nn.parallel.DistributedDataParallel over NCCL: an independent arm for
context (none of this library's engine on its path). --impl reference is the
reference itself, which cannot be built offline here.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import time

os.environ.setdefault("HOROVOD_FORCE_HOOKS", "1")  # same gradient path at N=1


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=20)
    p.add_argument("--warmup", type=int, default=5)
    p.add_argument("--impl", default="ours", choices=["ours", "reference", "ddp"])
    p.add_argument("--secondary", type=int, default=1,
                   help="1: also measure BERT-large after the flagship model")
    p.add_argument("--model", default="resnet50",
                   choices=["resnet50", "bert-large", "gpt2-medium"])
    p.add_argument("--batch", type=int, default=0, help="per-GPU batch (0 = config default)")
    p.add_argument("--backend", default=None, help="symm | nccl (HOROVOD_GPU_BACKEND)")
    p.add_argument("--fused-optimizer", type=int, default=1,
                   help="1: ResNet uses hvd.FusedSGD (same arithmetic as torch.optim.SGD)")
    p.add_argument("--symmetric-gradients", type=int, default=1,
                   help="1: gradients live in the symmetric heap and are reduced in place")
    return p.parse_args()


REFERENCE_UNAVAILABLE = (
    "reference (uber/horovod 0.22.1) does not build offline here: pip install "
    "--no-index of the source tree fails in CMake (cmake_minimum_required < 3.5 "
    "rejected by the installed CMake; third_party submodules are empty; torch "
    "binding includes THC/THC.h, absent from torch 2.11)")


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled during the timed region."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index):
        self.device_index = device_index
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.device_index), "--query-gpu=" + self.QUERY,
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, smax, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                smax = float(f[2])
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": smax,
                "reasons": sorted(reasons), "samples": len(sm)}


def build_workload(args, torch, device):
    from horovod_b200 import models
    if args.model == "resnet50":
        batch = args.batch or 256
        model = models.resnet50().to(device).to(memory_format=torch.channels_last)
        if getattr(args, "fused_optimizer", 0) and args.impl == "ours":
            from horovod_b200.torch.fused_sgd import FusedSGD
            opt = FusedSGD(model.parameters(), lr=0.01, momentum=0.9, weight_decay=1e-4)
        else:
            opt = torch.optim.SGD(model.parameters(), lr=0.01, momentum=0.9, weight_decay=1e-4)
        g = torch.Generator().manual_seed(1)
        # fp32 images in channels-last layout in pinned memory: the copy to the
        # device lands in the layout the model runs in, no conversion pass.
        host_x = [torch.randn(batch, 3, 224, 224, generator=g)
                  .contiguous(memory_format=torch.channels_last).pin_memory() for _ in range(2)]
        host_y = [torch.randint(0, 1000, (batch,), generator=g).pin_memory() for _ in range(2)]

        def to_dev(x):
            return x.to(device, non_blocking=True).contiguous(memory_format=torch.channels_last)

        def loss_fn(x, y):
            return torch.nn.functional.cross_entropy(model(x), y)
        cfg = {"model": "ResNet-50 v1.5", "global_batch": batch * args.gpus, "seq_len": None,
               "optimizer": "SGD momentum 0.9 wd 1e-4, fp32 master weights (%s)"
                            % ("hvd.FusedSGD: torch.optim.SGD arithmetic in one launch"
                               if isinstance(opt, torch.optim.Optimizer) and
                               type(opt).__name__ == "FusedSGD" else "torch.optim.SGD"),
               "memory_format": "channels_last"}
        metric, unit = "resnet50_train_images_per_sec", "images/s"
        return model, opt, host_x, host_y, to_dev, loss_fn, batch, cfg, metric, unit
    if args.model == "bert-large":
        batch, seq, vocab = args.batch or 32, 512, 30522
        model = models.bert_large().to(device)
        opt = torch.optim.Adam(model.parameters(), lr=1e-4, betas=(0.9, 0.999))
    else:
        batch, seq, vocab = args.batch or 8, 1024, 50257
        model = models.gpt2_medium().to(device)
        opt = torch.optim.Adam(model.parameters(), lr=1e-4)
    g = torch.Generator().manual_seed(1)
    host_x = [torch.randint(0, vocab, (batch, seq), generator=g).pin_memory() for _ in range(2)]
    if args.model == "bert-large":
        host_y = []
        for x in host_x:
            y = x.clone()
            keep = torch.rand(x.shape, generator=g) < 0.15
            y[~keep] = -100  # only the 15% masked positions are scored
            host_y.append(y.pin_memory())
    else:
        host_y = [torch.roll(x, -1, 1).pin_memory() for x in host_x]

    def to_dev(x):
        return x.to(device, non_blocking=True)

    def loss_fn(x, y):
        logits = model(x)
        return torch.nn.functional.cross_entropy(logits.view(-1, logits.size(-1)).float(),
                                                 y.view(-1), ignore_index=-100)
    cfg = {"model": "BERT-large MLM" if args.model == "bert-large" else "GPT-2 medium",
           "global_batch": batch * args.gpus, "seq_len": seq}
    metric = ("bert_large_train_sequences_per_sec" if args.model == "bert-large"
              else "gpt2_medium_train_sequences_per_sec")
    return model, opt, host_x, host_y, to_dev, loss_fn, batch, cfg, metric, "sequences/s"


def _seeded(seed, n, dtype, torch):
    g = torch.Generator().manual_seed(seed)
    if dtype.is_floating_point:
        return torch.randn(n, generator=g, dtype=torch.float32).to(dtype)
    return torch.randint(-50, 50, (n,), generator=g).to(dtype)


def collective_checks(hvd, torch, device):
    """One collective per kernel family and algorithm, compared with fp64
    results computed from every rank's seeded inputs. Returns (passed, failed
    descriptions); identical on all ranks."""
    n, rank = hvd.size(), hvd.rank()
    failed, passed = [], 0

    def check(name, ok):
        nonlocal passed
        if ok:
            passed += 1
        else:
            failed.append(name)

    # allreduce: small (one-shot), large fp32/bf16 (two-shot or NVLS), int32
    # (always peer loads/stores), and in place on the symmetric heap
    for label, dtype, count, tol in (("oneshot_fp32_64KB", torch.float32, 16 << 10, 1e-5),
                                     ("large_fp32_8MB", torch.float32, (2 << 20) + 3, 1e-5),
                                     ("large_bf16_8MB", torch.bfloat16, (4 << 20) + 1, 4e-2),
                                     ("twoshot_int32_4MB", torch.int32, (1 << 20) + 7, 0)):
        x = _seeded(100 + rank, count, dtype, torch).to(device)
        out = hvd.allreduce(x, op=hvd.Sum, name="check.ar." + label)
        ref = sum(_seeded(100 + r, count, dtype, torch).double() for r in range(n))
        err = (out.double().cpu() - ref).abs().max().item()
        check("allreduce_" + label, err <= tol * n * max(1.0, ref.abs().max().item()))
    if hvd.gpu_backend().startswith("symm"):
        count = (3 << 20) + 64
        heap = hvd.symmetric_empty(count)
        heap.copy_(_seeded(200 + rank, count, torch.float32, torch))
        hvd.allreduce_(heap, op=hvd.Average, name="check.ar.inplace")
        ref = sum(_seeded(200 + r, count, torch.float32, torch).double() for r in range(n)) / n
        check("allreduce_inplace_symmetric_12MB",
              (heap.double().cpu() - ref).abs().max().item() <= 1e-5 * max(1.0, ref.abs().max().item()))
    # reducescatter, ragged rows
    rows = 4 * n + 3
    x = _seeded(300 + rank, rows * 1000, torch.float32, torch).view(rows, 1000).to(device)
    out = hvd.reducescatter(x, op=hvd.Sum, name="check.rs")
    ref = sum(_seeded(300 + r, rows * 1000, torch.float32, torch).view(rows, 1000).double()
              for r in range(n))
    base, extra = rows // n, rows % n
    lo = rank * base + min(rank, extra)
    hi = lo + base + (1 if rank < extra else 0)
    check("reducescatter_ragged", tuple(out.shape) == (hi - lo, 1000) and
          (out.double().cpu() - ref[lo:hi]).abs().max().item() <= 1e-5 * n * 10)
    # allgather with a different dim 0 on every rank, small and large
    for label, width in (("small", 3), ("large", 1 << 19)):
        x = _seeded(400 + rank, (rank + 1) * width, torch.float32, torch).view(rank + 1, width)
        out = hvd.allgather(x.to(device), name="check.ag." + label)
        ref = torch.cat([_seeded(400 + r, (r + 1) * width, torch.float32, torch).view(r + 1, width)
                         for r in range(n)])
        check("allgather_" + label, torch.equal(out.cpu(), ref))
    # broadcast from the last rank, small and large
    for label, count in (("small", 1001), ("large", (5 << 20) + 1)):
        x = _seeded(500 + rank, count, torch.float32, torch).to(device)
        hvd.broadcast_(x, root_rank=n - 1, name="check.bc." + label)
        check("broadcast_" + label, torch.equal(x.cpu(), _seeded(500 + n - 1, count,
                                                                 torch.float32, torch)))
    # alltoall with uneven splits: rank r sends (r + p) % 3 + 1 rows to rank p
    width = 1 << 16
    splits = torch.tensor([(rank + p) % 3 + 1 for p in range(n)], dtype=torch.int32)
    send = _seeded(600 + rank, int(splits.sum()) * width, torch.float32, torch).view(-1, width)
    recv, rsplits = hvd.alltoall(send.to(device), splits=splits, name="check.a2a")
    pieces = []
    for r in range(n):
        sp = [(r + p) % 3 + 1 for p in range(n)]
        full = _seeded(600 + r, sum(sp) * width, torch.float32, torch).view(-1, width)
        pieces.append(full[sum(sp[:rank]):sum(sp[:rank]) + sp[rank]])
    check("alltoall_uneven", torch.equal(recv.cpu(), torch.cat(pieces)))
    # alltoall without splits (even split; no split table is exchanged): rank r
    # holds n * (r + 1) rows and sends r + 1 of them to every peer
    width = 1024
    send = _seeded(800 + rank, n * (rank + 1) * width, torch.float32, torch) \
        .view(n * (rank + 1), width)
    recv = hvd.alltoall(send.to(device), name="check.a2a.even")
    pieces = [_seeded(800 + r, n * (r + 1) * width, torch.float32, torch)
              .view(n * (r + 1), width)[rank * (r + 1):(rank + 1) * (r + 1)] for r in range(n)]
    check("alltoall_even", torch.equal(recv.cpu(), torch.cat(pieces)))
    # every rank must agree on the verdict
    mine = torch.tensor([float(len(failed))])
    worst = float(hvd.allreduce(mine, op=hvd.Max, name="check.verdict"))
    if worst > 0 and not failed:
        failed.append("a check failed on another rank")
    return passed, failed


def allreduce_bus_bandwidth(hvd, torch, device, nbytes=256 << 20, reps=5):
    """Bus bandwidth of one large fp32 allreduce, the third metric of record:
    in place on the symmetric heap (the path of the ResNet gradients) and
    staged from ordinary memory (the path of every other tensor). Timed with
    CUDA events on the caller's stream, which waits for the op, so the host
    launch path is inside the figure; max over ranks. bus = 2 (N-1)/N S / t."""
    import statistics
    import time
    n = hvd.size()
    count = nbytes // 4
    on_gpu = device.type == "cuda"

    def timed(x, name):
        for _ in range(3):
            hvd.allreduce_(x, op=hvd.Average, name=name)
        samples = []
        for _ in range(reps):
            if on_gpu:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                hvd.allreduce_(x, op=hvd.Average, name=name)
                e1.record()
                e1.synchronize()
                samples.append(e0.elapsed_time(e1) * 1e3)
            else:
                t0 = time.perf_counter()
                hvd.allreduce_(x, op=hvd.Average, name=name)
                samples.append((time.perf_counter() - t0) * 1e6)
        us = float(hvd.allreduce(torch.tensor([statistics.median(samples)], dtype=torch.float64),
                                 op=hvd.Max, name=name + ".us"))
        return {"us": round(us, 1),
                "bus_gbs": round(nbytes * 2.0 * (n - 1) / n / (us * 1e-6) / 1e9, 1)}

    out = {"bytes": nbytes, "dtype": "fp32", "n_gpus": n,
           "formula": "2 (N-1)/N x bytes / time, time = median of %d, max over ranks" % reps}
    staged = torch.ones(count, device=device)
    out["staged"] = timed(staged, "bus.staged")
    if hvd.gpu_backend().startswith("symm"):
        heap = hvd.symmetric_empty(count)
        heap.fill_(1.0)
        out["in_place_on_symmetric_heap"] = timed(heap, "bus.inplace")
    return out


def params_in_sync(hvd, torch, model):
    """fp64 sum and abs-sum of every parameter, gathered from all ranks and
    compared: after synchronous data-parallel steps they must be identical."""
    sums = torch.stack([torch.stack([p.detach().double().sum(), p.detach().double().abs().sum()])
                        for p in model.parameters()]).cpu()
    every = hvd.allgather(sums.unsqueeze(0), name="bench.param_checksums")
    return bool((every == every[0:1]).all().item()), int(sums.shape[0])


def loss_vs_single(hvd, torch, device, symmetric):
    """Trains a small causal LM (fp32, no dropout) for 5 SGD steps through
    hvd.DistributedOptimizer on rank-specific batches, and the same model with
    plain SGD on the concatenated batch in this process alone; equal batch
    sizes make the averaged gradient equal to the gradient of the concatenated
    batch. Returns the largest relative difference of the per-step losses
    (of the global mean loss)."""
    from horovod_b200 import models
    n, rank = hvd.size(), hvd.rank()
    vocab, seq, per_rank = 512, 64, 4

    def make():
        torch.manual_seed(1234)
        return models.TransformerLM(vocab, seq, 128, 2, 4, 512, causal=True).to(device)

    def batch(r):
        g = torch.Generator().manual_seed(7000 + r)
        return torch.randint(0, vocab, (per_rank, seq), generator=g)

    def loss_of(model, x):
        logits = model(x)
        return torch.nn.functional.cross_entropy(
            logits[:, :-1].reshape(-1, vocab), x[:, 1:].reshape(-1))

    dist_model, single = make(), make()
    opt = hvd.DistributedOptimizer(
        torch.optim.SGD(dist_model.parameters(), lr=0.1, momentum=0.9),
        named_parameters=[("check." + k, v) for k, v in dist_model.named_parameters()],
        symmetric_gradients=symmetric)
    ref_opt = torch.optim.SGD(single.parameters(), lr=0.1, momentum=0.9)
    mine = batch(rank).to(device)
    everything = torch.cat([batch(r) for r in range(n)]).to(device)
    worst = 0.0
    for _ in range(5):
        opt.zero_grad()
        loss = loss_of(dist_model, mine)
        loss.backward()
        opt.step()
        global_loss = float(hvd.allreduce(loss.detach().double().cpu().view(1), op=hvd.Average,
                                          name="check.loss"))
        ref_opt.zero_grad()
        ref = loss_of(single, everything)
        ref.backward()
        ref_opt.step()
        worst = max(worst, abs(global_loss - float(ref.detach())) / max(1e-12, abs(float(ref.detach()))))
    worst = float(hvd.allreduce(torch.tensor([worst], dtype=torch.float64), op=hvd.Max,
                                name="check.loss.worst"))
    return worst


def measure(args, model_name, hvd, torch, device, _C):
    """Device-timed and end-to-end throughput of one model configuration.
    Returns the fields of the JSON line (rank 0) or None (other ranks)."""
    margs = argparse.Namespace(**vars(args))
    margs.model = model_name
    if model_name != args.model:
        margs.batch = 0
    torch.manual_seed(0)
    (model, base_opt, host_x, host_y, to_dev, loss_fn, batch, cfg, metric,
     unit) = build_workload(margs, torch, device)
    symmetric = False
    if model_name == "resnet50":
        symmetric = bool(args.symmetric_gradients)
        opt = hvd.DistributedOptimizer(base_opt, named_parameters=model.named_parameters(),
                                       symmetric_gradients=symmetric)
    elif model_name == "bert-large":
        opt = hvd.DistributedOptimizer(base_opt, named_parameters=model.named_parameters(),
                                       compression=hvd.Compression.fp16)
    else:
        opt = hvd.DistributedOptimizer(base_opt, named_parameters=model.named_parameters(),
                                       op=hvd.Adasum if hvd.size() > 1 else hvd.Average)
    hvd.broadcast_parameters(model.state_dict(), root_rank=0)
    hvd.broadcast_optimizer_state(opt, root_rank=0)

    dev_x, dev_y = to_dev(host_x[0]), host_y[0].to(device)

    def step(x, y):
        opt.zero_grad()
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = loss_fn(x, y)
        loss.backward()
        opt.step()
        return loss

    def barrier():
        hvd.allreduce(torch.zeros(1), name="bench.barrier")
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step(dev_x, dev_y)
    barrier()

    # ---- device-timed pass (inputs resident, larger than L2) -----------------
    sampler = ClockSampler(hvd.local_rank())
    if hvd.rank() == 0:
        sampler.start()
    launches0 = _C.kernel_launch_count()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    # With HOROVOD_BENCH_CUPROFILE=1 the timed steps are bracketed by
    # cudaProfilerStart/Stop, so that `ncu --profile-from-start off` lists
    # the launches of exactly this region (numbers from such a run are not
    # bench values).
    cuprofile = os.environ.get("HOROVOD_BENCH_CUPROFILE") == "1"
    if cuprofile:
        torch.cuda.profiler.start()
    start.record()
    for _ in range(args.steps):
        step(dev_x, dev_y)
    end.record()
    torch.cuda.synchronize()
    if cuprofile:
        torch.cuda.profiler.stop()
    launches = _C.kernel_launch_count() - launches0
    clocks = sampler.stop() if hvd.rank() == 0 else None
    barrier()
    ms = start.elapsed_time(end)
    ms = float(hvd.allreduce(torch.tensor([ms], dtype=torch.float64), op=hvd.Max,
                             name="bench.ms"))

    # ---- end-to-end pass: H2D of the inputs and D2H of the loss every step ---
    copy_stream = torch.cuda.Stream()
    loss_host = torch.zeros(1, pin_memory=True)
    h2d = host_x[0].numel() * host_x[0].element_size() + host_y[0].numel() * host_y[0].element_size()
    barrier()
    t_start, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    wall0 = time.perf_counter()
    t_start.record()
    with torch.cuda.stream(copy_stream):
        nx, ny = to_dev(host_x[0]), host_y[0].to(device, non_blocking=True)
    for i in range(args.steps):
        torch.cuda.current_stream().wait_stream(copy_stream)
        x, y = nx, ny
        x.record_stream(torch.cuda.current_stream())
        y.record_stream(torch.cuda.current_stream())
        if i + 1 < args.steps:  # prefetch the next batch while this one trains
            with torch.cuda.stream(copy_stream):
                j = (i + 1) % len(host_x)
                nx, ny = to_dev(host_x[j]), host_y[j].to(device, non_blocking=True)
        loss = step(x, y)
        loss_host.copy_(loss.detach().float().view(1), non_blocking=True)
    t_end.record()
    torch.cuda.synchronize()
    e2e_ms = max(t_start.elapsed_time(t_end), (time.perf_counter() - wall0) * 1e3)
    e2e_ms = float(hvd.allreduce(torch.tensor([e2e_ms], dtype=torch.float64), op=hvd.Max,
                                 name="bench.e2e_ms"))

    n_param_bytes = sum(p.numel() * p.element_size() for p in model.parameters())
    in_sync, n_params = (True, 0)
    if hvd.size() > 1:
        in_sync, n_params = params_in_sync(hvd, torch, model)
    params = hvd.runtime_params()
    out = None
    if hvd.rank() == 0:
        total = batch * args.gpus * args.steps
        value = total / (ms / 1e3)
        cfg.update({"parallelism": "dp%d" % args.gpus, "per_gpu_batch": batch,
                    "l2": "working set larger than L2: %.0f MB of inputs per step plus "
                          "activations and %.0f MB of parameters"
                          % (h2d / 1e6, n_param_bytes / 1e6),
                    "data_per_rank": "the same batch on every rank, so the loss after K steps "
                                     "must not depend on the number of GPUs",
                    "gradient_path": hvd.gpu_backend(),
                    "symmetric_gradients": bool(symmetric and args.gpus > 1),
                    "fusion_threshold_mb": params["fusion_threshold_bytes"] / float(1 << 20),
                    "cycle_time_ms": params["cycle_time_ms"]})
        out = {
            "metric": metric, "value": round(value, 2), "unit": unit,
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(ms / args.steps, 3), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "impl": "ours", "config": cfg, "clocks": clocks,
            "e2e": {"value": round(total / (e2e_ms / 1e3), 2), "unit": unit,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4},
            "gpu_launches": int(launches),
            "final_loss": float(loss_host.item()),
        }
        if hvd.size() > 1:
            out["params_in_sync"] = in_sync
            out["params_checked"] = n_params
    # Let go of the model before the next one is built.
    del model, opt, base_opt, dev_x, dev_y
    torch.cuda.empty_cache()
    return out, in_sync


def main_ddp(args):
    """The same workload through torch DistributedDataParallel over NCCL."""
    import torch
    import torch.distributed as dist
    from torch.nn.parallel import DistributedDataParallel as DDP
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29511")
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit("--gpus %d but the job has %d ranks" % (args.gpus, world))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    torch.manual_seed(0)
    torch.backends.cudnn.benchmark = True
    (model, opt, host_x, host_y, to_dev, loss_fn, batch, cfg, metric,
     unit) = build_workload(args, torch, device)
    ddp = DDP(model, device_ids=[local], gradient_as_bucket_view=True, bucket_cap_mb=128)
    if args.model == "bert-large":
        from torch.distributed.algorithms.ddp_comm_hooks import default_hooks
        ddp.register_comm_hook(None, default_hooks.fp16_compress_hook)
    # The forward goes through the wrapper (it arms the gradient hooks).

    def step(x, y):
        opt.zero_grad()
        with torch.autocast("cuda", dtype=torch.bfloat16):
            out = ddp(x)
            if args.model == "resnet50":
                loss = torch.nn.functional.cross_entropy(out, y)
            else:
                loss = torch.nn.functional.cross_entropy(
                    out.view(-1, out.size(-1)).float(), y.view(-1), ignore_index=-100)
        loss.backward()
        opt.step()
        return loss

    def barrier():
        dist.barrier()
        torch.cuda.synchronize()

    def allmax(v):
        t = torch.tensor([v], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    dev_x, dev_y = to_dev(host_x[0]), host_y[0].to(device)
    for _ in range(args.warmup):
        step(dev_x, dev_y)
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(args.steps):
        step(dev_x, dev_y)
    end.record()
    torch.cuda.synchronize()
    clocks = sampler.stop() if rank == 0 else None
    barrier()
    ms = allmax(start.elapsed_time(end))

    copy_stream = torch.cuda.Stream()
    loss_host = torch.zeros(1, pin_memory=True)
    h2d = host_x[0].numel() * host_x[0].element_size() + host_y[0].numel() * host_y[0].element_size()
    barrier()
    t_start, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    wall0 = time.perf_counter()
    t_start.record()
    with torch.cuda.stream(copy_stream):
        nx, ny = to_dev(host_x[0]), host_y[0].to(device, non_blocking=True)
    for i in range(args.steps):
        torch.cuda.current_stream().wait_stream(copy_stream)
        x, y = nx, ny
        x.record_stream(torch.cuda.current_stream())
        y.record_stream(torch.cuda.current_stream())
        if i + 1 < args.steps:
            with torch.cuda.stream(copy_stream):
                j = (i + 1) % len(host_x)
                nx, ny = to_dev(host_x[j]), host_y[j].to(device, non_blocking=True)
        loss = step(x, y)
        loss_host.copy_(loss.detach().float().view(1), non_blocking=True)
    t_end.record()
    torch.cuda.synchronize()
    e2e_ms = allmax(max(t_start.elapsed_time(t_end), (time.perf_counter() - wall0) * 1e3))
    bus = None
    if world > 1:
        # The same figure as this library's arm prints: a 256 MB fp32
        # allreduce, CUDA events on the caller's stream, max over ranks.
        try:
            import statistics
            nbytes = 256 << 20
            buf = torch.ones(nbytes // 4, device=device)
            for _ in range(3):
                dist.all_reduce(buf, op=dist.ReduceOp.AVG)
            samples = []
            for _ in range(5):
                b0, b1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                b0.record()
                dist.all_reduce(buf, op=dist.ReduceOp.AVG)
                b1.record()
                b1.synchronize()
                samples.append(b0.elapsed_time(b1) * 1e3)
            us = allmax(statistics.median(samples))
            bus = {"bytes": nbytes, "dtype": "fp32", "n_gpus": world,
                   "nccl_all_reduce": {"us": round(us, 1),
                                       "bus_gbs": round(nbytes * 2.0 * (world - 1) / world
                                                        / (us * 1e-6) / 1e9, 1)}}
        except Exception as e:  # the throughput line must survive
            bus = {"error": "%s: %s" % (type(e).__name__, e)}
    if rank == 0:
        total = batch * args.gpus * args.steps
        cfg.update({"parallelism": "dp%d" % args.gpus, "per_gpu_batch": batch,
                    "gradient_path": "torch DistributedDataParallel, NCCL, bucket_cap_mb=128"
                                     + (", fp16_compress_hook" if args.model == "bert-large" else "")})
        print(json.dumps({
            "metric": metric, "value": round(total / (ms / 1e3), 2), "unit": unit,
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(ms / args.steps, 3), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "impl": "ddp", "config": cfg, "clocks": clocks,
            "e2e": {"value": round(total / (e2e_ms / 1e3), 2), "unit": unit,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4},
            "gpu_launches": 0, "final_loss": float(loss_host.item()),
            **({"allreduce_bus": bus} if bus is not None else {})}))
    dist.destroy_process_group()
    return 0


def main():
    args = parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": REFERENCE_UNAVAILABLE}))
        return 0
    if args.impl == "ddp":
        return main_ddp(args)
    if args.backend:
        os.environ["HOROVOD_GPU_BACKEND"] = args.backend

    import torch
    import horovod_b200.torch as hvd
    from horovod_b200 import _C

    if not torch.cuda.is_available():
        print(json.dumps({"error": "no CUDA device; bench.py needs a GPU"}))
        return 1
    hvd.init()
    if hvd.size() != args.gpus:
        raise SystemExit("--gpus %d but the job has %d ranks" % (args.gpus, hvd.size()))
    torch.cuda.set_device(hvd.local_rank())
    device = torch.device("cuda", hvd.local_rank())
    torch.backends.cudnn.benchmark = True

    # The flagship measurement comes first; what follows it must not cost the line.
    rc = 0
    out, in_sync = measure(args, args.model, hvd, torch, device, _C)
    if not in_sync:
        rc = 3
    secondary = None
    if args.secondary and args.model == "resnet50":
        try:
            secondary, sec_sync = measure(args, "bert-large", hvd, torch, device, _C)
            if not sec_sync:
                rc = 3
        except Exception as e:  # the flagship line must survive
            secondary = {"error": "%s: %s" % (type(e).__name__, e)}
    single = bus = checks = None
    if hvd.size() > 1:
        try:
            worst = loss_vs_single(hvd, torch, device,
                                   bool(args.symmetric_gradients and args.model == "resnet50"))
            single = {"max_rel_diff_of_step_losses": worst, "tolerance": 1e-4, "steps": 5,
                      "what": "2-layer causal LM, fp32, rank-specific batches through "
                              "DistributedOptimizer vs plain SGD on the concatenated batch"}
            if not worst <= 1e-4:
                rc = 3
        except Exception as e:  # the flagship line must survive
            single = {"error": "%s: %s" % (type(e).__name__, e)}
            rc = 3
        try:
            bus = allreduce_bus_bandwidth(hvd, torch, device)
        except Exception as e:  # the flagship line must survive
            bus = {"error": "%s: %s" % (type(e).__name__, e)}
        try:
            passed, failed = collective_checks(hvd, torch, device)
            checks = {"passed": passed, "failed": failed}
        except Exception as e:  # the flagship line must survive
            checks = {"passed": 0, "failed": ["%s: %s" % (type(e).__name__, e)]}
        if checks["failed"]:
            rc = 3
    if hvd.rank() == 0:
        if bus is not None:
            out["allreduce_bus"] = bus
        if checks is not None:
            out["collective_checks"] = checks
        if single is not None:
            out["loss_vs_single"] = single
        if secondary is not None:
            out["secondary"] = secondary
        print(json.dumps(out))
    hvd.shutdown()
    return rc


if __name__ == "__main__":
    sys.exit(main())
