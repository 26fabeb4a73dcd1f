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
    p.add_argument("--impl", default="ours", choices=["ours", "reference"])
    p.add_argument("--model", default="resnet50",
                   choices=["resnet50", "bert-large", "gpt2-medium"])
    p.add_argument("--batch", type=int, default=0, help="per-GPU batch (0 = config default)")
    p.add_argument("--backend", default=None, help="symm | nccl (HOROVOD_GPU_BACKEND)")
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
                 "--format=csv,noheader,nounits", "-lms", "200"],
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
        opt = torch.optim.SGD(model.parameters(), lr=0.01, momentum=0.9, weight_decay=1e-4)
        g = torch.Generator().manual_seed(1)
        host_x = [torch.randn(batch, 3, 224, 224, generator=g).pin_memory() for _ in range(2)]
        host_y = [torch.randint(0, 1000, (batch,), generator=g).pin_memory() for _ in range(2)]

        def to_dev(x):
            return x.to(device, non_blocking=True).contiguous(memory_format=torch.channels_last)

        def loss_fn(x, y):
            return torch.nn.functional.cross_entropy(model(x), y)
        cfg = {"model": "ResNet-50 v1.5", "global_batch": batch * args.gpus, "seq_len": None,
               "optimizer": "SGD momentum 0.9 wd 1e-4, fp32 master weights",
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


def main():
    args = parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": REFERENCE_UNAVAILABLE}))
        return 0
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
    torch.manual_seed(0)
    torch.backends.cudnn.benchmark = True

    (model, base_opt, host_x, host_y, to_dev, loss_fn, batch, cfg, metric,
     unit) = build_workload(args, torch, device)
    if args.model == "resnet50":
        opt = hvd.DistributedOptimizer(base_opt, named_parameters=model.named_parameters(),
                                       symmetric_gradients=bool(args.symmetric_gradients))
    elif args.model == "bert-large":
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

    if hvd.rank() == 0:
        total = batch * args.gpus * args.steps
        value = total / (ms / 1e3)
        cfg.update({"parallelism": "dp%d" % args.gpus, "per_gpu_batch": batch,
                    "l2": "inputs larger than L2 (%.0f MB activations+batch per step)"
                          % (h2d / 1e6),
                    "gradient_path": hvd.gpu_backend(),
                    "symmetric_gradients": bool(args.symmetric_gradients and args.gpus > 1
                                                and args.model == "resnet50"),
                    "fusion_threshold_mb": 128, "cycle_time_ms": 1.0})
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
        print(json.dumps(out))
    hvd.shutdown()
    return 0


if __name__ == "__main__":
    sys.exit(main())
