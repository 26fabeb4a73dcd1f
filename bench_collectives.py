"""Collective sweep: allreduce (fp32, bf16), reducescatter, allgather,
broadcast and alltoall on one tensor from 1 KB to 1 GB in powers of two, plus
a grouped allreduce of 64 fp32 tensors with log-uniform sizes in 4 KB-4 MB.
``allreduce_symm`` / ``grouped_symm`` are the same allreduces on tensors that
live in the symmetric heap (hvd.symmetric_empty), reduced in place without
staging (symm backend only).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 \
        --master-addr 127.0.0.1 --master-port 29500 bench_collectives.py \
        --backend symm --max-mb 1024

Every number is device time of the whole response on the communication
stream (CUDA events around the launches, after the producer wait), maximum
over ranks, median over iterations. ``--backend nccl`` runs the same harness
over the NCCL path (pack -> NCCL -> unpack as the reference issues it), which
is the baseline of the comparison. Bus bandwidth follows the usual
conventions: allreduce 2(N-1)/N * S / t, reducescatter/allgather (N-1)/N * S_total / t,
broadcast S / t, alltoall (N-1)/N * S / t. The roofline for each op is the
bytes that must cross one GPU's NVLink in one direction at the measured
770 GB/s: allreduce 2(N-1)/N * S (the bandwidth lower bound without in-network
reduction) or S when the NVSwitch reduces (multimem, 4+ ranks); (N-1)/N * S
for reducescatter, allgather and alltoall; S for broadcast.
Rank 0 prints one JSON line per (op, dtype, size).
"""
import argparse
import json
import os
import statistics
import sys
import time

ALLREDUCE, ALLGATHER, BROADCAST, ALLTOALL, REDUCESCATTER = 0, 1, 2, 5, 6
LINK_GBS = 770.0


def main():
    p = argparse.ArgumentParser()
    p.add_argument("--backend", default="symm", choices=["symm", "nccl"])
    p.add_argument("--min-kb", type=int, default=1)
    p.add_argument("--max-mb", type=int, default=256)
    p.add_argument("--step", type=int, default=2, help="factor between consecutive sizes")
    p.add_argument("--iters", type=int, default=20)
    p.add_argument("--warmup", type=int, default=5)
    p.add_argument("--ops", default="allreduce,allreduce_bf16,reducescatter,allgather,"
                                    "broadcast,alltoall,grouped,allreduce_symm,grouped_symm,"
                                    "reducescatter_symm")
    p.add_argument("--algo", default=None, help="force oneshot|twoshot|nvls")
    p.add_argument("--ctas", type=int, default=0)
    p.add_argument("--phases", action="store_true",
                   help="also report where the time goes inside the allreduce kernels "
                        "(device timestamps at phase boundaries, HOROVOD_KERNEL_TRACE=1)")
    args = p.parse_args()
    if args.phases:
        os.environ["HOROVOD_KERNEL_TRACE"] = "1"

    os.environ["HOROVOD_GPU_BACKEND"] = args.backend
    os.environ["HOROVOD_GPU_OP_TIMING"] = "1"
    os.environ["HOROVOD_FUSION_THRESHOLD"] = str(256 << 20)
    if args.algo:
        os.environ["HOROVOD_ALLREDUCE_ALGO"] = args.algo
    if args.ctas:
        os.environ["HOROVOD_COMM_CTAS"] = str(args.ctas)

    import torch
    import horovod_b200.torch as hvd
    from horovod_b200 import _C

    hvd.init()
    n, rank = hvd.size(), hvd.rank()
    torch.cuda.set_device(hvd.local_rank())
    dev = torch.device("cuda", hvd.local_rank())
    torch.manual_seed(rank)

    from horovod_b200.utils.clocks import ClockLog
    clock_log = ClockLog(hvd.local_rank()) if rank == 0 else None
    window = [0.0, 0.0]  # wall-clock bounds of the last measurement
    host_us = [0.0]      # host time inside the timed interval (rank 0, median)

    def measure(fn, want_type):
        """Runs fn() warmup+iters times, one response at a time, and returns
        the median device time (us, max over ranks) of the matching ops."""
        for _ in range(args.warmup):
            fn()
        torch.cuda.synchronize()
        _C.gpu_op_stats()
        window[0] = time.time()
        for _ in range(args.iters):
            fn()
        torch.cuda.synchronize()
        window[1] = time.time()
        stats = [t for t in _C.gpu_op_stats() if t[0] == want_type][-args.iters:]
        mine = [t[3] for t in stats]
        host_us[0] = statistics.median(t[4] for t in stats) if stats else 0.0
        t = torch.tensor(mine, dtype=torch.float64)
        t = hvd.allreduce(t, op=hvd.Max, name="sweep.times.%d" % len(mine))
        return statistics.median(t.tolist())

    PHASES = ("start", "packed", "barrier1", "reduced", "barrier2", "unpacked")

    XPHASES = ("start", "staged", "pulled", "done", "last_cta_done", "credit_wait")

    def phases(fn, PHASES=PHASES):
        """Median offsets (us since kernel start, CTA 0 of this rank) of the
        phase boundaries of the traced kernel, max over ranks."""
        cols = []
        for _ in range(args.iters):
            fn()
            torch.cuda.synchronize()
            t = _C.kernel_trace()
            # ("credit_wait": from kernel entry to "start", i.e. the wait for the
            # exchange region to be free)
            cols.append([(t[0] - t[i]) / 1e3 if PHASES[i] == "credit_wait" and t[i]
                         else (t[i] - t[0]) / 1e3 if t[i] >= t[0] and t[i] else -1.0
                         for i in range(len(PHASES))])
            hvd.allreduce(torch.zeros(1), name="sweep.phase.sync")
        med = [statistics.median(c[i] for c in cols) for i in range(len(PHASES))]
        t = hvd.allreduce(torch.tensor(med, dtype=torch.float64), op=hvd.Max,
                          name="sweep.phases")
        return {k: round(v, 1) for k, v in zip(PHASES, t.tolist()) if v >= 0}

    def emit(op, dtype, nbytes, us, bus_factor, wire_bytes, extra=None):
        if rank != 0:
            return
        bus = nbytes * bus_factor / (us * 1e-6) / 1e9 if us > 0 else 0.0
        roof_us = wire_bytes / (LINK_GBS * 1e9) * 1e6
        print(json.dumps({"op": op, "dtype": dtype, "bytes": nbytes, "n_gpus": n,
                          "backend": args.backend, "device_us": round(us, 2),
                          "host_us_between_events": round(host_us[0], 2),
                          "bus_gbs": round(bus, 2),
                          "roofline_us": round(roof_us, 2),
                          "frac_of_nvlink_roofline": round(roof_us / us, 4) if us > 0 else None,
                          "gradient_path": hvd.gpu_backend(),
                          "clocks": clock_log.window(window[0], window[1]),
                          **(extra or {})}), flush=True)

    def ar_wire(nbytes):
        nvls = n >= 4 and "nvls=1" in hvd.gpu_backend()
        return nbytes if nvls else 2 * nbytes * (n - 1) / n

    ops = args.ops.split(",")
    sizes = []
    s = args.min_kb << 10
    while s <= args.max_mb << 20:
        sizes.append(s)
        s *= max(2, args.step)

    heap = None
    if args.backend == "symm" and n > 1 and ("allreduce_symm" in ops or "grouped_symm" in ops
                                             or "reducescatter_symm" in ops):
        os.environ.setdefault("HOROVOD_SYMM_HEAP_MB", "2048")
        heap = hvd.symmetric_empty(max(sizes[-1], 160 << 20) // 4)
        heap.normal_()

    for nbytes in sizes:
        if "allreduce_symm" in ops and heap is not None:
            x = heap[:nbytes // 4]
            us = measure(lambda: hvd.allreduce_(x, op=hvd.Average, name="sw.ars"), ALLREDUCE)
            ph = {"phases_us": phases(lambda: hvd.allreduce_(x, op=hvd.Average, name="sw.ars"))} \
                if args.phases else None
            emit("allreduce_symm", "fp32", nbytes, us, 2 * (n - 1) / n, ar_wire(nbytes), ph)
        if "allreduce" in ops:
            x = torch.randn(nbytes // 4, device=dev)
            us = measure(lambda: hvd.allreduce_(x, op=hvd.Sum, name="sw.ar"), ALLREDUCE)
            ph = {"phases_us": phases(lambda: hvd.allreduce_(x, op=hvd.Sum, name="sw.ar"))} \
                if args.phases else None
            emit("allreduce", "fp32", nbytes, us, 2 * (n - 1) / n, ar_wire(nbytes), ph)
        if "allreduce_bf16" in ops:
            x = torch.randn(nbytes // 2, device=dev).bfloat16()
            us = measure(lambda: hvd.allreduce_(x, op=hvd.Sum, name="sw.arb"), ALLREDUCE)
            emit("allreduce", "bf16", nbytes, us, 2 * (n - 1) / n, ar_wire(nbytes))
        if "reducescatter_symm" in ops and heap is not None and nbytes >= 64 * n:
            # input in the symmetric heap, shards on 16-byte boundaries: no staging
            x = heap[:nbytes // 4 // (4 * n) * (4 * n)]
            us = measure(lambda: hvd.reducescatter(x, op=hvd.Sum, name="sw.rss"), REDUCESCATTER)
            emit("reducescatter_symm", "fp32", nbytes, us, (n - 1) / n, nbytes * (n - 1) / n)
        if "reducescatter" in ops and nbytes >= 4 * n:
            x = torch.randn(nbytes // 4 // n * n, device=dev)
            us = measure(lambda: hvd.reducescatter(x, op=hvd.Sum, name="sw.rs"), REDUCESCATTER)
            emit("reducescatter", "fp32", nbytes, us, (n - 1) / n, nbytes * (n - 1) / n)
        if "allgather" in ops and nbytes // n >= 4:
            x = torch.randn(nbytes // 4 // n, device=dev)
            us = measure(lambda: hvd.allgather(x, name="sw.ag"), ALLGATHER)
            ph = {"phases_us": phases(lambda: hvd.allgather(x, name="sw.ag"), XPHASES)} \
                if args.phases else None
            emit("allgather", "fp32", nbytes, us, (n - 1) / n, nbytes * (n - 1) / n, ph)
        if "broadcast" in ops:
            x = torch.randn(nbytes // 4, device=dev)
            us = measure(lambda: hvd.broadcast_(x, root_rank=0, name="sw.bc"), BROADCAST)
            ph = {"phases_us": phases(lambda: hvd.broadcast_(x, root_rank=0, name="sw.bc"),
                                      XPHASES)} if args.phases else None
            emit("broadcast", "fp32", nbytes, us, 1.0, nbytes, ph)
        if "alltoall" in ops and nbytes // n >= 4:
            x = torch.randn(nbytes // 4 // n * n, device=dev)
            us = measure(lambda: hvd.alltoall(x, name="sw.a2a"), ALLTOALL)
            ph = {"phases_us": phases(lambda: hvd.alltoall(x, name="sw.a2a"), XPHASES)} \
                if args.phases else None
            emit("alltoall", "fp32", nbytes, us, (n - 1) / n, nbytes * (n - 1) / n, ph)

    if "grouped" in ops:
        g = torch.Generator().manual_seed(0)
        import math
        logs = torch.rand(64, generator=g) * (math.log(4 << 20) - math.log(4 << 10)) \
            + math.log(4 << 10)
        counts = [max(1, int(math.exp(v)) // 4) for v in logs.tolist()]
        xs = [torch.randn(c, device=dev) for c in counts]
        total = sum(c * 4 for c in counts)
        us = measure(lambda: hvd.grouped_allreduce_(xs, op=hvd.Sum, name="sw.grp"), ALLREDUCE)
        emit("grouped_allreduce_64", "fp32", total, us, 2 * (n - 1) / n, ar_wire(total))
        if "grouped_symm" in ops and heap is not None:
            views, at = [], 0
            for c in counts:
                views.append(heap[at:at + c])
                at += (c + 63) // 64 * 64
            us = measure(lambda: hvd.grouped_allreduce_(views, op=hvd.Average, name="sw.grps"),
                         ALLREDUCE)
            emit("grouped_allreduce_64_symm", "fp32", total, us, 2 * (n - 1) / n,
                 ar_wire(total))

    if clock_log is not None:
        clock_log.stop()
    hvd.shutdown()
    return 0


if __name__ == "__main__":
    sys.exit(main())
