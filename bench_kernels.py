"""Single-GPU micro-benchmark of the library's local kernels, reported against
the measured HBM copy bandwidth (MEASURED_PEAKS.json: hbm_gbs).

    python bench_kernels.py                 # all cases
    python bench_kernels.py --case fused_local --mb 512 --iters 3   # small ncu target

Cases
  fused_local   the fused multi-tensor allreduce kernel on one rank (LOCAL
                variant): reads 161 ResNet-50-shaped gradient tensors, scales
                and writes them back in one launch (read + write = 2x bytes).
  fused_fp16    same with float16 tensors.
  reducescatter reduce-scatter kernel on one rank: stage -> reduce -> write
                (read + write staging + read staging + write = 4x bytes).
  exchange      allgather of one rank through the exchange kernel: with nobody
                to send to it is one copy into the output (2x bytes).
  batch_norm    fused batch norm + residual + ReLU on a channels-last bf16
                activation of 256 x 256 x 56 x 56 (411 MB): forward (statistics
                pass + apply pass: read x twice, read the residual, write y =
                4x bytes) and backward (reduce pass reads dy, y, x; apply pass
                reads them again and writes dx and dres = 8x bytes), timed with
                CUDA events on the current stream, next to the PyTorch eager
                composition batch_norm -> add -> relu on the same tensors.

  max_pool      3x3 / stride 2 / padding 1 max pooling on the ResNet stem
                activation 256 x 64 x 112 x 112 bf16 (411 MB): forward reads x,
                writes y (1/4 of x) and one index byte per output element
                (1/8 of x): 1.375x; backward reads dy and the indices and
                writes dx: 1.375x. Next to PyTorch's max_pool2d.
  fused_sgd     hvd.FusedSGD step (momentum + weight decay) over 161
                ResNet-50-shaped fp32 tensors: reads p, g, m, writes p, m
                (5x bytes). Next to torch.optim.SGD on the same tensors.

Timing is device time of the response on the communication stream (CUDA
events around the launches). Inputs are larger than L2 (126 MB) unless --mb
says otherwise. Prints one JSON line per case.
"""
import argparse
import json
import os
import statistics
import sys
import time

os.environ["HOROVOD_GPU_OP_TIMING"] = "1"
os.environ.setdefault("HOROVOD_FUSION_THRESHOLD", str(1 << 30))


def resnet50_like_sizes(total_elems):
    """161 tensor sizes with ResNet-50's skew (a few large convolutions, many
    tiny batch-norm vectors), scaled to about total_elems."""
    base = []
    for planes, blocks in ((64, 3), (128, 4), (256, 6), (512, 3)):
        for b in range(blocks):
            inp = planes * 4 if b else max(64, planes * 2)
            base += [inp * planes, planes, planes, planes * planes * 9, planes, planes,
                     planes * planes * 4, planes * 4, planes * 4]
            if b == 0:
                base += [inp * planes * 4, planes * 4, planes * 4]
    base += [64 * 3 * 49, 64, 64, 2048 * 1000, 1000]
    base = base[:161]
    scale = total_elems / float(sum(base))
    return [max(1, int(s * scale)) for s in base]


def main():
    p = argparse.ArgumentParser()
    p.add_argument("--case", default="all")
    p.add_argument("--mb", type=int, default=512, help="payload per case in MB")
    p.add_argument("--iters", type=int, default=10)
    p.add_argument("--warmup", type=int, default=3)
    args = p.parse_args()

    import torch
    import horovod_b200.torch as hvd
    from horovod_b200 import _C

    peaks = {}
    try:
        peaks = json.load(open(os.path.join(os.path.dirname(os.path.abspath(__file__)),
                                            "MEASURED_PEAKS.json")))
    except OSError:
        pass
    hbm = float(peaks.get("hbm_gbs", 6650.0))
    peak_src = "measured" if peaks else "fallback"

    hvd.init()
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    nbytes = args.mb << 20

    from horovod_b200.utils.clocks import ClockLog
    clock_log = ClockLog(0)

    def run(name, fn, want_type, algorithmic_bytes):
        for _ in range(args.warmup):
            fn()
        torch.cuda.synchronize()
        _C.gpu_op_stats()
        t_begin = time.time()
        for _ in range(args.iters):
            fn()
        torch.cuda.synchronize()
        t_end = time.time()
        us = [t[3] for t in _C.gpu_op_stats() if t[0] == want_type][-args.iters:]
        med = statistics.median(us)
        gbs = algorithmic_bytes / (med * 1e-6) / 1e9
        print(json.dumps({"case": name, "payload_mb": args.mb, "device_us": round(med, 1),
                          "algorithmic_gbs": round(gbs, 1),
                          "frac_of_%s_hbm_copy" % peak_src: round(gbs / hbm, 3),
                          "hbm_gbs_peak": hbm,
                          "clocks": clock_log.window(t_begin, t_end)}), flush=True)

    cases = ["fused_local", "fused_fp16", "reducescatter", "exchange", "batch_norm", "max_pool",
             "fused_sgd"] if args.case == "all" else [args.case]

    def timed_events(fn, reps):
        for _ in range(args.warmup):
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(reps):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) * 1e3)
        return statistics.median(ts)

    def report_line(name, us, algorithmic, extra=None):
        gbs = algorithmic / (us * 1e-6) / 1e9
        print(json.dumps({"case": name, "device_us": round(us, 1),
                          "algorithmic_gbs": round(gbs, 1),
                          "frac_of_%s_hbm_copy" % peak_src: round(gbs / hbm, 3),
                          "hbm_gbs_peak": hbm,
                          "clocks": clock_log.window(time.time() - 1.0, time.time()),
                          **(extra or {})}), flush=True)
    if "fused_local" in cases:
        xs = [torch.randn(n, device=dev) for n in resnet50_like_sizes(nbytes // 4)]
        total = sum(x.numel() * 4 for x in xs)
        run("fused_local", lambda: hvd.grouped_allreduce_(xs, op=hvd.Sum, postscale_factor=0.5,
                                                          name="k.fused"), 0, 2 * total)
    if "fused_fp16" in cases:
        xs = [torch.randn(n, device=dev).half() for n in resnet50_like_sizes(nbytes // 2)]
        total = sum(x.numel() * 2 for x in xs)
        run("fused_fp16", lambda: hvd.grouped_allreduce_(xs, op=hvd.Sum, postscale_factor=0.5,
                                                         name="k.fused16"), 0, 2 * total)
    if "reducescatter" in cases:
        n = min(nbytes, 448 << 20) // 4
        x = torch.randn(n, device=dev)
        run("reducescatter", lambda: hvd.reducescatter(x, op=hvd.Sum, name="k.rs"), 6, 4 * n * 4)
    if "exchange" in cases:
        n = min(nbytes, 192 << 20) // 4
        x = torch.randn(n, device=dev)
        run("exchange", lambda: hvd.allgather(x, name="k.ag"), 1, 2 * n * 4)
    if "batch_norm" in cases:
        import torch.nn.functional as F
        from horovod_b200.ops.batch_norm import batch_norm_act
        n = 256 if args.mb >= 512 else 64
        shape = (n, 256, 56, 56)
        x = torch.randn(shape, device=dev, dtype=torch.bfloat16) \
            .contiguous(memory_format=torch.channels_last).requires_grad_(True)
        res = torch.randn_like(x).requires_grad_(True)
        go = torch.randn_like(x)
        w = torch.ones(256, device=dev, requires_grad=True)
        b = torch.zeros(256, device=dev, requires_grad=True)
        rm, rv = torch.zeros(256, device=dev), torch.ones(256, device=dev)
        nbytes_act = x.numel() * 2

        def timed(fn, reps):
            for _ in range(args.warmup):
                fn()
            torch.cuda.synchronize()
            ts = []
            for _ in range(reps):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                fn()
                e1.record()
                torch.cuda.synchronize()
                ts.append(e0.elapsed_time(e1) * 1e3)
            return statistics.median(ts)

        def report(name, us, algorithmic):
            gbs = algorithmic / (us * 1e-6) / 1e9
            print(json.dumps({"case": name, "shape": list(shape), "device_us": round(us, 1),
                              "algorithmic_gbs": round(gbs, 1),
                              "frac_of_%s_hbm_copy" % peak_src: round(gbs / hbm, 3),
                              "hbm_gbs_peak": hbm,
                              "clocks": clock_log.window(time.time() - 1.0, time.time())}),
                  flush=True)

        def eager_fwd():
            return F.relu(F.batch_norm(x, rm, rv, w, b, True, 0.1, 1e-5) + res)

        def fused_fwd():
            return batch_norm_act(x, w, b, rm, rv, residual=res, training=True, relu=True)

        for name, fwd in (("batch_norm_fused", fused_fwd), ("batch_norm_eager", eager_fwd)):
            t_f = timed(lambda: fwd(), args.iters)
            y = fwd()

            def bwd():
                torch.autograd.grad(y, (x, res, w, b), go, retain_graph=True)
            t_b = timed(bwd, args.iters)
            report(name + "_forward", t_f, 4 * nbytes_act)
            report(name + "_backward", t_b, 8 * nbytes_act)
            del y
    if "max_pool" in cases:
        import torch.nn.functional as F
        from horovod_b200.ops.pooling import max_pool_3x3_s2
        n = 256 if args.mb >= 512 else 32
        x = torch.relu(torch.randn(n, 64, 112, 112, device=dev)).bfloat16() \
            .contiguous(memory_format=torch.channels_last).requires_grad_(True)
        xbytes = x.numel() * 2
        for name, fwd in (("max_pool_fused", max_pool_3x3_s2),
                          ("max_pool_torch", lambda t: F.max_pool2d(t, 3, stride=2, padding=1))):
            t_f = timed_events(lambda: fwd(x), args.iters)
            y = fwd(x)
            go = torch.randn_like(y)
            t_b = timed_events(lambda: torch.autograd.grad(y, x, go, retain_graph=True), args.iters)
            report_line(name + "_forward", t_f, 1.375 * xbytes, {"shape": list(x.shape)})
            report_line(name + "_backward", t_b, 1.375 * xbytes, {"shape": list(x.shape)})
            del y
    if "fused_sgd" in cases:
        from horovod_b200.torch.fused_sgd import FusedSGD
        sizes = resnet50_like_sizes(min(nbytes, 256 << 20) // 4)
        total = sum(sizes) * 4
        for name, cls in (("fused_sgd", FusedSGD), ("torch_sgd", torch.optim.SGD)):
            ps = [torch.randn(n, device=dev, requires_grad=True) for n in sizes]
            for p in ps:
                p.grad = torch.randn_like(p)
            opt = cls(ps, lr=0.01, momentum=0.9, weight_decay=1e-4)
            opt.step()  # creates the momentum buffers
            us = timed_events(opt.step, args.iters)
            report_line(name + "_step_call", us, 5 * total,
                        {"tensors": len(sizes), "payload_mb": total >> 20,
                         "note": "optimizer.step() as called by a training loop: bounded by "
                                 "its Python work when the GPU is otherwise idle"})
            if cls is FusedSGD:
                # The kernel alone, through the plan that step() cached.
                plan, n, n_chunks = next(iter(opt._plans.values()))[1]

                def kernel_only():
                    _C.sgd_step(plan, n, n_chunks, opt.CHUNK, True, 0.01, 0.9, 0.0, 1e-4, False,
                                False, False)
                us = timed_events(kernel_only, args.iters)
                report_line("fused_sgd_kernel", us, 5 * total,
                            {"tensors": len(sizes), "payload_mb": total >> 20})
    if "peer_copy" in cases and torch.cuda.device_count() >= 2:
        # Copy-engine copy between GPU 0 and GPU 1 over NVLink, issued on a
        # stream of the source GPU (push) or of the destination GPU (pull): the
        # link rate that the SM-driven exchange kernels are compared with.
        import ctypes
        rt = ctypes.CDLL("libcudart.so.12")
        n = min(nbytes, 256 << 20)
        a = torch.empty(n, dtype=torch.uint8, device="cuda:0").fill_(1)
        b = torch.empty(n, dtype=torch.uint8, device="cuda:1")
        b.copy_(a)  # turns peer access on
        torch.cuda.synchronize(0)
        torch.cuda.synchronize(1)
        for name, d in (("peer_copy_push", 0), ("peer_copy_pull", 1)):
            with torch.cuda.device(d):
                stream = torch.cuda.Stream(device=d)

                def copy():
                    rc = rt.cudaMemcpyAsync(ctypes.c_void_p(b.data_ptr()),
                                            ctypes.c_void_p(a.data_ptr()), ctypes.c_size_t(n),
                                            ctypes.c_int(3), ctypes.c_void_p(stream.cuda_stream))
                    assert rc == 0, rc
                for _ in range(args.warmup):
                    copy()
                stream.synchronize()
                e0 = torch.cuda.Event(enable_timing=True)
                e1 = torch.cuda.Event(enable_timing=True)
                e0.record(stream)
                for _ in range(args.iters):
                    copy()
                e1.record(stream)
                e1.synchronize()
                us = e0.elapsed_time(e1) * 1e3 / args.iters
            print(json.dumps({"case": name, "payload_mb": n >> 20, "device_us": round(us, 1),
                              "nvlink_gbs_one_direction": round(n / us / 1e3, 1)}), flush=True)
    clock_log.stop()
    hvd.shutdown()
    return 0


if __name__ == "__main__":
    sys.exit(main())
