"""Synthetic training benchmark in the style of the reference's
examples/pytorch/pytorch_synthetic_benchmark.py: a torchvision-style model,
one fixed random batch, SGD wrapped in hvd.DistributedOptimizer.

    horovodrun -np 8 python examples/pytorch_synthetic_benchmark.py --fp16-allreduce
"""
import argparse
import timeit

import numpy as np
import torch
import torch.nn.functional as F

import horovod_b200.torch as hvd
from horovod_b200 import models

parser = argparse.ArgumentParser()
parser.add_argument("--fp16-allreduce", action="store_true",
                    help="send gradients as fp16 (cast fused into the allreduce kernel)")
parser.add_argument("--use-adasum", action="store_true")
parser.add_argument("--batch-size", type=int, default=32)
parser.add_argument("--num-warmup-batches", type=int, default=10)
parser.add_argument("--num-batches-per-iter", type=int, default=10)
parser.add_argument("--num-iters", type=int, default=10)
parser.add_argument("--no-cuda", action="store_true")
parser.add_argument("--symmetric-gradients", action="store_true",
                    help="keep the gradients in symmetric memory and reduce them in place")
parser.add_argument("--bf16", action="store_true",
                    help="channels-last bf16 autocast (the fused batch-norm kernels need it)")
args = parser.parse_args()

hvd.init()
cuda = not args.no_cuda and torch.cuda.is_available()
if cuda:
    torch.cuda.set_device(hvd.local_rank())
device = torch.device("cuda", hvd.local_rank()) if cuda else torch.device("cpu")
torch.backends.cudnn.benchmark = True

model = models.resnet50().to(device)
if args.bf16 and cuda:
    model = model.to(memory_format=torch.channels_last)
lr_scaler = hvd.size() if not args.use_adasum else 1
optimizer = torch.optim.SGD(model.parameters(), lr=0.01 * lr_scaler)
compression = hvd.Compression.fp16 if args.fp16_allreduce else hvd.Compression.none
optimizer = hvd.DistributedOptimizer(optimizer, named_parameters=model.named_parameters(),
                                     compression=compression,
                                     op=hvd.Adasum if args.use_adasum else hvd.Average,
                                     symmetric_gradients=args.symmetric_gradients)
hvd.broadcast_parameters(model.state_dict(), root_rank=0)
hvd.broadcast_optimizer_state(optimizer, root_rank=0)

data = torch.randn(args.batch_size, 3, 224, 224, device=device)
if args.bf16 and cuda:
    data = data.contiguous(memory_format=torch.channels_last)
target = torch.randint(0, 1000, (args.batch_size,), device=device)


def benchmark_step():
    optimizer.zero_grad()
    with torch.autocast("cuda", dtype=torch.bfloat16, enabled=bool(args.bf16 and cuda)):
        loss = F.cross_entropy(model(data), target)
    loss.backward()
    optimizer.step()
    if cuda:
        torch.cuda.synchronize()


def log(s):
    if hvd.rank() == 0:
        print(s, flush=True)


log("Model: resnet50, batch size %d, ranks %d, device path: %s"
    % (args.batch_size, hvd.size(), hvd.gpu_backend()))
timeit.timeit(benchmark_step, number=args.num_warmup_batches)
img_secs = []
for x in range(args.num_iters):
    t = timeit.timeit(benchmark_step, number=args.num_batches_per_iter)
    img_sec = args.batch_size * args.num_batches_per_iter / t
    log("Iter #%d: %.1f img/sec per rank" % (x, img_sec))
    img_secs.append(img_sec)
mean, conf = np.mean(img_secs), 1.96 * np.std(img_secs)
log("Img/sec per rank: %.1f +-%.1f" % (mean, conf))
log("Total img/sec on %d rank(s): %.1f +-%.1f" % (hvd.size(), hvd.size() * mean,
                                                  hvd.size() * conf))
hvd.shutdown()
