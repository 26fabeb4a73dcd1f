"""The synthetic benchmark as an elastic job: throughput keeps being reported
while workers leave and join; the state (model, optimizer, position in the
benchmark) survives every change of membership.

    horovodrun -np 2 --min-np 1 --max-np 4 --host-discovery-script ./discover.sh \
        python examples/pytorch_synthetic_benchmark_elastic.py

Counterpart of the reference's examples/elastic/pytorch/pytorch_synthetic_benchmark_elastic.py.
"""
import argparse
import timeit

import torch
import torch.nn.functional as F

import horovod_b200.torch as hvd
from horovod_b200 import models

parser = argparse.ArgumentParser()
parser.add_argument("--model", default="resnet50", choices=["resnet50", "tiny"])
parser.add_argument("--batch-size", type=int, default=32)
parser.add_argument("--image-size", type=int, default=224)
parser.add_argument("--num-warmup-batches", type=int, default=10)
parser.add_argument("--num-batches-per-iter", type=int, default=10)
parser.add_argument("--num-batches-per-commit", type=int, default=1)
parser.add_argument("--num-iters", type=int, default=10)
parser.add_argument("--no-cuda", action="store_true")
args = parser.parse_args()

hvd.init()
cuda = not args.no_cuda and torch.cuda.is_available()
if cuda:
    torch.cuda.set_device(hvd.local_rank())
device = torch.device("cuda", hvd.local_rank()) if cuda else torch.device("cpu")

build = models.resnet50 if args.model == "resnet50" else models.resnet_tiny
model = build().to(device)
base_lr = 0.01
optimizer = hvd.DistributedOptimizer(torch.optim.SGD(model.parameters(), lr=base_lr * hvd.size()),
                                     named_parameters=model.named_parameters())
data = torch.randn(args.batch_size, 3, args.image_size, args.image_size, device=device)
target = torch.randint(0, 10, (args.batch_size,), device=device)


def benchmark_step(state):
    optimizer.zero_grad()
    F.cross_entropy(model(data), target).backward()
    optimizer.step()
    state.batch += 1
    if state.batch % args.num_batches_per_commit == 0:
        state.commit()  # also where a change of membership is noticed


def log(message):
    if hvd.rank() == 0:
        print(message, flush=True)


@hvd.elastic.run
def run_benchmark(state):
    if not state.warm:
        for _ in range(args.num_warmup_batches):
            benchmark_step(state)
        state.warm = True
        state.commit()
    for state.iter in range(state.iter, args.num_iters):
        seconds = timeit.timeit(lambda: benchmark_step(state), number=args.num_batches_per_iter)
        rate = args.batch_size * args.num_batches_per_iter / seconds
        log("Iter #%d: %.1f img/sec per rank, %d rank(s)" % (state.iter, rate, hvd.size()))
        state.rates.append(rate * hvd.size())
        state.commit()


def on_state_reset():
    # the per-rank learning rate stays; the total follows the number of ranks
    for group in optimizer.param_groups:
        group["lr"] = base_lr * hvd.size()


state = hvd.elastic.TorchState(model, optimizer, batch=0, iter=0, warm=False, rates=[])
state.register_reset_callbacks([on_state_reset])
run_benchmark(state)
log("Total img/sec over %d iteration(s): %.1f" % (len(state.rates),
                                                  sum(state.rates) / max(len(state.rates), 1)))
hvd.shutdown()
