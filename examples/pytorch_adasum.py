"""Adasum instead of averaging: gradients (here: the optimizer's updates) of
the ranks are combined pairwise so that the part they agree on is not counted
twice, which lets the learning rate stay at its single-rank value as ranks
are added. The script trains the same small regression model with
``op=hvd.Average`` (learning rate scaled by the number of ranks) and with
``op=hvd.Adasum`` (unscaled) and prints both loss curves.

    horovodrun -np 4 python examples/pytorch_adasum.py

See docs/adasum_user_guide.rst of the reference for the background.
"""
import argparse

import torch

import horovod_b200.torch as hvd

parser = argparse.ArgumentParser()
parser.add_argument("--steps", type=int, default=60)
parser.add_argument("--batch-size", type=int, default=64, help="per rank")
parser.add_argument("--lr", type=float, default=0.05)
parser.add_argument("--no-cuda", action="store_true")
args = parser.parse_args()

hvd.init()
cuda = not args.no_cuda and torch.cuda.is_available()
if cuda:
    torch.cuda.set_device(hvd.local_rank())
device = torch.device("cuda", hvd.local_rank()) if cuda else torch.device("cpu")

# y = <w*, x> + noise; every rank draws its own samples.
g = torch.Generator().manual_seed(0)
w_star = torch.randn(32, 1, generator=g)
g_rank = torch.Generator().manual_seed(100 + hvd.rank())


def batch():
    x = torch.randn(args.batch_size, 32, generator=g_rank)
    y = x @ w_star + 0.01 * torch.randn(args.batch_size, 1, generator=g_rank)
    return x.to(device), y.to(device)


def train(op, lr):
    torch.manual_seed(1)
    model = torch.nn.Sequential(torch.nn.Linear(32, 64), torch.nn.Tanh(),
                                torch.nn.Linear(64, 1)).to(device)
    opt = hvd.DistributedOptimizer(torch.optim.SGD(model.parameters(), lr=lr),
                                   named_parameters=model.named_parameters(), op=op)
    hvd.broadcast_parameters(model.state_dict(), root_rank=0)
    losses = []
    for _ in range(args.steps):
        x, y = batch()
        opt.zero_grad()
        loss = torch.nn.functional.mse_loss(model(x), y)
        loss.backward()
        opt.step()
        losses.append(float(hvd.allreduce(loss.detach().cpu(), name="loss")))
    return losses


averaged = train(hvd.Average, args.lr * hvd.size())
adasum = train(hvd.Adasum, args.lr)
if hvd.rank() == 0:
    for name, curve in (("average (lr x size)", averaged), ("adasum (lr unscaled)", adasum)):
        print("%-22s first loss %.4f last loss %.4f" % (name, curve[0], curve[-1]), flush=True)
hvd.shutdown()
