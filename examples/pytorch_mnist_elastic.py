"""The MNIST example as an elastic job: the model, the optimizer, the epoch,
the batch and the part of the epoch already seen (``ElasticSampler``) survive
workers leaving and joining; training goes on from the last commit.

    horovodrun -np 2 --min-np 1 --max-np 4 --host-discovery-script ./discover.sh \\
        python examples/pytorch_mnist_elastic.py --epochs 3

(It also runs as a plain job: ``horovodrun -np 2 python examples/pytorch_mnist_elastic.py``.)
Synthetic MNIST-shaped data, since nothing can be downloaded here.
Counterpart of the reference's examples/elastic/pytorch/pytorch_mnist_elastic.py.
"""
import argparse

import torch
import torch.nn as nn
import torch.nn.functional as F

import horovod_b200.torch as hvd

parser = argparse.ArgumentParser()
parser.add_argument("--epochs", type=int, default=2)
parser.add_argument("--batch-size", type=int, default=64)
parser.add_argument("--batches-per-commit", type=int, default=8,
                    help="a commit costs a copy of the state: not every batch")
parser.add_argument("--lr", type=float, default=0.01)
parser.add_argument("--samples", type=int, default=4096)
parser.add_argument("--no-cuda", action="store_true")
args = parser.parse_args()

hvd.init()
torch.manual_seed(42)
cuda = not args.no_cuda and torch.cuda.is_available()
if cuda:
    torch.cuda.set_device(hvd.local_rank())
device = torch.device("cuda", hvd.local_rank()) if cuda else torch.device("cpu")


class Net(nn.Module):
    def __init__(self):
        super().__init__()
        self.conv1 = nn.Conv2d(1, 10, 5)
        self.conv2 = nn.Conv2d(10, 20, 5)
        self.fc1 = nn.Linear(320, 50)
        self.fc2 = nn.Linear(50, 10)

    def forward(self, x):
        x = F.relu(F.max_pool2d(self.conv1(x), 2))
        x = F.relu(F.max_pool2d(self.conv2(x), 2))
        return self.fc2(F.relu(self.fc1(x.flatten(1))))


g = torch.Generator().manual_seed(0)
labels = torch.randint(0, 10, (args.samples,), generator=g)
images = torch.randn(args.samples, 1, 28, 28, generator=g) * 0.3
for i, c in enumerate(labels.tolist()):
    images[i, 0, 2 * c:2 * c + 8, 2 * c:2 * c + 8] += 1.0
dataset = torch.utils.data.TensorDataset(images, labels)
# The sampler shards what is LEFT of the epoch over the ranks there are now.
sampler = hvd.elastic.ElasticSampler(dataset)
loader = torch.utils.data.DataLoader(dataset, batch_size=args.batch_size, sampler=sampler)

model = Net().to(device)
optimizer = hvd.DistributedOptimizer(
    torch.optim.SGD(model.parameters(), lr=args.lr * hvd.size(), momentum=0.5),
    named_parameters=model.named_parameters())


@hvd.elastic.run
def train(state):
    for state.epoch in range(state.epoch, args.epochs):
        if state.batch == 0:            # not when resuming in the middle of an epoch
            state.sampler.set_epoch(state.epoch)
        model.train()
        seen, correct, loss_sum = 0, 0, 0.0
        first = state.batch                 # > 0 when an epoch is resumed after a reset
        for idx, (x, y) in enumerate(loader):
            x, y = x.to(device), y.to(device)
            optimizer.zero_grad()
            out = model(x)
            loss = F.cross_entropy(out, y)
            loss.backward()
            optimizer.step()
            seen += y.numel()
            correct += (out.argmax(1) == y).sum().item()
            loss_sum += loss.item() * y.numel()
            state.batch = first + idx + 1
            # positions count from the start of this pass over what was left
            state.sampler.record_batch(idx, args.batch_size)
            if state.batch % args.batches_per_commit == 0:
                state.commit()      # snapshot; also where membership changes are noticed
        stats = hvd.allreduce(torch.tensor([loss_sum / max(seen, 1), correct / max(seen, 1)]),
                              name="epoch_stats")
        if hvd.rank() == 0:
            print("epoch %d: loss %.4f accuracy %.3f on %d rank(s)"
                  % (state.epoch, stats[0], stats[1], hvd.size()), flush=True)
        state.batch = 0
        state.commit()


def on_state_reset():
    # keep the per-rank learning rate: the total follows the number of ranks
    for group in optimizer.param_groups:
        group["lr"] = args.lr * hvd.size()


state = hvd.elastic.TorchState(model, optimizer, sampler=sampler, epoch=0, batch=0)
state.register_reset_callbacks([on_state_reset])
train(state)
hvd.shutdown()
