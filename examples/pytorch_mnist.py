"""Data-parallel training of a small convolutional network on MNIST-shaped
synthetic data (there is no dataset download here): DistributedSampler-style
sharding, DistributedOptimizer, parameter/optimizer broadcast, metric
averaging with hvd.allreduce, checkpoint by rank 0.

    horovodrun -np 2 python examples/pytorch_mnist.py --epochs 2
"""
import argparse

import torch
import torch.nn as nn
import torch.nn.functional as F

import horovod_b200.torch as hvd

parser = argparse.ArgumentParser()
parser.add_argument("--epochs", type=int, default=2)
parser.add_argument("--batch-size", type=int, default=64)
parser.add_argument("--lr", type=float, default=0.01)
parser.add_argument("--checkpoint", default="")
args = parser.parse_args()

hvd.init()
torch.manual_seed(42)
cuda = torch.cuda.is_available()
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


# Synthetic "dataset": class c is a noisy blob at a class-specific position.
g = torch.Generator().manual_seed(0)
labels = torch.randint(0, 10, (4096,), generator=g)
images = torch.randn(4096, 1, 28, 28, generator=g) * 0.3
for i, c in enumerate(labels.tolist()):
    images[i, 0, 2 * c:2 * c + 8, 2 * c:2 * c + 8] += 1.0
dataset = torch.utils.data.TensorDataset(images, labels)
sampler = torch.utils.data.distributed.DistributedSampler(dataset, num_replicas=hvd.size(),
                                                          rank=hvd.rank())
loader = torch.utils.data.DataLoader(dataset, batch_size=args.batch_size, sampler=sampler)

model = Net().to(device)
optimizer = torch.optim.SGD(model.parameters(), lr=args.lr * hvd.size(), momentum=0.5)
optimizer = hvd.DistributedOptimizer(optimizer, named_parameters=model.named_parameters())
hvd.broadcast_parameters(model.state_dict(), root_rank=0)
hvd.broadcast_optimizer_state(optimizer, root_rank=0)

for epoch in range(args.epochs):
    sampler.set_epoch(epoch)
    model.train()
    total, correct, loss_sum = 0, 0, 0.0
    for x, y in loader:
        x, y = x.to(device), y.to(device)
        optimizer.zero_grad()
        out = model(x)
        loss = F.cross_entropy(out, y)
        loss.backward()
        optimizer.step()
        total += y.numel()
        correct += (out.argmax(1) == y).sum().item()
        loss_sum += loss.item() * y.numel()
    # average the metrics over ranks
    stats = hvd.allreduce(torch.tensor([loss_sum / total, correct / total]),
                          name="epoch_stats")
    if hvd.rank() == 0:
        print("epoch %d: loss %.4f accuracy %.3f" % (epoch, stats[0], stats[1]), flush=True)
        if args.checkpoint:
            torch.save({"model": model.state_dict(), "optimizer": optimizer.state_dict(),
                        "epoch": epoch}, args.checkpoint)
hvd.shutdown()
