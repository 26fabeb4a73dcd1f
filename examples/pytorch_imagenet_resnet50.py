"""ResNet-50 training on an image-folder dataset (or on synthetic images when
no folder is given), the way a real job is set up: per-rank data shards,
learning-rate warm-up scaled by the number of ranks, metrics averaged over
ranks, checkpoints written by rank 0 and resumed by everybody.

    horovodrun -np 8 python examples/pytorch_imagenet_resnet50.py --train-dir /data/train --val-dir /data/val
    horovodrun -np 2 python examples/pytorch_imagenet_resnet50.py --synthetic-samples 256 --epochs 1   # smoke run

Counterpart of the reference's examples/pytorch/pytorch_imagenet_resnet50.py.
"""
import argparse
import math
import os

import torch
import torch.nn.functional as F
import torch.utils.data.distributed

import horovod_b200.torch as hvd
from horovod_b200 import models

parser = argparse.ArgumentParser()
parser.add_argument("--train-dir", default=None, help="image folder; synthetic data when absent")
parser.add_argument("--val-dir", default=None)
parser.add_argument("--synthetic-samples", type=int, default=1024)
parser.add_argument("--image-size", type=int, default=224)
parser.add_argument("--num-classes", type=int, default=1000)
parser.add_argument("--model", default="resnet50", choices=["resnet50", "tiny"],
                    help="tiny: a 4-block ResNet for smoke runs on CPUs")
parser.add_argument("--checkpoint-format", default="./checkpoint-{epoch}.pt")
parser.add_argument("--batch-size", type=int, default=32, help="per rank")
parser.add_argument("--batches-per-allreduce", type=int, default=1,
                    help="local gradient accumulation before each allreduce")
parser.add_argument("--epochs", type=int, default=90)
parser.add_argument("--base-lr", type=float, default=0.0125, help="per rank")
parser.add_argument("--warmup-epochs", type=float, default=5)
parser.add_argument("--momentum", type=float, default=0.9)
parser.add_argument("--wd", type=float, default=5e-5)
parser.add_argument("--fp16-allreduce", action="store_true")
parser.add_argument("--use-adasum", action="store_true")
parser.add_argument("--gradient-predivide-factor", type=float, default=1.0)
parser.add_argument("--no-cuda", action="store_true")
parser.add_argument("--seed", type=int, default=42)
args = parser.parse_args()

hvd.init()
torch.manual_seed(args.seed)
cuda = not args.no_cuda and torch.cuda.is_available()
if cuda:
    torch.cuda.set_device(hvd.local_rank())
    torch.backends.cudnn.benchmark = True
device = torch.device("cuda", hvd.local_rank()) if cuda else torch.device("cpu")
allreduce_batch = args.batch_size * args.batches_per_allreduce


def dataset(folder, samples):
    if folder:
        from torchvision import datasets, transforms  # only needed with real data
        return datasets.ImageFolder(folder, transforms.Compose([
            transforms.RandomResizedCrop(args.image_size), transforms.RandomHorizontalFlip(),
            transforms.ToTensor(),
            transforms.Normalize([0.485, 0.456, 0.406], [0.229, 0.224, 0.225])]))
    g = torch.Generator().manual_seed(args.seed)
    return torch.utils.data.TensorDataset(
        torch.randn(samples, 3, args.image_size, args.image_size, generator=g),
        torch.randint(0, args.num_classes, (samples,), generator=g))


train_set = dataset(args.train_dir, args.synthetic_samples)
val_set = dataset(args.val_dir, max(args.synthetic_samples // 4, hvd.size()))
# Every rank reads its own shard of every epoch.
train_sampler = torch.utils.data.distributed.DistributedSampler(
    train_set, num_replicas=hvd.size(), rank=hvd.rank())
val_sampler = torch.utils.data.distributed.DistributedSampler(
    val_set, num_replicas=hvd.size(), rank=hvd.rank())
train_loader = torch.utils.data.DataLoader(train_set, batch_size=allreduce_batch,
                                           sampler=train_sampler, pin_memory=cuda)
val_loader = torch.utils.data.DataLoader(val_set, batch_size=args.batch_size,
                                         sampler=val_sampler, pin_memory=cuda)

build = models.resnet50 if args.model == "resnet50" else models.resnet_tiny
model = build(num_classes=args.num_classes).to(device)
# Adasum does not need the learning rate scaled by the number of ranks (only by
# the ranks that sum before Adasum combines: none on this single-level setup).
lr_scaler = args.batches_per_allreduce * (1 if args.use_adasum else hvd.size())
optimizer = torch.optim.SGD(model.parameters(), lr=args.base_lr * lr_scaler,
                            momentum=args.momentum, weight_decay=args.wd)
optimizer = hvd.DistributedOptimizer(
    optimizer, named_parameters=model.named_parameters(),
    compression=hvd.Compression.fp16 if args.fp16_allreduce else hvd.Compression.none,
    backward_passes_per_step=args.batches_per_allreduce,
    op=hvd.Adasum if args.use_adasum else hvd.Average,
    gradient_predivide_factor=args.gradient_predivide_factor)

# Resume from the newest checkpoint; rank 0 looks, everybody learns the answer.
resume_from_epoch = 0
if hvd.rank() == 0:
    for epoch in range(args.epochs, 0, -1):
        if os.path.exists(args.checkpoint_format.format(epoch=epoch)):
            resume_from_epoch = epoch
            break
resume_from_epoch = int(hvd.broadcast(torch.tensor(resume_from_epoch), root_rank=0,
                                      name="resume_from_epoch"))
if resume_from_epoch > 0 and hvd.rank() == 0:
    saved = torch.load(args.checkpoint_format.format(epoch=resume_from_epoch))
    model.load_state_dict(saved["model"])
    optimizer.load_state_dict(saved["optimizer"])
hvd.broadcast_parameters(model.state_dict(), root_rank=0)
hvd.broadcast_optimizer_state(optimizer, root_rank=0)


def adjust_learning_rate(epoch, batch_idx):
    """Linear warm-up from the single-rank rate to the scaled rate, then the
    usual step decay at epochs 30, 60 and 80."""
    if epoch < args.warmup_epochs:
        progress = (epoch + float(batch_idx + 1) / len(train_loader)) / args.warmup_epochs
        factor = 1.0 / hvd.size() * (progress * (hvd.size() - 1) + 1)
    else:
        factor = 10.0 ** -sum(epoch >= e for e in (30, 60, 80))
    for group in optimizer.param_groups:
        group["lr"] = args.base_lr * lr_scaler * factor


class Metric:
    """Running average of a per-batch value, averaged over the ranks."""

    def __init__(self, name):
        self.name, self.sum, self.n = name, 0.0, 0

    def update(self, value):
        self.sum += float(hvd.allreduce(value.detach().cpu(), name=self.name))
        self.n += 1

    @property
    def avg(self):
        return self.sum / max(self.n, 1)


def accuracy(output, target):
    return output.argmax(dim=1).eq(target).float().mean()


def train(epoch):
    model.train()
    train_sampler.set_epoch(epoch)
    loss_m, acc_m = Metric("train_loss"), Metric("train_accuracy")
    for batch_idx, (data, target) in enumerate(train_loader):
        adjust_learning_rate(epoch, batch_idx)
        data, target = data.to(device, non_blocking=True), target.to(device, non_blocking=True)
        optimizer.zero_grad()
        # One allreduce per `batches_per_allreduce` micro-batches.
        for i in range(0, len(data), args.batch_size):
            chunk, labels = data[i:i + args.batch_size], target[i:i + args.batch_size]
            output = model(chunk)
            loss = F.cross_entropy(output, labels)
            acc_m.update(accuracy(output, labels))
            loss_m.update(loss)
            (loss / math.ceil(len(data) / args.batch_size)).backward()
        optimizer.step()
    if hvd.rank() == 0:
        print("epoch %d train loss %.4f accuracy %.4f" % (epoch + 1, loss_m.avg, acc_m.avg),
              flush=True)


def validate(epoch):
    model.eval()
    loss_m, acc_m = Metric("val_loss"), Metric("val_accuracy")
    with torch.no_grad():
        for data, target in val_loader:
            data, target = data.to(device), target.to(device)
            output = model(data)
            loss_m.update(F.cross_entropy(output, target))
            acc_m.update(accuracy(output, target))
    if hvd.rank() == 0:
        print("epoch %d val loss %.4f accuracy %.4f" % (epoch + 1, loss_m.avg, acc_m.avg),
              flush=True)


for epoch in range(resume_from_epoch, args.epochs):
    train(epoch)
    validate(epoch)
    if hvd.rank() == 0:
        torch.save({"model": model.state_dict(), "optimizer": optimizer.state_dict()},
                   args.checkpoint_format.format(epoch=epoch + 1))
hvd.shutdown()
