"""Elastic training: the job survives workers leaving and joining.

    horovodrun -np 2 --min-np 1 --max-np 4 --host-discovery-script ./discover.sh \
        python examples/pytorch_elastic.py

State (model, optimizer, epoch, batch) is committed every few batches; after a
failure the survivors restore the last commit, re-rendezvous with whatever
workers exist now, and rank 0 broadcasts its state.
"""
import torch
import torch.nn.functional as F

import horovod_b200.torch as hvd

hvd.init()
torch.manual_seed(0)
model = torch.nn.Sequential(torch.nn.Linear(32, 64), torch.nn.ReLU(), torch.nn.Linear(64, 4))
base_lr = 0.05
optimizer = torch.optim.SGD(model.parameters(), lr=base_lr * hvd.size())
optimizer = hvd.DistributedOptimizer(optimizer, named_parameters=model.named_parameters())

g = torch.Generator().manual_seed(1)
xs, ys = torch.randn(2048, 32, generator=g), torch.randint(0, 4, (2048,), generator=g)
dataset = torch.utils.data.TensorDataset(xs, ys)
sampler = hvd.elastic.ElasticSampler(dataset, shuffle=True)
loader = torch.utils.data.DataLoader(dataset, batch_size=32, sampler=sampler)


@hvd.elastic.run
def train(state):
    for state.epoch in range(state.epoch, 5):
        for batch_idx, (x, y) in enumerate(loader):
            optimizer.zero_grad()
            F.cross_entropy(model(x), y).backward()
            optimizer.step()
            state.sampler.record_batch(batch_idx, 32)
            if batch_idx % 10 == 0:
                state.commit()
        if hvd.rank() == 0:
            print("epoch %d done on %d rank(s)" % (state.epoch, hvd.size()), flush=True)
        state.sampler.set_epoch(state.epoch + 1)
        state.commit()


def on_reset():
    # keep the per-sample learning rate constant when the world size changes
    for group in optimizer.param_groups:
        group["lr"] = base_lr * hvd.size()


state = hvd.elastic.TorchState(model=model, optimizer=optimizer, sampler=sampler, epoch=0)
state.register_reset_callbacks([on_reset])
train(state)
hvd.shutdown()
