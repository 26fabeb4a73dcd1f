"""Elastic training loop used by the integration tests. Logs one JSON line per
finished epoch and can fail on purpose: --exit-at "epoch:hostname:local_rank"
makes that worker exit with code 1 at the start of that epoch (once)."""
import argparse
import json
import os
import sys
import time

import torch

import horovod_b200.torch as hvd

p = argparse.ArgumentParser()
p.add_argument("--log", required=True)
p.add_argument("--epochs", type=int, default=6)
p.add_argument("--batches", type=int, default=4)
p.add_argument("--exit-at", default="")
p.add_argument("--sleep", type=float, default=0.15)
args = p.parse_args()

hvd.init()
torch.manual_seed(0)
model = torch.nn.Linear(4, 2)
opt = hvd.DistributedOptimizer(torch.optim.SGD(model.parameters(), lr=0.01),
                               named_parameters=model.named_parameters())
host = os.environ.get("HOROVOD_HOSTNAME", "")
lrank = os.environ.get("HOROVOD_LOCAL_RANK", "")


@hvd.elastic.run
def train(state):
    while state.epoch < args.epochs:
        if args.exit_at:
            e, h, lr = args.exit_at.split(":")
            marker = args.log + ".exited"
            if state.epoch == int(e) and host == h and lrank == lr and not os.path.exists(marker):
                open(marker, "w").close()
                os._exit(1)
        while state.batch < args.batches:
            opt.zero_grad()
            loss = model(torch.ones(3, 4)).sum()
            loss.backward()
            opt.step()
            time.sleep(args.sleep)
            state.batch += 1
            state.commit()
        with open(args.log, "a") as f:
            f.write(json.dumps({"epoch": state.epoch, "rank": hvd.rank(), "size": hvd.size(),
                                "host": host}) + "\n")
        state.batch = 0
        state.epoch += 1
        state.commit()


state = hvd.elastic.TorchState(model=model, optimizer=opt, epoch=0, batch=0)
train(state)
hvd.shutdown()
sys.exit(0)
