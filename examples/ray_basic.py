"""Running a job from a Ray driver: ``RayExecutor`` places one actor per rank
(here: two hosts with two ranks each, every host on its own node), tells
every actor its coordinates and the rendezvous address, and runs a function
on all of them. Needs the ``ray`` package and a running cluster
(``ray.init(address="auto")``).

Counterpart of the reference's examples/ray/basic_ray_elastic.py and
docs/ray.rst.
"""
import torch

import horovod_b200.torch as hvd
from horovod_b200.ray import ElasticRayExecutor, RayExecutor


def train(steps=10):
    hvd.init()
    model = torch.nn.Linear(8, 1)
    opt = hvd.DistributedOptimizer(torch.optim.SGD(model.parameters(), lr=0.1 * hvd.size()),
                                   named_parameters=model.named_parameters())
    hvd.broadcast_parameters(model.state_dict(), root_rank=0)
    for _ in range(steps):
        opt.zero_grad()
        model(torch.randn(16, 8)).pow(2).mean().backward()
        opt.step()
    result = (hvd.rank(), hvd.size(), float(model.weight.abs().sum()))
    hvd.shutdown()
    return result


def static_job():
    settings = RayExecutor.create_settings(timeout_s=30)
    executor = RayExecutor(settings, num_hosts=2, num_workers_per_host=2, use_gpu=False)
    executor.start()
    try:
        print(executor.run(train, kwargs={"steps": 20}))
    finally:
        executor.shutdown()


def elastic_job():
    # train() would use hvd.elastic.run and a TorchState in a real elastic job
    settings = ElasticRayExecutor.create_settings(min_np=2, max_np=8, elastic_timeout=120)
    executor = ElasticRayExecutor(settings, use_gpu=False, cpus_per_slot=1)
    executor.start()
    print(executor.run(train))


if __name__ == "__main__":
    import ray
    ray.init(address="auto")
    static_job()
