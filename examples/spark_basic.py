"""Running a job on the executors of a Spark cluster: ``horovod_b200.spark.run``
starts one barrier task per rank, gives every task its coordinates and the
rendezvous address of the driver, runs the function and returns the results
ordered by rank. Needs ``pyspark`` 3.0 or newer and an active SparkContext.

Counterpart of the reference's docs/spark.rst ("horovod.spark.run").
"""
import torch

import horovod_b200.spark
import horovod_b200.torch as hvd


def train(magic_number):
    hvd.init()
    total = hvd.allreduce(torch.tensor([float(hvd.rank() + magic_number)]), op=hvd.Sum)
    out = (hvd.rank(), hvd.size(), float(total))
    hvd.shutdown()
    return out


if __name__ == "__main__":
    from pyspark.sql import SparkSession
    spark = SparkSession.builder.appName("horovod_b200 on spark").getOrCreate()
    print(horovod_b200.spark.run(train, args=(42,), num_proc=2))
    spark.stop()
