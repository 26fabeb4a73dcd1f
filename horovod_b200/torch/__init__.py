"""``import horovod_b200.torch as hvd`` — the PyTorch API.

Parity: horovod/torch/__init__.py:34-54.
"""
import horovod_b200 as _pkg
from horovod_b200.common.util import check_extension

# Fails with a build hint instead of an obscure import error further down
# (horovod/torch/__init__.py:17-31).
check_extension("horovod_b200.torch", "HOROVOD_WITH_PYTORCH", _pkg.__file__, "_C")

from horovod_b200.common.exceptions import (HorovodInternalError, HostsUpdatedInterrupt,  # noqa: E402
                                             WorkerRemovedError)
from horovod_b200.common.process_sets import (ProcessSet, add_process_set,
                                              global_process_set, process_set_ids,
                                              remove_process_set)
from horovod_b200.torch import elastic
from horovod_b200.torch.compression import Compression
from horovod_b200.torch.functions import (allgather_object, broadcast_object,
                                          broadcast_optimizer_state, broadcast_parameters)
from horovod_b200.torch.mpi_ops import (Adasum, Average, Max, Min, Product, Sum, allgather,
                                        allgather_async, allreduce, allreduce_, barrier,
                                        grouped_allgather, grouped_reducescatter,
                                        grouped_allgather_async, grouped_reducescatter_async,
                                        allreduce_async, allreduce_async_, alltoall,
                                        alltoall_async, broadcast, broadcast_,
                                        broadcast_async, broadcast_async_, ccl_built,
                                        cross_rank, cross_size, cuda_built, ddl_built,
                                        gloo_built, gloo_enabled, gpu_backend,
                                        grouped_allreduce, grouped_allreduce_,
                                        grouped_allreduce_async, grouped_allreduce_async_,
                                        init, is_homogeneous, is_initialized, join,
                                        local_rank, local_size, mpi_built, mpi_enabled,
                                        mpi_threads_supported, nccl_built, poll, rank,
                                        reducescatter, reducescatter_async, rocm_built,
                                        runtime_params,
                                        shutdown, size, sparse_allreduce_async,
                                        start_timeline, stop_timeline, symmetric_empty,
                                        synchronize, topology, set_shadow_check, ShadowMismatch)
from horovod_b200.torch.fused_sgd import FusedSGD
from horovod_b200.torch.optimizer import DistributedOptimizer
from horovod_b200.torch.sync_batch_norm import SyncBatchNorm
