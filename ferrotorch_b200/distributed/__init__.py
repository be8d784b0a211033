"""Distributed runtime: backends, collectives, DDP (CPU control plane); the GPU engines live in ``ferrotorch_b200.parallel``."""
from .backend import (Backend, TcpBackend, SimulatedBackend, SubBackend, FAULT_NONE, FAULT_DROP_NEXT_SEND, FAULT_DELAY_SEND_MS,
                      FAULT_CORRUPT_LENGTH, FAULT_CLOSE)
from .collective import (ReduceOp, DEFAULT_COLLECTIVE_TIMEOUT, allreduce, allreduce_with_timeout, broadcast, all_gather,
                         all_gather_with_timeout, reduce_scatter, reduce_scatter_tensor, reduce_scatter_with_timeout, all_to_all,
                         all_to_all_with_timeout, all_to_all_single_uneven, barrier, send, recv, sendrecv, PendingCollective,
                         async_all_gather, async_reduce_scatter, async_allreduce)
from .ddp import DDP, compute_buckets, DEFAULT_BUCKET_SIZE_BYTES
from ..errors import (DistributedError, InvalidWorldSize, InvalidRank, SelfSend, SizeMismatch, IoError, ChannelClosed, UnsupportedOp,
                      Timeout, NoConnection, BackendUnavailable)
from .extras import (DeviceMesh, Placement, Replicate, Shard, Partial, DTensor, PipelineSchedule, Pipeline, RpcAgent, MAX_RPC_BYTES,
                     ShardingStrategy, FSDP, TensorShardSpec, ShardMetadata, save_distributed, load_distributed, reshard, AsyncCheckpointer)
from .backends_ext import (is_nccl_available, is_gloo_available, is_mpi_available, is_ucc_available, NcclUniqueId, NcclBackend, GlooBackend, MpiBackend,
                           UccBackend, HybridBackend, nccl_allreduce, nccl_broadcast, nccl_all_gather, nccl_reduce_scatter, gpu_allreduce, gpu_broadcast,
                           recv_with_timeout, recv_into, recv_into_with_timeout, RpcError, TcpRpcBackend, DistCheckpointError, DistributedCheckpoint,
                           flat_shard_metadata)
from ..serialize.formats import CheckpointFuture  # noqa: E402


def __getattr__(name):
    if name == "SyncBatchNorm2d":                             # lives with the GPU engines, which import this package: resolve on first use
        from ..parallel.ddp import SyncBatchNorm2d
        return SyncBatchNorm2d
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
