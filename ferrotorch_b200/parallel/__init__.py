"""Parallelism: flat parameter units, FSDP / DDP / tensor / pipeline parallel engines, collectives, symmetric memory."""
from .flat import FlatUnit, TensorSpec
from .fsdp import FSDP, ShardingStrategy, AdamWConfig
from .ddp import DDP, SyncBatchNorm2d
from .cp import UlyssesAttention, ring_attention
from .p2p import P2PChannel, GpuPipelineStage
from .tp import ColumnParallelLinear, RowParallelLinear, ParallelEmbedding, TpGemmContext

__all__ = ["FlatUnit", "TensorSpec", "FSDP", "ShardingStrategy", "AdamWConfig", "DDP", "SyncBatchNorm2d", "ColumnParallelLinear", "RowParallelLinear",
           "ParallelEmbedding", "TpGemmContext", "UlyssesAttention", "ring_attention", "P2PChannel", "GpuPipelineStage"]
