"""Parallelism and communication (crates/axonml-distributed): backends, process groups,
collectives, DistributedDataParallel, FullyShardedDataParallel (ZeRO-2/3), tensor and pipeline
parallelism, launcher."""
from .backend import (Backend, CommTimeout, CpuBackend, MockBackend, NcclBackend, ReduceOp,
                      init_from_env)
from .comm import (all_gather, all_reduce_max, all_reduce_mean, all_reduce_min, all_reduce_product,
                   all_reduce_sum, barrier, broadcast, broadcast_from, gather_tensor,
                   is_main_process, rank, reduce_scatter_mean, reduce_scatter_sum, ring_all_reduce,
                   scatter_tensor, sync_gradient, sync_gradients, world_size)
from .ddp import (DDP, DistributedDataParallel, GradientBucket, GradientSynchronizer,
                  GradSyncStrategy)
from .fsdp import (FSDP, CPUOffload, FSDPMemoryStats, FullyShardedDataParallel, ShardingStrategy)
from .process_group import ProcessGroup, World
from .pipeline import Pipeline, PipelineMemoryStats, PipelineSchedule, PipelineStage
from .tensor_parallel import (ColumnParallelLinear, RowParallelLinear, VocabParallelEmbedding,
                              vocab_parallel_cross_entropy)
from .mesh import DeviceMesh
from .checkpoint import load_sharded, save_sharded
from .context_parallel import (UlyssesAttention, allgather_kv_attention, ring_attention, shard_sequence,
                               ulysses_attention)
