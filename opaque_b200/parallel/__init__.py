"""Multi-GPU building blocks over NVLink / NVSwitch peer memory.

``peer``     – peer-mapped buffers (CUDA IPC handles exchanged through ``torch.distributed``),
               device tables of peer pointers, and the bounded-wait flag barrier.
``sharded``  – the flat parameter space: bf16 parameters replicated in every rank's peer
               buffer, fp32 gradient / master / Adam / DP-FTRL state sharded 1/W per rank,
               and the fused reduce-scatter → noise → AdamW-BC → all-gather step.
"""
from .peer import PeerBuffer, PeerGroup
from .sharded import FlatSpace, ShardedDPOptimizer

__all__ = ["FlatSpace", "PeerBuffer", "PeerGroup", "ShardedDPOptimizer"]
