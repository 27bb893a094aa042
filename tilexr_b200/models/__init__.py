"""Model-level building blocks that use the communication kernels."""
from .moe import ExpertParallelMoE, MoEConfig

__all__ = ["ExpertParallelMoE", "MoEConfig"]
from .tp_mlp import SequenceParallelMLP, TPMlpConfig, shard_weights  # noqa: F401
