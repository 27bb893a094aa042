"""Model-level building blocks that use the communication kernels."""
from .moe import ExpertParallelMoE, MoEConfig

__all__ = ["ExpertParallelMoE", "MoEConfig"]
