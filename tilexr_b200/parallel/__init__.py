"""Communicator bring-up and rank worlds."""
from .comm import Comm, World, group, init_emulated_world, init_from_torch_distributed, init_host_memory, init_process
from .hierarchical import HierarchicalComm, HostMemoryOps

__all__ = ["Comm", "HierarchicalComm", "HostMemoryOps", "World", "group", "init_emulated_world", "init_from_torch_distributed", "init_host_memory", "init_process"]
