"""Communicator bring-up and rank worlds."""
from .comm import Comm, World, group, init_emulated_world, init_from_torch_distributed, init_host_memory, init_process
from .hierarchical import HierarchicalComm, HostMemoryOps
from .hierarchical_ep import DeviceEpOps, HierarchicalEP, HostEpOps

__all__ = ["Comm", "DeviceEpOps", "HierarchicalComm", "HierarchicalEP", "HostEpOps", "HostMemoryOps", "World", "group", "init_emulated_world", "init_from_torch_distributed", "init_host_memory", "init_process"]
