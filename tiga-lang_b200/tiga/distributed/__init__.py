"""Destination-partitioned execution: partition model and halo runtime."""
from .model import (ByDestination, DeviceMesh, GraphPlacement, HaloMap, derive_halo_map, destination_owner,
                    owned_range, partition_bounds)

__all__ = ["ByDestination", "DeviceMesh", "DistributedRuntime", "GraphPlacement", "HaloMap", "NCCLTransport",
           "ProcessGroupTransport", "derive_halo_map", "destination_owner", "owned_range", "partition_bounds"]


def __getattr__(name):
    # the runtime imports torch.distributed and the Graph class: load it on first use
    if name in {"DistributedRuntime", "NCCLTransport", "ProcessGroupTransport", "current_distributed_runtime",
                "execute_sharded_message_passing", "halo_weighted_sum", "shard_plan_for", "build_shard_plan"}:
        from . import runtime

        return getattr(runtime, name)
    raise AttributeError(name)
