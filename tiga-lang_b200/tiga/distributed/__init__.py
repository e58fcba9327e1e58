"""Destination-partitioned execution: partition model and halo runtime."""
from .model import (ByDestination, DeviceMesh, GraphPlacement, HaloMap, derive_halo_map, destination_owner,
                    owned_range, partition_bounds)

__all__ = ["ByDestination", "DeviceMesh", "GraphPlacement", "HaloMap", "derive_halo_map",
           "destination_owner", "owned_range", "partition_bounds"]
