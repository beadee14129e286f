"""Helpers: partition math, dtype tables, configuration, logging, timing."""
from .partition import partition, partition_sizes, max_shard, bus_bandwidth_gbs  # noqa: F401
