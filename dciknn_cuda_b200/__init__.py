"""B200-native Prioritized DCI k-NN: drop-in for dciknn_cuda's DCI / MDCI.

Reference surface: dciknn_cuda/__init__.py:22 exports DCI and MDCI.
"""
from .core import DCI, MDCI, merge_shards, shard_bounds
from . import tuning

__all__ = ["DCI", "MDCI", "merge_shards", "shard_bounds", "tuning"]
