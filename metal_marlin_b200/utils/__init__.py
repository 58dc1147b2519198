from .checkpoint import LazyCheckpoint, filter_weights, load_checkpoint, load_sharded_checkpoint, remap_weight_keys, save_checkpoint
from .nan_guard import NaNGuard, NaNStats

__all__ = ["LazyCheckpoint", "filter_weights", "load_checkpoint", "load_sharded_checkpoint", "remap_weight_keys", "save_checkpoint", "NaNGuard",
           "NaNStats"]
