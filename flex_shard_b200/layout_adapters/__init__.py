"""Adapters from other frameworks' sharding annotations to ``GlobalLayout``."""
from .dtensor import dtensor_layout, dtensor_to_global_layout
from .spmd_types import spmd_layout, spmd_types_to_global_layout
