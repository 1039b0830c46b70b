"""B200 execution target for Pi0."""
from .engine import Pi0Inference
from .ops import op_names, op_table

__all__ = ["Pi0Inference", "op_table", "op_names"]
