"""Hardware-independent Pi0 model description (checkpoint schema, synthetic weights)."""
from .spec import weight_shapes
from .weights import random_checkpoint

__all__ = ["weight_shapes", "random_checkpoint"]
