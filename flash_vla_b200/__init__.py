"""B200-native Pi0 vision-language-action inference.

    from flash_vla_b200 import Pi0Inference, random_checkpoint

    engine = Pi0Inference(random_checkpoint(), num_views=3, chunk_size=50)
    actions = engine.forward(images, state, noise)

The public names match the reference package (`src/flash_vla/__init__.py:19-34`);
they resolve lazily so that importing the model description alone does not load
the CUDA library.
"""
from __future__ import annotations

__all__ = ["Pi0Inference", "random_checkpoint", "op_table"]


def __getattr__(name: str):
    if name == "random_checkpoint":
        from .models.pi0 import random_checkpoint
        return random_checkpoint
    if name in ("Pi0Inference", "op_table"):
        from .hardware.nvidia.b200 import pi0
        return getattr(pi0, name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
