"""The parts a model is put together from, and their registries.  Importing this package registers
the built-in parts."""
from . import attention, block, depth, latent_attention, mamba2, mlp, moe, norm, rope  # noqa: F401  (registration)
from .cache_need import FixedStateNeed, FixedStateView, PagedKVNeed, PagedKVView, PagedLatentNeed
from .context import BuildContext
from .linear import Linear
from .registry import (register_block, register_combiner, register_feed_forward, register_mixer, register_norm,
                       register_position)
from .spec import (AttentionSpec, DenseActSpec, DepthAverageSpec, LatentAttentionSpec, LayerSpec, Mamba2Spec, ModelSpec,
                   NormSpec, PositionSpec, RoutedExpertsSpec, Stage, SwiGLUSpec, TensorRole)

__all__ = ["FixedStateNeed", "FixedStateView", "PagedKVNeed", "PagedKVView", "PagedLatentNeed", "BuildContext", "Linear",
           "register_combiner", "DenseActSpec", "DepthAverageSpec", "LatentAttentionSpec", "Mamba2Spec",
           "register_block", "register_feed_forward", "register_mixer", "register_norm",
           "register_position", "AttentionSpec", "LayerSpec", "ModelSpec", "NormSpec", "PositionSpec",
           "RoutedExpertsSpec", "Stage", "SwiGLUSpec", "TensorRole"]
