"""Parts a model is put together from.  Importing the package registers the built-in kinds."""
from . import attention, block, embedding, latent_attention, linear_attention, mlp, norm, projected, rope  # noqa: F401
from .base import (Block, CacheView, Embedding, FeedForward, Head, KVCacheSpec, LatentCacheSpec, Mixer, Norm, ParamSpec, Part, PositionEncoding,
                   ResidualStream, Runtime, StateLayout, StateSpec, PagedLayout, build_part, register_cache_kind, register_part,
                   unregister_cache_kind, unregister_part)
from .specs import (AttentionSpec, BlockSpec, DeltaRuleSpec, DifferentialAttentionSpec, EmbeddingSpec, ExpertsSpec, FeedForwardSpec,
                    GatedDeltaSpec, GatedLinearAttentionSpec, GatedMLPSpec, LatentAttentionSpec, MatrixMemorySpec, NormedParallelSpec, LightningSpec, RetentionSpec, XieluMLPSpec,
                    HeadSpec, MixerSpec, ModelSpec, NormSpec, ParallelSpec, PolyNormMLPSpec, PositionSpec, RunSpec)
from .projected import ProjectedMixer
