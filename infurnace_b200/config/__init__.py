"""Typed configurations and the plain-data description of a model (no torch needed)."""
from .specs import (  # noqa: F401
    TensorSpec, KVCacheNeed, StateNeed, RMSNormSpec, RotarySpec, AttentionSpec, GatedMLPSpec,
    PreNormBlockSpec, EmbeddingSpec, LMHeadSpec, LayerCall, ModelPlan,
    ScalarRMSNormSpec, SinusoidEmbeddingSpec, DenseMLPSpec, GatedRecurrenceSpec, TalkingAttentionSpec, PostNormBlockSpec,
    NormedEmbeddingSpec, StreamInjectSpec, RetentionSpec, TimeMixSpec, GatedUnitSpec, RotaryValueAttentionSpec,
    ParallelMixerSpec, RoutedExpertsSpec, TokenSideSpec, SandwichBlockSpec,
    PagedStream, PagedCacheNeed, GroupRMSNormSpec, CausalConvSpec, LatentAttentionSpec, DepthAverageBlockSpec,
    RealGatedRecurrenceSpec,
)
from .qwen3 import Qwen3Config  # noqa: F401
from .kafunex import KafunexConfig  # noqa: F401
from .lunelorn import LunelornConfig  # noqa: F401
from .filorax import FiloraxConfig  # noqa: F401
from .golonex import GolonexConfig  # noqa: F401
