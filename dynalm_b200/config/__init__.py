from .llama import LlamaConfig, RopeScaling
from .plan import (BlockSpec, EmbeddingSpec, FeedForwardSpec, HeadSpec, LayerRun, MixerSpec,
                   ModelPlan, NormSpec, PositionSpec)
from .reader import KeyReader, read_json_file

__all__ = ["LlamaConfig", "RopeScaling", "BlockSpec", "EmbeddingSpec", "FeedForwardSpec", "HeadSpec",
           "LayerRun", "MixerSpec", "ModelPlan", "NormSpec", "PositionSpec", "KeyReader", "read_json_file"]
