from mini_train_sys_b200.models.blocks import (CausalSelfAttention, DenseFeedForward, FeedForwardOutput,
                                               MoEFeedForward, RMSNorm, SwiGLUMLP, TransformerBlock)
from mini_train_sys_b200.models.config import ModelConfig, MoEModelConfig
from mini_train_sys_b200.models.ops import OpsBackend, RouterPostprocessOutput, get_ops_backend
from mini_train_sys_b200.models.rotary import RotaryEmbedding
from mini_train_sys_b200.models.router import RouterOutput, TopKRouter
from mini_train_sys_b200.models.transformer import MiniMoETransformer, MiniTransformer

__all__ = [
    "CausalSelfAttention", "DenseFeedForward", "FeedForwardOutput", "MoEFeedForward", "RMSNorm", "SwiGLUMLP",
    "TransformerBlock", "ModelConfig", "MoEModelConfig", "OpsBackend", "RouterPostprocessOutput",
    "get_ops_backend", "RotaryEmbedding", "RouterOutput", "TopKRouter", "MiniMoETransformer", "MiniTransformer",
]
