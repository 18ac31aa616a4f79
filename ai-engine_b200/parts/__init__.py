from .attention import ATTENTION_WORK, AttentionWork, GQAAttention
from .base import (Block, BuildEnv, CacheNeed, FeedForward, KVRequest, LayerCache, Mixer, Norm, Part,
                   PositionEncoding, StateRequest, StepPlanner)
from .block import PreNormBlock
from .embedding import LMHead, TokenEmbedding
from .mlp import SwiGLU
from .model import Layer, Model, tensor_specs_of
from .norm import RMSNorm
from .registry import (lookup, register, register_block, register_feed_forward, register_mixer,
                       register_norm, register_position_encoding)
from .rope import RotaryEncoding, rotary_inv_freq
from .spec import LayerSpec, ModelSpec, PartSpec, RunStep

register("mixer", "gqa_attention", GQAAttention)
register("feed_forward", "swiglu", SwiGLU)
register("norm", "rmsnorm", RMSNorm)
register("position_encoding", "rotary", RotaryEncoding)
register("block", "prenorm", PreNormBlock)
register("embedding", "token_embedding", TokenEmbedding)
register("head", "lm_head", LMHead)

__all__ = ["ATTENTION_WORK", "AttentionWork", "GQAAttention", "Block", "BuildEnv", "CacheNeed", "FeedForward",
           "KVRequest", "LayerCache", "Mixer", "Norm", "Part", "PositionEncoding", "StateRequest", "StepPlanner", "PreNormBlock", "LMHead",
           "TokenEmbedding", "SwiGLU", "Layer", "Model", "tensor_specs_of", "RMSNorm", "lookup",
           "register", "register_block", "register_feed_forward", "register_mixer",
           "register_norm", "register_position_encoding", "RotaryEncoding", "rotary_inv_freq",
           "LayerSpec", "ModelSpec", "PartSpec", "RunStep"]
