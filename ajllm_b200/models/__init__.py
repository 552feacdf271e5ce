"""Model family: decoder-only Transformer LMs, dense and mixture-of-experts."""

from ajllm_b200.models.attention import SelfAttention
from ajllm_b200.models.factory import build_model, count_parameters, default_d_ff
from ajllm_b200.models.feed_forward import SiLUFeedForward, SwiGLU
from ajllm_b200.models.layers import Embedding, InitSpec, Linear, RMSNorm
from ajllm_b200.models.moe import MoEFeedForward, route_tokens
from ajllm_b200.models.transformer import TransformerBlock, TransformerLM

__all__ = [
    "SelfAttention", "build_model", "count_parameters", "default_d_ff", "SiLUFeedForward", "SwiGLU",
    "Embedding", "InitSpec", "Linear", "RMSNorm", "MoEFeedForward", "route_tokens", "TransformerBlock",
    "TransformerLM",
]
