"""Ops layer: oracle math (CPU) and sm_100a kernels (CUDA) behind one functional API."""

from ajllm_b200.ops import native, reference
from ajllm_b200.ops.functional import (
    add_rms_norm,
    cross_entropy,
    eager_cuda,
    embedding,
    gemm,
    gemm_batched,
    linear,
    linear_batched,
    linear_cross_entropy,
    linear_swiglu,
    paged_attention_ragged,
    rms_norm,
    rope_attention,
    silu,
    split_packed_qkv,
    swiglu_ffn,
    swiglu_ffn_batched,
    swiglu_interleaved,
)

__all__ = [
    "native", "reference", "eager_cuda", "add_rms_norm", "cross_entropy", "embedding", "gemm", "linear",
    "linear_cross_entropy", "linear_swiglu", "paged_attention_ragged", "rms_norm", "rope_attention", "silu", "split_packed_qkv", "swiglu_ffn", "swiglu_ffn_batched", "swiglu_interleaved",
]
