"""Block-scaled fp8 weights for serving.

Weights are stored as e4m3 with one fp32 scale per 128 x 128 block; activations are quantised on
the fly to e4m3 with one scale per token and 128-wide slice of the feature dimension. The product is
``sum_g (x_q[:, g] . w_q[g]) * sx[:, g] * sw[n_block, g]`` with fp32 accumulation. On CUDA this is the
tcgen05 ``kind::f8f6f4`` GEMM with per-128-K rescaled partial accumulators; the CPU path dequantises
and multiplies in fp32 and is the oracle. The reference has no quantisation.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from ajllm_b200.ops import reference

BLOCK = 128


@dataclass
class Fp8Weight:
    q: torch.Tensor          # [out, in] float8_e4m3fn
    scale: torch.Tensor      # [ceil(out/128), ceil(in/128)] fp32
    out_features: int
    in_features: int

    @staticmethod
    def from_dense(weight: torch.Tensor) -> "Fp8Weight":
        q, scale = reference.quantize_weight_fp8_blocks(weight, BLOCK)
        return Fp8Weight(q.contiguous(), scale.contiguous(), weight.shape[0], weight.shape[1])

    def dequantize(self) -> torch.Tensor:
        scale = self.scale.repeat_interleave(BLOCK, 0).repeat_interleave(BLOCK, 1)
        return self.q.float() * scale[: self.out_features, : self.in_features]


def fp8_linear(x: torch.Tensor, weight: Fp8Weight) -> torch.Tensor:
    """``x @ W.T`` with both operands in block-scaled e4m3; returns ``x.dtype``."""
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    if x2.is_cuda:
        from ajllm_b200.ops import fp8 as fp8_ops
        out = fp8_ops.fp8_block_gemm(x2, weight)
    else:
        xq, sx = reference.quantize_activation_fp8_rows(x2, BLOCK)
        out = reference.fp8_block_linear(xq, sx, weight.q, weight.scale, BLOCK).to(x.dtype)
    return out.reshape(*lead, weight.out_features)
