"""GPU side of the block-scaled fp8 path: per-token activation quantisation and the fp8 GEMM."""

from __future__ import annotations

import os

import torch

from ajllm_b200.ops import native

BLOCK = 128
_K_PARTS = os.environ.get("AJB_FP8_K_PARTS", "1") != "0"      # 0: every tile walks the whole K on its own


def quantize_rows(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """bf16 ``[rows, cols]`` -> (e4m3 ``[rows, cols]``, fp32 scales ``[rows, ceil(cols / 128)]``)."""
    rows, cols = x.shape
    x = x.contiguous()
    q = torch.empty(rows, cols, dtype=torch.float8_e4m3fn, device=x.device)
    scales = torch.empty(rows, (cols + BLOCK - 1) // BLOCK, dtype=torch.float32, device=x.device)
    native.call("ajb_fp8_quantize_rows", x.data_ptr(), q.data_ptr(), scales.data_ptr(), rows, cols, native.stream_ptr())
    return q, scales


def fp8_block_gemm(x: torch.Tensor, weight) -> torch.Tensor:
    """``x @ W.T`` with ``x`` quantised on the fly; ``weight`` is an ``engine.quant.Fp8Weight``."""
    xq, sx = quantize_rows(x.to(torch.bfloat16))
    rows, k = xq.shape
    n = weight.out_features
    out = torch.empty(rows, n, dtype=torch.bfloat16, device=x.device)
    # few rows = few tiles: the K blocks of a tile are then divided over several CTAs whose fp32 parts a second kernel sums
    splits = int(native.lib().ajb_fp8_block_gemm_splits(rows, n, k)) if _K_PARTS else 1
    workspace = torch.empty(splits, rows, n, dtype=torch.float32, device=x.device) if splits > 1 else None
    native.call("ajb_fp8_block_gemm", xq.data_ptr(), weight.q.data_ptr(), sx.data_ptr(), weight.scale.data_ptr(),
                out.data_ptr(), rows, n, k, xq.stride(0), weight.q.stride(0), out.stride(0), splits,
                native.ptr(workspace), native.stream_ptr())
    return out.to(x.dtype)
