"""Inference engine: paged KV cache, continuous batching, sampling, speculative decoding, fp8 weights."""

from ajllm_b200.engine.kv_cache import BlockAllocator, OutOfBlocks, PagedKVCache
from ajllm_b200.engine.scheduler import SamplingParams, Scheduler, Sequence, SeqStatus

__all__ = ["BlockAllocator", "OutOfBlocks", "PagedKVCache", "SamplingParams", "Scheduler", "Sequence", "SeqStatus"]

from ajllm_b200.engine.engine import EngineStats, LLMEngine, RequestOutput  # noqa: E402
from ajllm_b200.engine.quant import Fp8Weight, fp8_linear  # noqa: E402

__all__ += ["EngineStats", "LLMEngine", "RequestOutput", "Fp8Weight", "fp8_linear"]
