"""GPU entry points of the serving path: in-place RoPE on packed rows with explicit positions, paged
attention for decode / verify rows, the training flash kernel for prompts that start from an empty
cache, and the batched sampler."""

from __future__ import annotations

import math

import torch

from ajllm_b200.ops import native

_MAX_ROWS = 64


def rope_packed_(qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, positions: torch.Tensor, num_heads: int,
                 num_kv_heads: int, head_dim: int) -> None:
    """Rotate the q and k heads of packed ``[tokens, (Hq + 2 Hkv) * hd]`` rows in place at ``positions``."""
    native.call("ajb_rope_qk", qkv.data_ptr(), cos.data_ptr(), sin.data_ptr(), positions.data_ptr(), qkv.shape[0], 1,
                num_heads, num_kv_heads, head_dim, qkv.stride(0), 0, native.stream_ptr())


class PagedPlan:
    """Launch plan of one ragged decode / verify batch: sequences grouped by their number of new rows, with the
    block tables, row offsets and context lengths of every group already on the device. Built once per engine
    step and reused by every layer."""

    def __init__(self, block_tables: torch.Tensor, q_lens_host: list[int], context_lens_host: list[int], heads: int,
                 kv_heads: int) -> None:
        group = heads // kv_heads
        max_q = max(1, _MAX_ROWS // group)
        classes: dict[int, list[tuple[int, int, int]]] = {}
        cursor = 0
        for i, (n, ctx) in enumerate(zip(q_lens_host, context_lens_host)):
            for a in range(0, n, max_q):
                b = min(n, a + max_q)
                classes.setdefault(b - a, []).append((i, cursor + a, ctx - (n - b)))
            cursor += n
        self.total_rows = cursor
        self.max_context = max(context_lens_host) if context_lens_host else 0
        device = block_tables.device
        self.launches = []
        identity = list(range(block_tables.shape[0]))
        for q_len, items in classes.items():
            rows = [it[0] for it in items]
            tables = block_tables if rows == identity else \
                block_tables.index_select(0, torch.tensor(rows, dtype=torch.long, device=device)).contiguous()
            packed = torch.tensor([[it[1] for it in items], [it[2] for it in items]], dtype=torch.int32, device=device)
            self.launches.append((q_len, len(items), tables, packed[0], packed[1]))


def paged_attention_planned(q: torch.Tensor, key_cache: torch.Tensor, value_cache: torch.Tensor, plan: PagedPlan,
                            scale: float | None = None) -> torch.Tensor:
    """``scale`` defaults to ``1 / sqrt(head width of q)``; callers whose heads are zero-padded pass the true one."""
    total, heads, head_dim = q.shape
    kv_heads = key_cache.shape[2]
    out = torch.empty_like(q)
    scale = 1.0 / math.sqrt(head_dim) if scale is None else scale
    num_blocks, block_size = key_cache.shape[0], key_cache.shape[1]
    for q_len, count, tables, starts, ctxs in plan.launches:
        # few (sequence, KV head) pairs cannot fill the device: cut every sequence's keys over several CTAs, up to
        # two CTAs per SM (what the kernel's shared memory admits) and never more parts than the longest context has
        # 64-key tiles
        max_context = getattr(plan, "max_context", None) or tables.shape[1] * block_size
        splits = paged_splits(count * kv_heads, max_context)
        part_o = part_ml = None
        if splits > 1:
            part_o = torch.empty(total, heads, splits, head_dim, dtype=torch.float32, device=q.device)
            part_ml = torch.empty(total, heads, splits, 2, dtype=torch.float32, device=q.device)
        native.call("ajb_paged_attention", q.data_ptr(), key_cache.data_ptr(), value_cache.data_ptr(), tables.data_ptr(),
                    ctxs.data_ptr(), starts.data_ptr(), out.data_ptr(), count, num_blocks, block_size,
                    tables.shape[1], heads, kv_heads, head_dim, q_len, scale, splits, native.ptr(part_o),
                    native.ptr(part_ml), native.stream_ptr())
    return out


_SM_COUNT: list[int] = []


def paged_splits(ctas: int, max_context: int) -> int:
    """Parts per sequence for the paged-attention kernel given the (sequence, KV head) pairs of a launch."""
    if not _SM_COUNT:
        _SM_COUNT.append(int(native.lib().ajb_sm_count()))
    want = (2 * _SM_COUNT[0]) // max(1, ctas)
    tiles = max(1, (max_context + 63) // 64)
    # a part should keep enough 64-key steps to amortise its start and the merge kernel: 16 steps when the launch
    # already covers half the SMs (measured: 16 sequences x 1024 keys, 24 us whole against 34 us in two parts), 8 below that
    per_part = 16 if 2 * ctas >= _SM_COUNT[0] else 8
    return max(1, min(want, tiles // per_part, 16))


def paged_attention(q: torch.Tensor, key_cache: torch.Tensor, value_cache: torch.Tensor, block_tables: torch.Tensor,
                    context_lens, q_lens, q_lens_host: list[int], context_lens_host: list[int]) -> torch.Tensor:
    """Ragged decode / verify attention. ``q`` is ``[total_rows, Hq, hd]``; launches are grouped by the
    number of new rows per sequence, and long row runs are cut into chunks the kernel can hold."""
    plan = PagedPlan(block_tables, q_lens_host, context_lens_host, q.shape[1], key_cache.shape[2])
    return paged_attention_planned(q, key_cache, value_cache, plan)


def prompt_attention(qkv_rows: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int,
                     scale: float | None = None) -> torch.Tensor:
    """Causal attention of one prompt that starts from an empty cache, read in place from its packed
    (already rotated) ``[T, (Hq + 2 Hkv) * hd]`` rows. Returns ``[T, Hq * hd]``."""
    T, width = qkv_rows.shape
    out = torch.empty(T, num_heads * head_dim, dtype=torch.bfloat16, device=qkv_rows.device)
    lse = torch.empty(num_heads, T, dtype=torch.float32, device=qkv_rows.device)
    native.call("ajb_flash_fwd", qkv_rows.data_ptr(), out.data_ptr(), lse.data_ptr(), 1, T, num_heads, num_kv_heads,
                head_dim, qkv_rows.stride(0), 1, 1.0 / math.sqrt(head_dim) if scale is None else scale,
                native.stream_ptr())
    return out


def sample_rows(logits: torch.Tensor, temperature: torch.Tensor, top_p: torch.Tensor, seeds: torch.Tensor,
                counters: torch.Tensor) -> torch.Tensor:
    """One token per row of fp32 ``logits`` ``[rows, vocab]``; per-row temperature (``<= 0`` = greedy),
    top-p, and a counter-based random stream ``(seed, counter)``. Returns int32 ``[rows]`` on the device."""
    logits = logits.contiguous()
    rows, vocab = logits.shape
    out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    # few rows over a large vocabulary: the row maxima are found by about two CTAs per SM, not one CTA per row
    if not _SM_COUNT:
        _SM_COUNT.append(int(native.lib().ajb_sm_count()))
    chunks = max(1, min(2 * _SM_COUNT[0] // max(1, rows), vocab // 4096, 64))
    workspace = torch.empty(rows, chunks, 2, dtype=torch.int32, device=logits.device) if chunks > 1 else None
    native.call("ajb_sample_rows", logits.data_ptr(), logits.stride(0), rows, vocab,
                temperature.data_ptr(), top_p.data_ptr(), seeds.data_ptr(), counters.data_ptr(), out.data_ptr(),
                chunks, native.ptr(workspace), native.stream_ptr())
    return out


def spec_verify(target_logits: torch.Tensor, draft_logits: torch.Tensor, draft_tokens: torch.Tensor,
                temperature: torch.Tensor, seeds: torch.Tensor, counters: torch.Tensor) -> torch.Tensor:
    """Accept/reject step of speculative decoding for a batch of sequences.

    ``target_logits [seqs, k + 1, vocab]``, ``draft_logits [seqs, k, vocab]`` (fp32), ``draft_tokens [seqs, k]``
    (int32). Returns int32 ``[seqs, 2]`` = (accepted draft tokens, next token)."""
    seqs, k1, vocab = target_logits.shape
    result = torch.empty(seqs, 2, dtype=torch.int32, device=target_logits.device)
    native.call("ajb_spec_verify", target_logits.contiguous().data_ptr(), draft_logits.contiguous().data_ptr(),
                draft_tokens.contiguous().data_ptr(), seqs, k1 - 1, vocab, temperature.data_ptr(), seeds.data_ptr(),
                counters.data_ptr(), result.data_ptr(), native.stream_ptr())
    return result
