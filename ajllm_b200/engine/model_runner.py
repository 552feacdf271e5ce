"""Runs a :class:`~ajllm_b200.models.TransformerLM` in serving mode over a paged KV cache.

One call processes a ragged batch: every scheduled sequence contributes ``n_i`` new tokens (a prompt
chunk, one decode token, or ``k+1`` tokens of a speculative verify). Keys and values of the new tokens
are written to the sequence's cache slots and each new token attends to everything cached for its
sequence up to and including itself. Under tensor parallelism activations are replicated, every rank
holds its own heads of the cache, and the two row-parallel projections end in an all-reduce.
Weights may be bf16 tensors or block-scaled fp8 (:mod:`ajllm_b200.engine.quant`).

Pure decoding steps (one new token per sequence) are replayed from CUDA graphs: a step is a few hundred short
kernels, and launching them one by one costs more host time than they run. One graph per batch-size bucket is
captured on first use over static input buffers (token ids, positions, cache slots, block tables, context
lengths); a step copies its inputs into those buffers and replays. Rows that pad a batch up to its bucket read
and write a scratch cache block that no sequence owns. Under tensor parallelism the graphs contain the fused
GEMM -> all-reduce kernels: their call numbers and arrival counts live in device memory and advance with every
execution, captured or not, so every rank replays the same graph and the kernels pair up as in eager mode
(NCCL collectives are not captured: without the fused kernels, tensor-parallel decoding launches step by step).
"""

from __future__ import annotations

import os
from dataclasses import dataclass

import torch

from ajllm_b200 import ops
from ajllm_b200.engine.kv_cache import PagedKVCache
from ajllm_b200.engine.quant import Fp8Weight, fp8_linear
from ajllm_b200.models.moe import MoEFeedForward
from ajllm_b200.ops import reference


@dataclass
class RunItem:
    seq_id: int
    token_ids: list[int]
    num_logits: int          # how many trailing positions need logits (0 = none)


def _matmul(x: torch.Tensor, weight) -> torch.Tensor:
    if isinstance(weight, Fp8Weight):
        return fp8_linear(x, weight)
    return ops.linear(x, weight)


class DecodeStaging:
    """Host side of a replayed decoding step: token ids, positions, cache slots, context lengths and block tables of
    the step, kept in two host arrays that persist across steps (pinned when a GPU is present) so that a step costs
    two host-to-device copies and no allocation. Block-table rows are rewritten only for rows whose sequence changed;
    a row that keeps its sequence only gets the blocks appended since the previous step."""

    def __init__(self, bucket: int, q_len: int, max_blocks: int, scratch_block: int, block_size: int, pinned: bool) -> None:
        self.bucket, self.q_len, self.max_blocks = bucket, q_len, max_blocks
        self.scratch_block, self.block_size = scratch_block, block_size
        rows = bucket * q_len
        self.rows = torch.zeros(3, rows, dtype=torch.long, pin_memory=pinned)                  # ids, positions, slots
        self.meta = torch.zeros(bucket * (1 + max_blocks), dtype=torch.int32, pin_memory=pinned)   # ctx, then tables
        self._rows = self.rows.numpy()
        self._ctx = self.meta.numpy()[:bucket]
        self._tables = self.meta.numpy()[bucket:].reshape(bucket, max_blocks)
        self._tables[:] = scratch_block
        self._row_table = [None] * bucket        # block table (object) a row mirrors, and how often it had shrunk then
        self._row_shrinks = [0] * bucket
        self._row_blocks = [0] * bucket          # how many of its blocks are written

    def fill(self, items, cache) -> None:
        """Stages one step; reserves the cache slots of the new tokens (``cache.append_slots``)."""
        q_len, n = self.q_len, len(items)
        rows, ctx, tables = self._rows, self._ctx, self._tables
        block_size = self.block_size
        for i, item in enumerate(items):
            seq_id = item.seq_id
            start = cache.length(seq_id)
            slots = cache.append_slots(seq_id, q_len)
            lo = i * q_len
            if q_len == 1:
                rows[0, lo] = item.token_ids[0]
                rows[1, lo] = start
                rows[2, lo] = slots[0]
            else:
                rows[0, lo:lo + q_len] = item.token_ids
                rows[1, lo:lo + q_len] = range(start, start + q_len)
                rows[2, lo:lo + q_len] = slots
            ctx[i] = start + q_len
            table = cache.tables[seq_id]
            blocks = table.blocks
            # same table object and no block given back since (rejected draft tokens, preemption): only new blocks
            same = self._row_table[i] is table and self._row_shrinks[i] == table.shrinks
            have = self._row_blocks[i] if same else 0
            if have != len(blocks) or not same:
                tables[i, have:len(blocks)] = blocks[have:]
                self._row_table[i], self._row_shrinks[i], self._row_blocks[i] = table, table.shrinks, len(blocks)
        # padding rows: q_len tokens of nothing in the scratch block
        for i in range(n, self.bucket):
            if self._row_table[i] is not None or ctx[i] != q_len:
                lo = i * q_len
                rows[0, lo:lo + q_len] = 0
                rows[1, lo:lo + q_len] = range(q_len)
                rows[2, lo:lo + q_len] = range(self.scratch_block * block_size, self.scratch_block * block_size + q_len)
                ctx[i] = q_len
                tables[i, 0] = self.scratch_block
                self._row_table[i], self._row_blocks[i] = None, 0


class _DecodeGraph:
    """Static buffers and the captured graph of one (batch-size bucket, new tokens per sequence) pair: one new token
    for plain decoding, ``k + 1`` for the verification pass of speculative decoding."""

    def __init__(self, bucket: int, q_len: int, max_blocks: int, device: torch.device, scratch_block: int,
                 block_size: int) -> None:
        self.bucket, self.q_len = bucket, q_len
        rows = bucket * q_len
        self.staging = DecodeStaging(bucket, q_len, max_blocks, scratch_block, block_size, pinned=device.type == "cuda")
        self.rows = torch.zeros(3, rows, dtype=torch.long, device=device)
        self.ids, self.pos, self.slots = self.rows[0], self.rows[1], self.rows[2]
        self.pos32 = torch.zeros(rows, dtype=torch.int32, device=device)
        self.meta = torch.zeros(bucket * (1 + max_blocks), dtype=torch.int32, device=device)
        self.ctx = self.meta[:bucket]
        self.tables = self.meta[bucket:].view(bucket, max_blocks)
        self.starts = torch.arange(bucket, dtype=torch.int32, device=device) * q_len
        self.logits: torch.Tensor | None = None
        self.graph: torch.cuda.CUDAGraph | None = None

    def upload(self) -> None:
        self.rows.copy_(self.staging.rows, non_blocking=True)
        self.meta.copy_(self.staging.meta, non_blocking=True)


class ModelRunner:
    FUSED_ALL_REDUCE_MAX_ROWS = 2048     # beyond this the partial tiles (tp copies per rank) outgrow the win
    GRAPH_BUCKETS = (1, 2, 4, 8, 16, 32, 64, 128, 256)

    def __init__(self, model, cache: PagedKVCache, quantization: str | None = None) -> None:
        self.model = model
        self.cache = cache
        self.tp = getattr(model, "tp", None)
        self.device = next(model.parameters()).device
        self.dtype = next(model.parameters()).dtype
        if model.norm_placement != "pre":
            raise ValueError("the serving engine supports pre-norm models")
        # GPU kernels run at 64- or 128-wide heads: other head sizes are zero-padded after the rotation, cached padded,
        # and the attention output is cut back (the softmax scale stays that of the true head size)
        attn0 = model.layers[0].attention
        self.head_dim = attn0.head_dim
        self.kernel_head_dim = cache.head_dim
        self.softmax_scale = 1.0 / (self.head_dim ** 0.5)
        self.weights = []
        for layer in model.layers:
            entry = {"qkv": layer.attention.qkv_proj.data, "out": layer.attention.output_proj.data}
            ff = layer.feed_forward
            if isinstance(ff, MoEFeedForward):
                entry["moe"] = ff
            elif hasattr(ff, "w13"):
                entry["w13"], entry["w2"] = ff.w13.data, ff.w2.data
            else:
                entry["w1"], entry["w2"] = ff.w1.data, ff.w2.data
            if quantization == "fp8":
                for key in ("qkv", "out", "w13", "w2", "w1"):
                    if key in entry:
                        entry[key] = Fp8Weight.from_dense(entry[key])
            elif quantization not in (None, "none", "bf16"):
                raise ValueError(f"unknown quantization '{quantization}'")
            self.weights.append(entry)
        # decoding graphs: dense feed-forward blocks (expert routing has data-dependent shapes); with several ranks only
        # when every row-parallel projection runs as the fused kernel (bf16 weights)
        self._graphs: dict[tuple[int, int], _DecodeGraph] = {}
        self._scratch_block: int | None = None
        single = self.tp is None or self.tp.size == 1
        fused_everywhere = (not single and getattr(self.tp, "fused", None) is not None
                            and quantization in (None, "none", "bf16"))
        self.use_graphs = (self.device.type == "cuda" and self.dtype == torch.bfloat16
                           and (single or fused_everywhere)
                           and not any("moe" in w for w in self.weights)
                           and os.environ.get("AJB_DECODE_GRAPHS", "1") != "0")

    # ------------------------------------------------------------------ graph-replayed decoding
    def _decode_static(self, g: _DecodeGraph) -> torch.Tensor:
        """One decoding step over the static buffers of ``g`` (every sequence: ``q_len`` new tokens, the rest cached)."""
        from ajllm_b200.ops import serving
        model, cache = self.model, self.cache
        n = g.bucket * g.q_len
        plan = object.__new__(serving.PagedPlan)
        plan.total_rows = n
        plan.launches = [(g.q_len, g.bucket, g.tables, g.starts, g.ctx)]
        g.pos32.copy_(g.pos)
        stream = model.token_embeddings(g.ids)
        if model.position_embeddings is not None:
            stream = stream + model.position_embeddings(g.pos)
        pending = None
        for index, (layer, w) in enumerate(zip(model.layers, self.weights)):
            attn = layer.attention
            stream, normed = layer.norm1.add_and_norm(stream, pending)
            qkv = _matmul(normed, w["qkv"])
            if attn.use_rope:
                serving.rope_packed_(qkv, attn.rope_cos, attn.rope_sin, g.pos32, attn.num_heads, attn.num_kv_heads, attn.head_dim)
            qkv = self._padded_heads(qkv, attn)
            q, k, v = ops.split_packed_qkv(qkv, attn.num_heads, attn.num_kv_heads, self.kernel_head_dim)
            cache.write(index, g.slots, k, v)
            attended = serving.paged_attention_planned(q.contiguous(), cache.keys[index], cache.values[index], plan,
                                                       self.softmax_scale)
            attended = self._row_parallel(self._true_heads(attended.reshape(n, -1), attn), w["out"])
            stream, normed = layer.norm2.add_and_norm(stream, attended)
            if "w13" in w:
                pending = self._row_parallel(ops.swiglu_interleaved(_matmul(normed, w["w13"])), w["w2"])
            else:
                pending = self._row_parallel(ops.silu(_matmul(normed, w["w1"])), w["w2"])
        hidden = model.final_norm.add_and_norm(stream, pending)[1]
        return ops.linear(hidden, model.head_weight).float()

    def capture_decode_graphs(self, max_seqs: int, q_lens: tuple[int, ...] = (1,)) -> int:
        """Captures the decoding graph of every batch-size bucket up to ``max_seqs`` for each number of new tokens per
        sequence in ``q_lens`` (a start-up cost instead of a stall in the first step that meets a new bucket). Every
        rank of a tensor-parallel group must call it with the same arguments. Returns the number of graphs held."""
        if not self.use_graphs:
            return 0
        attn0 = self.model.layers[0].attention
        group = attn0.num_heads // attn0.num_kv_heads
        top = next((b for b in self.GRAPH_BUCKETS if b >= max_seqs), self.GRAPH_BUCKETS[-1])
        for q_len in q_lens:
            if q_len < 1 or q_len > self.cache.block_size or group * q_len > 64:
                continue
            for bucket in self.GRAPH_BUCKETS:
                if bucket <= top:
                    self._graph_for(bucket, q_len)
        return len(self._graphs)

    def _graph_for(self, bucket: int, q_len: int) -> _DecodeGraph:
        g = self._graphs.get((bucket, q_len))
        if g is not None:
            return g
        cache = self.cache
        if self._scratch_block is None:
            self._scratch_block = cache.allocator.allocate()       # padding rows read and write this block only
        max_blocks = (self.model.context_length + cache.block_size - 1) // cache.block_size
        g = _DecodeGraph(bucket, q_len, max_blocks, self.device, self._scratch_block, cache.block_size)
        g.staging.fill([], cache)            # every row is a padding row: the capture reads and writes the scratch block only
        g.upload()
        # one eager run on a side stream first (lazy kernel attributes, allocator warm-up), then the capture
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            self._decode_static(g)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize(self.device)
        g.graph = torch.cuda.CUDAGraph()
        # thread-local error mode: with a process group alive, its watchdog thread polls CUDA events while this thread
        # captures, which the default (global) mode treats as a capture violation
        with torch.cuda.graph(g.graph, capture_error_mode="thread_local"):
            g.logits = self._decode_static(g)
        self._graphs[(bucket, q_len)] = g
        return g

    def _forward_decode_graph(self, items: list[RunItem]) -> torch.Tensor | None:
        """Replay path for a step in which every sequence feeds the same number of new tokens on top of a non-empty
        cache and wants logits for all of them (plain decoding: one; speculative verification: ``k + 1``); ``None``
        when the step does not qualify."""
        n = len(items)
        if n == 0 or n > self.GRAPH_BUCKETS[-1]:
            return None
        cache, model = self.cache, self.model
        q_len = len(items[0].token_ids)
        attn0 = model.layers[0].attention
        # a sequence's rows share one attention CTA (64 rows at most) and padding rows live in one scratch block
        if q_len < 1 or q_len > cache.block_size or (attn0.num_heads // attn0.num_kv_heads) * q_len > 64:
            return None
        for item in items:
            if len(item.token_ids) != q_len or item.num_logits != q_len or cache.length(item.seq_id) == 0:
                return None
            if cache.length(item.seq_id) + q_len > model.context_length:
                raise ValueError(f"sequence {item.seq_id} would exceed the context length {model.context_length}")
        bucket = next(b for b in self.GRAPH_BUCKETS if b >= n)
        g = self._graph_for(bucket, q_len)
        g.staging.fill(items, cache)
        g.upload()
        g.graph.replay()
        return g.logits[:n * q_len]

    def _padded_heads(self, qkv: torch.Tensor, attn) -> torch.Tensor:
        if self.kernel_head_dim == self.head_dim:
            return qkv
        from ajllm_b200.ops.functional import repack_heads
        return repack_heads(qkv, attn.num_heads + 2 * attn.num_kv_heads, self.head_dim, self.kernel_head_dim)

    def _true_heads(self, attended: torch.Tensor, attn) -> torch.Tensor:
        if self.kernel_head_dim == self.head_dim:
            return attended
        from ajllm_b200.ops.functional import repack_heads
        return repack_heads(attended, attn.num_heads, self.kernel_head_dim, self.head_dim)

    def _reduce(self, x: torch.Tensor) -> torch.Tensor:
        if self.tp is not None and self.tp.size > 1:
            self.tp.all_reduce_sum_(x)
        return x

    def _row_parallel(self, x: torch.Tensor, weight) -> torch.Tensor:
        """Row-parallel projection summed over the tensor-parallel ranks.

        With a fused tensor-parallel context and a bf16 weight the partial products are exchanged by the
        GEMM kernel itself (GEMM -> all-reduce over peer memory); otherwise GEMM, then a NCCL all-reduce."""
        fused = getattr(self.tp, "fused", None) if self.tp is not None else None
        if (fused is not None and x.is_cuda and x.dtype == torch.bfloat16 and not isinstance(weight, Fp8Weight)
                and x.shape[0] <= self.FUSED_ALL_REDUCE_MAX_ROWS):
            return fused.gemm_all_reduce(x, weight)
        return self._reduce(_matmul(x, weight))

    @torch.no_grad()
    def forward(self, items: list[RunItem]) -> torch.Tensor:
        """Returns logits ``[sum_i num_logits_i, vocab]`` in item order."""
        if self.use_graphs:
            logits = self._forward_decode_graph(items)
            if logits is not None:
                return logits
        model, cache = self.model, self.cache
        tokens, positions, slots, q_lens, ctx_lens, seq_ids, logit_rows = [], [], [], [], [], [], []
        cursor = 0
        for item in items:
            start = cache.length(item.seq_id)
            n = len(item.token_ids)
            if start + n > model.context_length:
                raise ValueError(f"sequence {item.seq_id} would exceed the context length {model.context_length}")
            slots.extend(cache.append_slots(item.seq_id, n))
            tokens.extend(item.token_ids)
            positions.extend(range(start, start + n))
            q_lens.append(n)
            ctx_lens.append(start + n)
            seq_ids.append(item.seq_id)
            logit_rows.extend(range(cursor + n - item.num_logits, cursor + n))
            cursor += n
        dev = self.device
        ids = torch.tensor(tokens, dtype=torch.long, device=dev)
        pos = torch.tensor(positions, dtype=torch.long, device=dev)
        slot_t = torch.tensor(slots, dtype=torch.long, device=dev)
        tables = cache.block_table_tensor(seq_ids, dev)
        ctx_t = torch.tensor(ctx_lens, dtype=torch.int32, device=dev)
        qlen_t = torch.tensor(q_lens, dtype=torch.int32, device=dev)

        on_gpu = dev.type == "cuda" and self.dtype == torch.bfloat16
        if on_gpu:
            from ajllm_b200.ops import serving
            pos32 = pos.to(torch.int32)
            # split the batch: long prompts with nothing cached use the training flash kernel, the rest is paged
            fresh, cached_idx, cached_qlens, cached_ctx, cached_items = [], [], [], [], []
            cursor = 0
            for i, (n, ctx) in enumerate(zip(q_lens, ctx_lens)):
                if n == ctx and n > 16:
                    fresh.append((cursor, cursor + n))
                else:
                    cached_idx.extend(range(cursor, cursor + n))
                    cached_qlens.append(n)
                    cached_ctx.append(ctx)
                    cached_items.append(i)
                cursor += n
            cached_rows = cached_tables = None
            if cached_idx:
                cached_rows = torch.tensor(cached_idx, dtype=torch.long, device=dev)
                cached_tables = tables if len(cached_items) == len(q_lens) else \
                    tables.index_select(0, torch.tensor(cached_items, dtype=torch.long, device=dev)).contiguous()
                attn0 = model.layers[0].attention
                paged_plan = serving.PagedPlan(cached_tables, cached_qlens, cached_ctx, attn0.num_heads, attn0.num_kv_heads)
                all_cached = len(cached_idx) == len(tokens)
        stream = model.token_embeddings(ids)
        if model.position_embeddings is not None:
            stream = stream + model.position_embeddings(pos)
        pending = None
        for index, (layer, w) in enumerate(zip(model.layers, self.weights)):
            attn = layer.attention
            stream, normed = layer.norm1.add_and_norm(stream, pending)
            qkv = _matmul(normed, w["qkv"])
            if on_gpu:
                if attn.use_rope:
                    serving.rope_packed_(qkv, attn.rope_cos, attn.rope_sin, pos32, attn.num_heads, attn.num_kv_heads,
                                         attn.head_dim)
                khd = self.kernel_head_dim
                qkv = self._padded_heads(qkv, attn)
                q, k, v = ops.split_packed_qkv(qkv, attn.num_heads, attn.num_kv_heads, khd)
                cache.write(index, slot_t, k, v)
                attended = torch.empty(ids.shape[0], attn.num_heads * khd, dtype=qkv.dtype, device=dev)
                for lo, hi in fresh:          # prompts starting from an empty cache: tiled kernel on the packed rows
                    attended[lo:hi] = serving.prompt_attention(qkv[lo:hi], attn.num_heads, attn.num_kv_heads, khd,
                                                               self.softmax_scale)
                if cached_rows is not None:
                    if all_cached:          # pure decode / verify step: no gather, no scatter
                        attended = serving.paged_attention_planned(q.contiguous(), cache.keys[index], cache.values[index],
                                                                   paged_plan, self.softmax_scale).reshape(ids.shape[0], -1)
                    else:
                        part = serving.paged_attention_planned(q.index_select(0, cached_rows).contiguous(), cache.keys[index],
                                                               cache.values[index], paged_plan, self.softmax_scale)
                        attended.index_copy_(0, cached_rows, part.reshape(part.shape[0], -1))
                attended = self._true_heads(attended, attn)
            else:
                q, k, v = ops.split_packed_qkv(qkv, attn.num_heads, attn.num_kv_heads, attn.head_dim)
                if attn.use_rope:
                    q = reference.rope_interleaved(q, attn.rope_cos, attn.rope_sin, pos)
                    k = reference.rope_interleaved(k, attn.rope_cos, attn.rope_sin, pos)
                cache.write(index, slot_t, k, v)
                attended = ops.paged_attention_ragged(q, cache.keys[index], cache.values[index], tables, ctx_t, qlen_t,
                                                      q_lens, ctx_lens)
            attended = self._row_parallel(attended.reshape(ids.shape[0], -1), w["out"])
            stream, normed = layer.norm2.add_and_norm(stream, attended)
            if "moe" in w:
                pending = w["moe"](normed)
            elif "w13" in w:
                hidden_ff = (ops.swiglu_interleaved(_matmul(normed, w["w13"])) if isinstance(w["w13"], Fp8Weight)
                             else ops.linear_swiglu(normed, w["w13"]))
                pending = self._row_parallel(hidden_ff, w["w2"])
            else:
                pending = self._row_parallel(ops.silu(_matmul(normed, w["w1"])), w["w2"])
        hidden = model.final_norm.add_and_norm(stream, pending)[1]
        if not logit_rows:
            return hidden.new_zeros(0, model.vocab_size)
        rows = hidden[torch.tensor(logit_rows, dtype=torch.long, device=dev)]
        return ops.linear(rows, model.head_weight).float()
