"""Paged KV cache: fixed-size token blocks handed out by a free-list allocator.

The reference has no KV cache (``ajllm/generation/generator.py:21-25`` re-runs the model on the whole
context for every new token). Here each layer owns ``[num_blocks, block_size, kv_heads, head_dim]``
key and value pools; a sequence owns a list of block ids (its block table) and token ``t`` of the
sequence lives in block ``table[t // block_size]`` at offset ``t % block_size``. Blocks are
reference-counted so a prefix can be shared by forked sequences. Rolling a sequence back (speculative
tokens that were rejected) only shortens its length and returns blocks that became empty.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch


class OutOfBlocks(RuntimeError):
    """The pool cannot satisfy an allocation; the scheduler reacts by preempting a sequence."""


class BlockAllocator:
    def __init__(self, num_blocks: int) -> None:
        self.num_blocks = num_blocks
        self._free = list(range(num_blocks - 1, -1, -1))
        self._refs = [0] * num_blocks

    @property
    def free_blocks(self) -> int:
        return len(self._free)

    def allocate(self) -> int:
        if not self._free:
            raise OutOfBlocks("KV cache pool is exhausted")
        block = self._free.pop()
        self._refs[block] = 1
        return block

    def share(self, block: int) -> None:
        assert self._refs[block] > 0
        self._refs[block] += 1

    def release(self, block: int) -> None:
        assert self._refs[block] > 0, f"double free of block {block}"
        self._refs[block] -= 1
        if self._refs[block] == 0:
            self._free.append(block)

    def ref_count(self, block: int) -> int:
        return self._refs[block]


@dataclass
class BlockTable:
    """Blocks of one sequence, in order, plus the number of tokens stored."""

    blocks: list[int] = field(default_factory=list)
    length: int = 0
    shrinks: int = 0          # how often blocks were given back (a mirror of `blocks` elsewhere must then be rebuilt)


class PagedKVCache:
    def __init__(self, num_layers: int, num_blocks: int, block_size: int, kv_heads: int, head_dim: int,
                 dtype: torch.dtype, device: torch.device) -> None:
        self.block_size = block_size
        self.num_layers, self.kv_heads, self.head_dim = num_layers, kv_heads, head_dim
        self.allocator = BlockAllocator(num_blocks)
        shape = (num_layers, num_blocks, block_size, kv_heads, head_dim)
        self.keys = torch.zeros(shape, dtype=dtype, device=device)
        self.values = torch.zeros(shape, dtype=dtype, device=device)
        self.tables: dict[int, BlockTable] = {}

    # ---------------------------------------------------------------- bookkeeping
    def blocks_needed(self, seq_id: int, new_tokens: int) -> int:
        table = self.tables.get(seq_id)
        have = len(table.blocks) if table else 0
        length = table.length if table else 0
        want = (length + new_tokens + self.block_size - 1) // self.block_size
        return max(0, want - have)

    def can_append(self, seq_id: int, new_tokens: int) -> bool:
        return self.blocks_needed(seq_id, new_tokens) <= self.allocator.free_blocks

    def append_slots(self, seq_id: int, new_tokens: int) -> list[int]:
        """Reserve room for ``new_tokens`` more tokens and return their flat slot ids
        (``block * block_size + offset``)."""
        table = self.tables.setdefault(seq_id, BlockTable())
        need = self.blocks_needed(seq_id, new_tokens)
        if need > self.allocator.free_blocks:
            raise OutOfBlocks(f"sequence {seq_id} needs {need} blocks, {self.allocator.free_blocks} free")
        for _ in range(need):
            table.blocks.append(self.allocator.allocate())
        slots = []
        for t in range(table.length, table.length + new_tokens):
            slots.append(table.blocks[t // self.block_size] * self.block_size + t % self.block_size)
        table.length += new_tokens
        return slots

    def truncate(self, seq_id: int, new_length: int) -> None:
        """Forget the tokens past ``new_length`` (speculative rollback)."""
        table = self.tables[seq_id]
        assert 0 <= new_length <= table.length
        table.length = new_length
        keep = (new_length + self.block_size - 1) // self.block_size
        while len(table.blocks) > keep:
            self.allocator.release(table.blocks.pop())
            table.shrinks += 1

    def fork(self, parent_id: int, child_id: int) -> None:
        """``child`` shares every block of ``parent`` (copy-on-write is the caller's duty: a shared last
        block must be copied before either sequence appends to it)."""
        parent = self.tables[parent_id]
        for block in parent.blocks:
            self.allocator.share(block)
        self.tables[child_id] = BlockTable(list(parent.blocks), parent.length)

    def free(self, seq_id: int) -> None:
        table = self.tables.pop(seq_id, None)
        if table is None:
            return
        for block in table.blocks:
            self.allocator.release(block)

    def length(self, seq_id: int) -> int:
        table = self.tables.get(seq_id)
        return table.length if table else 0

    # ---------------------------------------------------------------- device views
    def block_table_tensor(self, seq_ids: list[int], device: torch.device) -> torch.Tensor:
        import numpy as np
        width = max((len(self.tables[s].blocks) for s in seq_ids), default=1) or 1
        out = np.zeros((len(seq_ids), width), dtype=np.int32)
        for row, s in enumerate(seq_ids):
            blocks = self.tables[s].blocks
            out[row, :len(blocks)] = blocks
        return torch.from_numpy(out).to(device)

    def write(self, layer: int, slots: torch.Tensor, keys: torch.Tensor, values: torch.Tensor) -> None:
        """``keys`` / ``values`` are ``[tokens, kv_heads, head_dim]``; ``slots`` the flat slot of each token."""
        flat_k = self.keys[layer].view(-1, self.kv_heads, self.head_dim)
        flat_v = self.values[layer].view(-1, self.kv_heads, self.head_dim)
        flat_k.index_copy_(0, slots, keys.to(flat_k.dtype))
        flat_v.index_copy_(0, slots, values.to(flat_v.dtype))
