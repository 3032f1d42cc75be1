"""Paged KV cache: a pool of 64-token pages per layer, a free list, and per-sequence block tables
(layout of the reference's block attention: key_cache ``[max_block_num, num_head, block_size, head_size]``,
``block_tables [batch, max_blocks_per_seq]``, python/paddle/incubate/nn/functional/block_multihead_attention.py:33)."""
from __future__ import annotations

import torch

PAGE = 64


class PagedKVCache:
    def __init__(self, num_layers, num_kv_heads, num_blocks, max_batch, max_seq_len, head_dim=128,
                 dtype=torch.bfloat16, device="cuda"):
        assert head_dim == 128, "the decode kernels are specialised for head_dim 128"
        self.num_layers, self.num_kv_heads, self.num_blocks = num_layers, num_kv_heads, num_blocks
        self.max_blocks_per_seq = (max_seq_len + PAGE - 1) // PAGE
        shape = (num_blocks, num_kv_heads, PAGE, head_dim)
        self.k = [torch.zeros(shape, dtype=dtype, device=device) for _ in range(num_layers)]
        self.v = [torch.zeros(shape, dtype=dtype, device=device) for _ in range(num_layers)]
        self.free = list(range(num_blocks - 1, -1, -1))
        self._table_host = torch.zeros((max_batch, self.max_blocks_per_seq), dtype=torch.int32)
        self.block_table = torch.zeros((max_batch, self.max_blocks_per_seq), dtype=torch.int32, device=device)
        self.seq_lens = torch.zeros(max_batch, dtype=torch.int32, device=device)
        self._owned = [[] for _ in range(max_batch)]

    @staticmethod
    def blocks_needed(batch, seq_len):
        return batch * ((seq_len + PAGE - 1) // PAGE)

    def reserve(self, seq_idx, total_len):
        """Make sure sequence ``seq_idx`` owns pages for ``total_len`` tokens; returns False when the pool is empty."""
        need = (total_len + PAGE - 1) // PAGE
        own = self._owned[seq_idx]
        if need > self.max_blocks_per_seq or need - len(own) > len(self.free):
            return False
        changed = False
        while len(own) < need:
            blk = self.free.pop()
            self._table_host[seq_idx, len(own)] = blk
            own.append(blk)
            changed = True
        if changed:
            self.block_table[seq_idx].copy_(self._table_host[seq_idx], non_blocking=True)
        return True

    def release(self, seq_idx):
        self.free.extend(reversed(self._owned[seq_idx]))
        self._owned[seq_idx] = []
        self.seq_lens[seq_idx] = 0

    def reset(self):
        for i in range(len(self._owned)):
            if self._owned[i]:
                self.release(i)
        self.seq_lens.zero_()
