"""Token pool of a latent-attention model: ONE row [c | kr] per token and layer, shared by all heads
(c: the normed KV latent, kr: the rotated shared key part).  Same indexing as MHATokenToKVPool — slot
ids from the token allocator, slot 0..page_size-1 is the dummy page — so ReqToTokenPool and the
paged allocator are used unchanged.  Layers that read another layer's latent own no buffer: they
alias their source's."""
from __future__ import annotations

from typing import Dict, Optional

import torch


class LatentTokenToKVPool:
    def __init__(self, size: int, page_size: int, dtype: torch.dtype, row_dims: Dict[int, int],
                 source_of: Dict[int, int], device: str, block_summaries: Optional[Dict[int, int]] = None):
        """row_dims: {layer that owns a buffer: row width}; source_of: {layer: owning layer};
        block_summaries: {layer: tokens per block} for layers that also keep one fp32 row (the mean of
        the block's token rows) per block of consecutive positions."""
        self.size, self.page_size, self.dtype, self.device = size, page_size, dtype, device
        self.source_of = dict(source_of)
        self.kv_buffer = {l: torch.zeros((size + page_size, d), dtype=dtype, device=device)
                          for l, d in row_dims.items()}
        for l, src in self.source_of.items():
            if src not in self.kv_buffer:
                raise ValueError(f"layer {l} reads the latent of layer {src}, which owns none")

        # A block's summary lives at the slot of the block's LAST token: slot // block when blocks
        # cannot straddle pages (the block size divides the page size: rows = slots / block), else at the
        # slot itself (one row per slot).  Pages are handed out whole, so the rows are as paged as the
        # tokens and need no allocator of their own; nothing is cleared on reuse, a row is rewritten when
        # its block completes and read only for blocks that have.
        self.block_summary, self.block_div = {}, {}
        for l, block in (block_summaries or {}).items():
            if l not in self.kv_buffer:
                raise ValueError(f"layer {l} summarises blocks of rows it does not own")
            div = block if page_size % block == 0 else 1
            self.block_div[l] = div
            self.block_summary[l] = torch.zeros(((size + page_size) // div + 1, row_dims[l]),
                                                dtype=torch.float32, device=device)

    def get_block_summary(self, layer_id: int):
        """-> (fp32 buffer [rows, row width], divisor from token slot to row)."""
        return self.block_summary[layer_id], self.block_div[layer_id]

    def get_kv_buffer(self, layer_id: int) -> torch.Tensor:
        return self.kv_buffer[self.source_of.get(layer_id, layer_id)]

    def owns(self, layer_id: int) -> bool:
        return layer_id in self.kv_buffer

    def get_kv_size_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in list(self.kv_buffer.values()) +
                   list(self.block_summary.values()))


class SeqStatePool:
    """Per-sequence carry of layers whose output at a token depends on the token before it (token
    shift, and any other fixed-size recurrent state): state[layer] is [slots, width] fp32, the slot is
    the sequence's row in ReqToTokenPool, so it is taken and given back with it.  Nothing is
    cleared on reuse: a kernel that reads the state of a token at position 0 substitutes zeros."""

    def __init__(self, slots: int, widths: Dict[int, int], device: str):
        self.slots = slots
        self.state = {l: torch.zeros((slots, w), dtype=torch.float32, device=device)
                      for l, w in widths.items()}

    def get(self, layer_id: int) -> Optional[torch.Tensor]:
        return self.state.get(layer_id)

    def size_bytes(self) -> int:
        return sum(t.numel() * 4 for t in self.state.values())
