"""Physical KV storage.

``KvBuffer`` is one tensor ``[layers, pages, 2, page_size, kv_heads, head_dim]``
(K at index 0, V at index 1 of the third axis).  A page of one layer is contiguous
(``2 * page_size * kv_heads * head_dim`` elements), so attention kernels fetch a
page's K or V with one tiled copy, and the host tier moves one logical block as
``layers`` strided chunks.  ``LatentKvBuffer`` is the MLA variant: one row of
``kv_lora_rank + rope_dim`` per token, ``[layers, pages, page_size, width]``.

``PagePool``/``KvPool`` are the simple non-prefix page allocators used by model
lines that keep per-request recurrent state next to paged attention KV.

Reference parity: pegainfer-kv-cache/src/buffer.rs:22-71, src/layout.rs:5-33
(page-first fused buffer); pegainfer-core/src/page_pool.rs:7-130,
pegainfer-core/src/kv_pool.rs:17-449.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass
class KvLayout:
    num_layers: int
    num_pages: int
    page_size: int
    kv_heads: int
    head_dim: int
    dtype: torch.dtype = torch.bfloat16

    @property
    def page_elems(self) -> int:
        return 2 * self.page_size * self.kv_heads * self.head_dim

    @property
    def bytes_per_block(self) -> int:
        """Bytes one logical block occupies across all layers."""
        return self.num_layers * self.page_elems * torch.empty((), dtype=self.dtype).element_size()

    @staticmethod
    def pages_for_budget(budget_bytes: int, num_layers: int, page_size: int, kv_heads: int, head_dim: int, elem=2) -> int:
        per = num_layers * 2 * page_size * kv_heads * head_dim * elem
        return max(0, budget_bytes // per)


class KvBuffer:
    def __init__(self, layout: KvLayout, device="cpu"):
        self.layout = layout
        l = layout
        self.data = torch.zeros(
            (l.num_layers, l.num_pages, 2, l.page_size, l.kv_heads, l.head_dim), dtype=l.dtype, device=device
        )

    def layer(self, i: int) -> torch.Tensor:
        return self.data[i]

    def block_view(self, bid: int) -> torch.Tensor:
        """``[layers, 2, page_size, kv_heads, head_dim]`` strided view of one block."""
        return self.data[:, bid]


class LatentKvBuffer:
    def __init__(self, num_layers, num_pages, page_size, width, dtype=torch.bfloat16, device="cpu"):
        self.page_size = page_size
        self.width = width
        self.data = torch.zeros((num_layers, num_pages, page_size, width), dtype=dtype, device=device)

    def layer(self, i: int) -> torch.Tensor:
        return self.data[i]

    def block_view(self, bid: int) -> torch.Tensor:
        return self.data[:, bid]


class PagePool:
    """LIFO free list of page ids; page 0 reserved for padding rows."""

    def __init__(self, num_pages: int):
        self.num_pages = num_pages
        self._free = list(range(num_pages - 1, 0, -1))

    def available(self) -> int:
        return len(self._free)

    def alloc(self, n: int) -> list:
        if n > len(self._free):
            raise RuntimeError(f"page pool exhausted: need {n}, have {len(self._free)}")
        out = [self._free.pop() for _ in range(n)]
        return out

    def free(self, pages) -> None:
        self._free.extend(reversed(list(pages)))


class KvState:
    """Pages + length of one sequence in a :class:`KvPool`."""

    def __init__(self, pool: "KvPool"):
        self.pool = pool
        self.pages: list = []
        self.seq_len = 0

    def ensure(self, new_len: int) -> None:
        need = (new_len + self.pool.page_size - 1) // self.pool.page_size - len(self.pages)
        if need > 0:
            self.pages.extend(self.pool.pages.alloc(need))

    def advance(self, n: int) -> None:
        self.seq_len += n

    def release(self) -> None:
        self.pool.pages.free(self.pages)
        self.pages = []
        self.seq_len = 0


class KvPool:
    def __init__(self, num_pages: int, page_size: int):
        self.page_size = page_size
        self.pages = PagePool(num_pages)

    def new_state(self) -> KvState:
        return KvState(self)
