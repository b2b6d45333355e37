"""Host-side bookkeeping of the paged bf16 KV cache: which pages each sequence owns.

The counterpart of the reference's session state (`GpuSession`: `len`, `truncate`, `reset`,
gpt-oss/src/gpu.rs:365-413; `Session::truncate`, gpt-oss/src/model.rs:204-213) for a cache
made of 16-token pages instead of one ring of rows per layer.  Pure integer bookkeeping; the
page contents live in a device buffer and are only ever touched by the kernels.
"""
from __future__ import annotations

import numpy as np

from . import compute

PAGE = 16
HEAD_DIM = 64
GROUP = 8


def tile_bytes(kv_heads: int) -> int:
    """Bytes of one page across `kv_heads` heads: K rows then V rows, 4 KiB per head."""
    return kv_heads * 2 * PAGE * HEAD_DIM * 2


class PagedKvCache:
    """One layer's pages for `seqs` sequences on one GPU.

    `block_table[s][i]` is the pool page holding positions `16 i .. 16 i + 15` of sequence `s`
    (or, with `ring_pages`, of positions whose page index is `i` modulo `ring_pages`: the paged
    form of the reference's sliding ring, gpt-oss/src/gpu.rs:567-574).
    """

    def __init__(self, gpu: compute.Gpu, seqs: int, max_pages: int, pool_pages: int, kv_heads: int,
                 *, ring_pages: int = 0, mirrored_pool: bool = False, rng: np.random.Generator | None = None):
        self.gpu, self.seqs, self.max_pages, self.pool_pages = gpu, seqs, max_pages, pool_pages
        self.kv_heads, self.ring_pages = kv_heads, ring_pages
        nbytes = pool_pages * tile_bytes(kv_heads)
        self.pool = gpu.buffer(nbytes) if mirrored_pool else gpu.device_buffer(nbytes)
        self.pool.zero()
        self.table = gpu.buffer(seqs * max_pages * 4)
        self.table_host = np.full((seqs, max_pages), -1, np.int32)
        self.lens = np.zeros(seqs, np.int64)
        order = np.arange(pool_pages)
        if rng is not None:  # hand pages out in a scattered order, as a long-running server would
            order = rng.permutation(pool_pages)
        self.free = list(order[::-1].astype(int))
        self._dirty = True

    # -- allocation --------------------------------------------------------------------------
    def pages_needed(self, length: int) -> int:
        n = -(-length // PAGE)
        return min(n, self.ring_pages) if self.ring_pages else n

    def reserve(self, seq: int, new_len: int) -> None:
        """Makes sure sequence `seq` owns the pages positions `< new_len` live in."""
        need = self.pages_needed(new_len)
        if need > self.max_pages:
            raise ValueError(f"sequence {seq}: {new_len} positions need more than {self.max_pages} pages")
        row = self.table_host[seq]
        for i in range(need):
            if row[i] < 0:
                if not self.free:
                    raise MemoryError("page pool exhausted")
                row[i] = self.free.pop()
                self._dirty = True
        self.lens[seq] = max(self.lens[seq], new_len)

    def truncate(self, seq: int, length: int) -> None:
        """Goes back to `length` positions and gives the pages past it back to the pool."""
        if length >= self.lens[seq]:
            return
        if self.ring_pages:
            # a ring has already overwritten what lay more than ring_pages back
            if self.lens[seq] - length > self.ring_pages * PAGE:
                raise ValueError("cannot rewind a ring past what it still holds")
        else:
            keep = -(-length // PAGE)
            row = self.table_host[seq]
            for i in range(keep, self.max_pages):
                if row[i] >= 0:
                    self.free.append(int(row[i]))
                    row[i] = -1
                    self._dirty = True
        self.lens[seq] = length

    def reset(self) -> None:
        for s in range(self.seqs):
            self.lens[s] = 0
            row = self.table_host[s]
            for i in range(self.max_pages):
                if row[i] >= 0:
                    self.free.append(int(row[i]))
                    row[i] = -1
        self._dirty = True

    # -- device view -------------------------------------------------------------------------
    def flush_table(self) -> None:
        """Writes the block table into its buffer if it changed (uploaded by the next batch)."""
        if self._dirty:
            self.table.write(self.table_host)
            self._dirty = False

    def descriptor(self, pool_index: int, table_index: int) -> compute.PagedCache:
        """The `cc_paged_cache` naming this cache's buffers by their position in a batch."""
        return compute.PagedCache(compute.Slice(pool_index, 0, len(self.pool)),
                                  compute.Slice(table_index, 0, len(self.table)),
                                  self.max_pages, self.ring_pages, self.kv_heads)


def shard_kv_heads(kv_heads: int, world: int, rank: int) -> range:
    """KV heads rank `rank` of `world` owns: contiguous, 8/N each for N in 1, 2, 4, 8.  The
    query heads of a KV head g are 8g .. 8g+7, so heads shard with it and attention needs no
    exchange between ranks."""
    if world <= 0 or kv_heads % world != 0:
        raise ValueError(f"{kv_heads} KV heads do not split over {world} ranks")
    per = kv_heads // world
    return range(rank * per, (rank + 1) * per)
