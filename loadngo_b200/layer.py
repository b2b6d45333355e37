"""The attention hot path of one gpt-oss layer on one GPU, as a caller drives it.

This is the paged counterpart of `GpuModel::encode_attention`'s middle section
(gpt-oss/src/gpu.rs:741-806): rotate Q and K, append K and V to the cache, attend.  It only
sequences calls on a `compute.Batch`; all arithmetic happens in libcuda_compute.so.
"""
from __future__ import annotations

import numpy as np

from . import compute
from .compute import Slice
from .paged import GROUP, HEAD_DIM, PAGE, PagedKvCache

BF16 = 2


class PagedAttentionLayer:
    """Buffers and call sequence for `seqs` sequences, `kv_heads` local KV heads.

    window: keys a query sees, itself included; 0 = all (a full-causal layer).
    Inputs and outputs are host arrays of bfloat16 bit patterns (uint16): q [n][heads][64],
    k and v [n][kv_heads][64], out [n][heads][64].
    """

    # positions of the layer's buffers inside every batch it records
    Q, K, V, QROT, OUT, POS, SEQ, LENS, TABLE, SINKS, POOL, BT, QOFF, STARTS = range(14)

    def __init__(self, gpu: compute.Gpu, *, seqs: int, max_context: int, max_new: int, kv_heads: int = 8,
                 window: int = 0, sinks: np.ndarray | None = None, pool_pages: int | None = None,
                 ring_pages: int = 0, rope: dict | None = None, rng: np.random.Generator | None = None,
                 mirrored_pool: bool = False):
        self.gpu, self.seqs, self.kv_heads, self.window = gpu, seqs, kv_heads, window
        self.heads = kv_heads * GROUP
        self.max_context, self.max_new = max_context, max_new
        self.scale = 1.0 / float(np.sqrt(np.float32(HEAD_DIM)))
        max_pages = ring_pages if ring_pages else -(-max_context // PAGE)
        if pool_pages is None:
            pool_pages = seqs * max_pages
        self.cache = PagedKvCache(gpu, seqs, max_pages, pool_pages, kv_heads, ring_pages=ring_pages, rng=rng,
                                  mirrored_pool=mirrored_pool)
        n = max_new
        self.q = gpu.buffer(n * self.heads * HEAD_DIM * BF16)
        self.k = gpu.buffer(n * kv_heads * HEAD_DIM * BF16)
        self.v = gpu.buffer(n * kv_heads * HEAD_DIM * BF16)
        self.q_rot = gpu.buffer(2 * n * self.heads * HEAD_DIM * BF16)
        self.out = gpu.buffer(n * self.heads * HEAD_DIM * BF16)
        self.positions = gpu.buffer(n * 4)
        self.seq_ids = gpu.buffer(n * 4)
        self.seq_lens = gpu.buffer(seqs * 4)
        self.q_offsets = gpu.buffer((seqs + 1) * 4)
        self.starts = gpu.buffer(seqs * 4)
        self.rope = dict(head_dim=HEAD_DIM, theta=150000.0, factor=32.0, original_context=4096.0,
                         beta_fast=32.0, beta_slow=1.0)
        if rope:
            self.rope.update(rope)
        # One table for every position the layer can hold, computed once in f64 on the host
        # (what GpuModel::prepare does per pass, gpt-oss/src/gpu.rs:689-697).
        self.table = gpu.upload(compute.rope_table(0, max_context, **self.rope))
        sink_values = np.zeros(self.heads, np.float32) if sinks is None else np.asarray(sinks, np.float32)
        self.has_sinks = sinks is not None
        self.sinks = gpu.upload(sink_values)

    def buffers(self) -> list:
        return [self.q, self.k, self.v, self.q_rot, self.out, self.positions, self.seq_ids, self.seq_lens,
                self.table, self.sinks, self.cache.pool, self.cache.table, self.q_offsets, self.starts]

    def _s(self, index: int, nbytes: int, offset: int = 0) -> Slice:
        return Slice(index, offset, nbytes)

    # -- recording ------------------------------------------------------------------------------
    def record_append(self, batch: compute.Batch, n: int, in_f32: bool = False) -> None:
        h, g = self.heads, self.kv_heads
        esz = 4 if in_f32 else BF16
        batch.rope_append_paged(
            (self._s(self.Q, n * h * HEAD_DIM * esz), self._s(self.K, n * g * HEAD_DIM * esz),
             self._s(self.V, n * g * HEAD_DIM * esz)),
            in_f32, self._s(self.QROT, 2 * n * h * HEAD_DIM * BF16), self._s(self.TABLE, len(self.table)), 0,
            self._s(self.POS, n * 4), self._s(self.SEQ, n * 4), self.cache.descriptor(self.POOL, self.BT), n)

    def record_decode(self, batch: compute.Batch, n: int, max_seq_len: int) -> None:
        h = self.heads
        batch.attention_decode_paged(
            self._s(self.QROT, 2 * n * h * HEAD_DIM * BF16), self.cache.descriptor(self.POOL, self.BT),
            self._s(self.LENS, n * 4), n, max_seq_len, self._s(self.SINKS, h * 4) if self.has_sinks else None,
            self.window, self.scale, self._s(self.OUT, n * h * HEAD_DIM * BF16))

    def record_decode_step(self, batch: compute.Batch, n: int, max_seq_len: int, in_f32: bool = False) -> None:
        """`record_append` + `record_decode` for one new token per sequence as one launch."""
        h, g = self.heads, self.kv_heads
        esz = 4 if in_f32 else BF16
        batch.attention_decode_step_paged(
            (self._s(self.Q, n * h * HEAD_DIM * esz), self._s(self.K, n * g * HEAD_DIM * esz),
             self._s(self.V, n * g * HEAD_DIM * esz)),
            in_f32, self._s(self.TABLE, len(self.table)), 0, self.cache.descriptor(self.POOL, self.BT),
            self._s(self.LENS, n * 4), n, max_seq_len, self._s(self.SINKS, h * 4) if self.has_sinks else None,
            self.window, self.scale, self._s(self.OUT, n * h * HEAD_DIM * BF16))

    def record_prefill(self, batch: compute.Batch, seqs: int, total: int, max_t: int) -> None:
        h = self.heads
        batch.attention_prefill_paged(
            self._s(self.QROT, 2 * total * h * HEAD_DIM * BF16), self.cache.descriptor(self.POOL, self.BT),
            self._s(self.QOFF, (seqs + 1) * 4), self._s(self.STARTS, seqs * 4), seqs, total, max_t,
            self._s(self.SINKS, h * 4) if self.has_sinks else None, self.window, self.scale,
            self._s(self.OUT, total * h * HEAD_DIM * BF16))

    # -- whole steps with host arrays --------------------------------------------------------------
    def _stage(self, q, k, v, positions, seq_ids) -> int:
        n = q.shape[0]
        assert n <= self.max_new
        self.q.write(q)
        self.k.write(k)
        self.v.write(v)
        self.positions.write(np.asarray(positions, np.int32))
        self.seq_ids.write(np.asarray(seq_ids, np.int32))
        return n

    def decode_step(self, q: np.ndarray, k: np.ndarray, v: np.ndarray, seq_ids=None, fused: bool = True) -> np.ndarray:
        """One new token for each of `n` sequences: append at each sequence's next position and
        attend.  Host arrays in, host array out (uploads and the read-back are part of it).
        `fused`: one launch for the step; else the append and the attention as two."""
        n = q.shape[0]
        seq_ids = np.arange(n) if seq_ids is None else np.asarray(seq_ids)
        positions = self.cache.lens[seq_ids].astype(np.int32)
        for s, p in zip(seq_ids, positions):
            self.cache.reserve(int(s), int(p) + 1)
        self.cache.flush_table()
        self._stage(q, k, v, positions, seq_ids)
        # the decode kernel reads block-table row i and seq_lens[i] for query i
        assert np.array_equal(seq_ids, np.arange(n)), "decode_step serves sequences 0..n-1 in order"
        self.seq_lens.write((positions + 1).astype(np.int32))
        batch = self.gpu.batch(self.buffers())
        if fused:
            self.record_decode_step(batch, n, int(positions.max()) + 1)
        else:
            self.record_append(batch, n)
            self.record_decode(batch, n, int(positions.max()) + 1)
        batch.read_back(self._s(self.OUT, n * self.heads * HEAD_DIM * BF16))
        done = batch.run()
        if isinstance(done.gpu_time, Exception):
            raise done.gpu_time
        return self.out.view(np.uint16)[: n * self.heads * HEAD_DIM].reshape(n, self.heads, HEAD_DIM).copy()

    def open_decode_loop(self, n: int, max_seq_len: int, fused: bool = True) -> None:
        """Records one decode step for sequences 0..n-1 (append, attend, read the output back)
        to be replayed once per token by `decode_step_replayed`; `max_seq_len` bounds the length
        any of the sequences reaches while the loop is open (it sizes the split of long caches)."""
        self._loop_n = n
        self._loop = self.gpu.batch(self.buffers())
        if fused:
            self.record_decode_step(self._loop, n, max_seq_len)
        else:
            self.record_append(self._loop, n)
            self.record_decode(self._loop, n, max_seq_len)
        self._loop.read_back(self._s(self.OUT, n * self.heads * HEAD_DIM * BF16))
        self._loop.end_recording()

    def decode_step_replayed(self, q: np.ndarray, k: np.ndarray, v: np.ndarray) -> np.ndarray:
        """`decode_step` without recording anything: stage this token's inputs and replay."""
        n = self._loop_n
        seq_ids = np.arange(n)
        positions = self.cache.lens[seq_ids].astype(np.int32)
        for s_, p_ in zip(seq_ids, positions):
            self.cache.reserve(int(s_), int(p_) + 1)
        self.cache.flush_table()
        self._stage(q, k, v, positions, seq_ids)
        self.seq_lens.write((positions + 1).astype(np.int32))
        done = self._loop.replay()
        if isinstance(done.gpu_time, Exception):
            raise done.gpu_time
        return self.out.view(np.uint16)[: n * self.heads * HEAD_DIM].reshape(n, self.heads, HEAD_DIM).copy()

    def close_decode_loop(self) -> None:
        self._loop.drop()
        self._loop = None

    def prefill(self, q: np.ndarray, k: np.ndarray, v: np.ndarray, counts) -> np.ndarray:
        """`counts[s]` new positions for sequence s (rows of q, k, v back to back), appended at
        each sequence's next position, then attended causally."""
        counts = np.asarray(counts, np.int64)
        seqs = counts.size
        starts = self.cache.lens[:seqs].astype(np.int32)
        offsets = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
        total = int(offsets[-1])
        positions = np.concatenate([np.arange(starts[s], starts[s] + counts[s]) for s in range(seqs)])
        seq_ids = np.repeat(np.arange(seqs), counts)
        for s in range(seqs):
            self.cache.reserve(s, int(starts[s] + counts[s]))
        self.cache.flush_table()
        self._stage(q, k, v, positions, seq_ids)
        self.q_offsets.write(offsets)
        self.starts.write(starts)
        batch = self.gpu.batch(self.buffers())
        self.record_append(batch, total)
        self.record_prefill(batch, seqs, total, int(counts.max()))
        batch.read_back(self._s(self.OUT, total * self.heads * HEAD_DIM * BF16))
        done = batch.run()
        if isinstance(done.gpu_time, Exception):
            raise done.gpu_time
        return self.out.view(np.uint16)[: total * self.heads * HEAD_DIM].reshape(total, self.heads, HEAD_DIM).copy()

    def truncate(self, seq: int, length: int) -> None:
        self.cache.truncate(seq, length)

    def free(self) -> None:
        for b in self.buffers():
            b.free()
