"""Shared test helpers: seeded inputs, page packing, error measures."""
from __future__ import annotations

import numpy as np

from oracle import oracle

PAGE, D = 16, 64


def xorshift_values(seed: int, n: int) -> np.ndarray:
    """The deterministic inputs of the reference's kernel tests, values in [-1, 1)
    (metal-compute/tests/attention_grouped.rs:25-35)."""
    return oracle.xorshift_values(seed, n)


def config1_inputs(positions: int = 320, heads: int = 64, kv_heads: int = 8, seed: int = 0):
    """Config-1 draw order: q, k, v standard normal -> f32 -> bf16 (RNE); sinks f32."""
    rng = np.random.default_rng(seed)
    q = oracle.round_bf16(rng.standard_normal((positions, heads, D)).astype(np.float32))
    k = oracle.round_bf16(rng.standard_normal((positions, kv_heads, D)).astype(np.float32))
    v = oracle.round_bf16(rng.standard_normal((positions, kv_heads, D)).astype(np.float32))
    sinks = rng.standard_normal(heads).astype(np.float32)
    return q, k, v, sinks


def pack_pages(kcache: np.ndarray, vcache: np.ndarray, block_row: np.ndarray, pool: np.ndarray,
               ring_pages: int = 0) -> None:
    """Writes f32 caches [len][kv_heads][64] (already bf16-representable) into `pool`
    ([pages][kv_heads][2][16][64] uint16) at the pages `block_row` names."""
    length = kcache.shape[0]
    kb, vb = oracle.f32_to_bf16_bits(kcache), oracle.f32_to_bf16_bits(vcache)
    first = 0
    if ring_pages:
        first = max(0, (-(-length // PAGE) - ring_pages) * PAGE)
    pos = np.arange(first, length)
    lp = pos // PAGE
    pages = np.asarray(block_row)[lp % ring_pages if ring_pages else lp]
    pool[pages, :, 0, pos % PAGE, :] = kb[first:]
    pool[pages, :, 1, pos % PAGE, :] = vb[first:]


def decode_f64(q_rot: np.ndarray, kcache: np.ndarray, vcache: np.ndarray, length: int, window: int,
               scale: float, sinks) -> np.ndarray:
    """float64 definition (metal-compute/tests/attention_grouped.rs:65-100) for ONE query at
    position length - 1: q_rot [heads][64], caches [>= length][kv_heads][64]."""
    heads = q_rot.shape[0]
    kv_heads = kcache.shape[1]
    group = heads // kv_heads
    first = max(0, length - window) if window > 0 else 0
    out = np.zeros((heads, q_rot.shape[1]), np.float64)
    for g in range(kv_heads):
        k = kcache[first:length, g].astype(np.float64)
        v = vcache[first:length, g].astype(np.float64)
        s = (q_rot[g * group:(g + 1) * group].astype(np.float64) @ k.T) * float(scale)
        sink = np.full(group, -np.inf) if sinks is None else sinks[g * group:(g + 1) * group].astype(np.float64)
        m = np.maximum(s.max(axis=1), sink)
        e = np.exp(s - m[:, None])
        z = e.sum(axis=1) + np.exp(sink - m)
        out[g * group:(g + 1) * group] = (e / z[:, None]) @ v
    return out


def errors(got: np.ndarray, want: np.ndarray):
    got = np.asarray(got, np.float64).reshape(-1)
    want = np.asarray(want, np.float64).reshape(-1)
    max_abs = float(np.abs(got - want).max()) if got.size else 0.0
    denom = np.linalg.norm(got) * np.linalg.norm(want)
    cosine = float(got @ want / denom) if denom > 0 else 1.0
    return max_abs, cosine
