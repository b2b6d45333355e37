"""The whole attention block (RMSNorm, QKV projection, RoPE + append, attention, output
projection, residual) in bf16 against the CPU oracle, and its tensor-parallel split by KV group
against the unsplit block.

The oracle side follows the reference's CPU path (gpt-oss/src/model.rs:423-467) with bf16 weights
as weights/src/dense.rs:82-94 (exact widening, wide accumulation); the GPU side rounds its
activations to bf16 between stages, so the comparison has a tolerance: cosine >= 0.9995 and max
abs <= 6e-2 on a residual stream of magnitude ~3."""
import numpy as np
import pytest

from loadngo_b200 import compute
from loadngo_b200.block import HIDDEN, AttentionBlock, shard_weights
from oracle import oracle
from tests import helpers

pytestmark = pytest.mark.gpu
D = 64


def make_weights(rng):
    w_qkv = oracle.round_bf16((rng.standard_normal((5120, HIDDEN)) * 0.02).astype(np.float32))
    w_o = oracle.round_bf16((rng.standard_normal((HIDDEN, 4096)) * 0.02).astype(np.float32))
    norm = (1.0 + rng.standard_normal(HIDDEN) * 0.02).astype(np.float32)
    sinks = rng.standard_normal(64).astype(np.float32)
    return w_qkv, w_o, norm, sinks


class OracleBlock:
    def __init__(self, w_qkv, w_o, norm, sinks, seqs, capacity, window):
        self.w_qkv, self.w_o, self.norm = w_qkv.astype(np.float64), w_o.astype(np.float64), norm
        self.sessions = [oracle.Session(64, 8, D, capacity, window=window, sinks=sinks, rope=oracle.Rope(),
                                        cache_bf16=True) for _ in range(seqs)]

    def feed(self, seq, h):
        """h [t][2880] f32 -> residual after the block."""
        t = h.shape[0]
        x = np.zeros_like(h)
        for i in range(t):
            oracle.lib().oracle_rms_norm(h[i], self.norm, 1e-5, HIDDEN, x[i])
        qkv = (x.astype(np.float64) @ self.w_qkv.T).astype(np.float32)
        q, k, v = qkv[:, :4096].reshape(t, 64, D), qkv[:, 4096:4608].reshape(t, 8, D), qkv[:, 4608:].reshape(t, 8, D)
        att, _ = self.sessions[seq].feed(q, k, v, threads=8)
        o = (att.reshape(t, 4096).astype(np.float64) @ self.w_o.T).astype(np.float32)
        return h + o


@pytest.mark.parametrize("window", [0, 128])
def test_block_matches_the_oracle(gpu, window):
    rng = np.random.default_rng(41)
    w_qkv, w_o, norm, sinks = make_weights(rng)
    counts = [150, 77]
    ref = OracleBlock(w_qkv, w_o, norm, sinks, 2, 400, window)
    block = AttentionBlock(gpu, seqs=2, max_context=400, max_tokens=sum(counts), w_qkv=oracle.f32_to_bf16_bits(w_qkv),
                           w_o=oracle.f32_to_bf16_bits(w_o), norm=norm, sinks=sinks, window=window, rng=rng)
    h = oracle.round_bf16(rng.standard_normal((sum(counts), HIDDEN)).astype(np.float32))
    got = oracle.bf16_bits_to_f32(block.prefill(oracle.f32_to_bf16_bits(h), counts))
    want = np.concatenate([ref.feed(0, h[:counts[0]]), ref.feed(1, h[counts[0]:])])
    err, cos = helpers.errors(got, want)
    print(f"\nblock prefill window={window}: max_abs={err:.4f} cos={cos:.6f}")
    assert err <= 6e-2 and cos >= 0.9995
    for _ in range(3):
        hd = oracle.round_bf16(rng.standard_normal((2, HIDDEN)).astype(np.float32))
        got = oracle.bf16_bits_to_f32(block.decode(oracle.f32_to_bf16_bits(hd)))
        want = np.concatenate([ref.feed(0, hd[:1]), ref.feed(1, hd[1:])])
        err, cos = helpers.errors(got, want)
        assert err <= 6e-2 and cos >= 0.9995, f"decode step: {err} {cos}"
    block.free()


def test_split_by_kv_group_sums_to_the_unsplit_block(gpu):
    """Four ranks emulated one after the other on this GPU: each owns 2 KV groups, the matching
    rows of W_qkv and columns of W_o; the sum of their partial output projections is the unsplit
    block's (what the all-reduce computes across GPUs)."""
    rng = np.random.default_rng(43)
    w_qkv, w_o, norm, sinks = make_weights(rng)
    counts = [130]
    h = oracle.f32_to_bf16_bits(oracle.round_bf16(rng.standard_normal((130, HIDDEN)).astype(np.float32)))
    whole = AttentionBlock(gpu, seqs=1, max_context=256, max_tokens=130, w_qkv=oracle.f32_to_bf16_bits(w_qkv),
                           w_o=oracle.f32_to_bf16_bits(w_o), norm=norm, sinks=sinks)
    whole.prefill(h, counts)
    want = oracle.bf16_bits_to_f32(whole.read_partial(130))
    whole.free()
    total = np.zeros((130, HIDDEN), np.float64)
    for rank in range(4):
        lq, lo = shard_weights(w_qkv, w_o, 4, rank)
        part = AttentionBlock(gpu, seqs=1, max_context=256, max_tokens=130, w_qkv=oracle.f32_to_bf16_bits(lq),
                              w_o=oracle.f32_to_bf16_bits(lo), norm=norm, sinks=sinks[rank * 16:(rank + 1) * 16],
                              kv_local=2)
        part.prefill(h, counts)
        total += oracle.bf16_bits_to_f32(part.read_partial(130))
        part.free()
    err, cos = helpers.errors(total, want)
    print(f"\nsum of 4 shards vs unsplit output projection: max_abs={err:.4f} cos={cos:.6f}")
    assert err <= 3e-2 and cos >= 0.9999
