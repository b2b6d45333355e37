"""A whole gpt-oss forward pass for one position at a time, issued through the batch API exactly
as `GpuModel::pass` issues it for decoding with the experts routed on the GPU
(gpt-oss/src/gpu.rs:931-992): per layer `encode_attention` (gpu.rs:703-827) then
`encode_routed_experts` (gpu.rs:829-888), then `encode_output` (gpu.rs:891-918), one submission
per token.  Weights stay as the GGUF stores them: Q8_0 projections, embedding and output matrix,
MXFP4 experts, float32 norms, biases, sinks and router.

Only call sequencing lives here; every number is computed by libcuda_compute.so.  Reading GGUF
files is not part of this package: the constructor takes the tensors as arrays.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from . import compute
from .compute import FULL, GroupedShape, Slice

SWIGLU = (7.0, 1.702)   # limit and alpha of the clamped SwiGLU (gpt-oss/src/gpu.rs `SWIGLU`)


@dataclass
class Config:
    """The fields of `Config` (gpt-oss/src/config.rs:38-97) this pass needs."""
    layers: int
    hidden: int
    heads: int
    kv_heads: int
    head_dim: int
    window: int
    eps: float
    experts: int
    experts_used: int
    expert_hidden: int
    vocab: int
    theta: float
    factor: float
    original_context: float

    def is_sliding(self, layer: int) -> bool:   # config.rs:101-103: even layers slide
        return layer % 2 == 0


def split_q8_0(blocks: np.ndarray):
    """`split_blocks` (weights/src/q8_0.rs:17-31): the codes in order, then the scales."""
    b = np.ascontiguousarray(blocks, np.uint8).reshape(-1, 34)
    return np.ascontiguousarray(b[:, 2:]).reshape(-1), np.ascontiguousarray(b[:, :2]).reshape(-1)


def ggml_to_ocp(blocks: np.ndarray):
    """`ggml_to_ocp` (weights/src/mxfp4.rs:119-149): low nibbles are elements 0-15 of a block,
    high nibbles 16-31; repacked two per byte with the even element in the low nibble."""
    b = np.ascontiguousarray(blocks, np.uint8).reshape(-1, 17)
    lo, hi = b[:, 1:] & 0x0f, b[:, 1:] >> 4
    codes = np.concatenate([lo, hi], axis=1)                      # elements 0..31 of every block
    elements = (codes[:, 0::2] | (codes[:, 1::2] << 4)).astype(np.uint8)
    return np.ascontiguousarray(elements).reshape(-1), np.ascontiguousarray(b[:, 0])


class GpuModel:
    """Decoding one token per submission.  `tensors[name]` follows the GGUF names
    (`blk.{l}.attn_q.weight` ...); Q8_0 and MXFP4 tensors are the raw block bytes."""

    H, X, Q, K, V, ATT, TMP, TABLE, ROUTER, IDS, WEIGHTS, GATE, UP, HIDDEN, YE, LOGITS, CACHES = range(17)

    def __init__(self, gpu: compute.Gpu, config: Config, tensors: dict, capacity: int):
        c = self.config = config
        self.gpu, self.capacity = gpu, capacity
        qw, kw = c.heads * c.head_dim, c.kv_heads * c.head_dim
        widths = [c.hidden, c.hidden, qw, kw, kw, qw, c.hidden, c.head_dim, c.experts, 16, 16,
                  c.experts_used * c.expert_hidden, c.experts_used * c.expert_hidden, c.experts_used * c.expert_hidden,
                  c.experts_used * c.hidden, c.vocab]
        self.buffers = [gpu.buffer(max(w, 4) * 4) for w in widths]
        # the caches: sliding layers a ring of (window + 1 positions) rounded up to 32 rows, full
        # layers `capacity` rounded up to 32 (gpu.rs:567-578 with one position per pass)
        self.slots = []
        for l in range(c.layers):
            slots = -(-(c.window + 1) // 32) * 32 if c.is_sliding(l) else -(-capacity // 32) * 32
            self.slots.append(slots)
            for _ in range(2):
                cache = gpu.buffer(slots * kw * 4)
                cache.zero()
                self.buffers.append(cache)
        res = gpu.resident
        self.layers = []
        for l in range(c.layers):
            t = lambda name: tensors[f"blk.{l}.{name}"]
            layer = {}
            for name in ("attn_q", "attn_k", "attn_v", "attn_output"):
                codes, scales = split_q8_0(t(f"{name}.weight"))
                layer[name] = (res(codes), res(scales), res(np.asarray(t(f"{name}.bias"), np.float32)))
            layer["attn_norm"] = res(np.asarray(t("attn_norm.weight"), np.float32))
            layer["ffn_norm"] = res(np.asarray(t("post_attention_norm.weight"), np.float32))
            layer["sinks"] = res(np.asarray(t("attn_sinks.weight"), np.float32))
            layer["router"] = res(np.asarray(t("ffn_gate_inp.weight"), np.float32))
            layer["router_bias"] = res(np.asarray(t("ffn_gate_inp.bias"), np.float32))
            for name in ("ffn_gate_exps", "ffn_up_exps", "ffn_down_exps"):
                elements, scales = ggml_to_ocp(t(f"{name}.weight"))
                layer[name] = (res(elements), res(scales), res(np.asarray(t(f"{name}.bias"), np.float32)))
            self.layers.append(layer)
        codes, scales = split_q8_0(tensors["output.weight"])
        self.output = (res(codes), res(scales))
        self.output_norm = res(np.asarray(tensors["output_norm.weight"], np.float32))
        self.len = 0

    # -- gpu.rs:703-827 ---------------------------------------------------------------------------
    def encode_attention(self, batch, l: int, start: int) -> None:
        c, layer, slots = self.config, self.layers[l], self.slots[l]
        hidden, qw, kw = c.hidden, c.heads * c.head_dim, c.kv_heads * c.head_dim
        kc, vc = self.CACHES + 2 * l, self.CACHES + 2 * l + 1
        f = lambda b, row, w, rows: Slice(b, row * w * 4, rows * w * 4)
        row_of = lambda b, w: f(b, 0, w, 1)

        def mul(name, rows, cols, x, y):                  # Q8::mul with n = 1 (gpu.rs:121-137)
            batch.gemv_q8_0((batch.attach(layer[name][0]), batch.attach(layer[name][1])), x, y, rows, cols)

        batch.copy_rows((row_of(self.H, hidden), hidden), (row_of(self.X, hidden), hidden), 1, hidden)
        batch.rmsnorm_rows((row_of(self.X, hidden), batch.attach(layer["attn_norm"])), 1, (hidden, hidden), c.eps)
        mul("attn_q", qw, hidden, row_of(self.X, hidden), row_of(self.Q, qw))
        mul("attn_k", kw, hidden, row_of(self.X, hidden), row_of(self.K, kw))
        mul("attn_v", kw, hidden, row_of(self.X, hidden), row_of(self.V, kw))
        for buf, name, width in ((self.Q, "attn_q", qw), (self.K, "attn_k", kw), (self.V, "attn_v", kw)):
            batch.add_rows(row_of(buf, width), (batch.attach(layer[name][2]), 0), 1, width)
        table = row_of(self.TABLE, c.head_dim)
        batch.rotate_halves(row_of(self.Q, qw), table, 1, (c.heads, c.head_dim))
        batch.rotate_halves(row_of(self.K, kw), table, 1, (c.kv_heads, c.head_dim))
        row = start % slots
        for src, dst in ((self.K, kc), (self.V, vc)):
            batch.copy_rows((row_of(src, kw), kw), (f(dst, row, kw, 1), kw), 1, kw)
        shape = GroupedShape(1, start, c.heads, c.kv_heads, c.head_dim, c.window if c.is_sliding(l) else FULL, slots,
                             1.0 / float(np.sqrt(np.float32(c.head_dim))))
        rows = min(slots, start + 1)
        batch.attention_grouped_with_sinks((row_of(self.Q, qw), f(kc, 0, kw, rows), f(vc, 0, kw, rows)),
                                           batch.attach(layer["sinks"]), row_of(self.ATT, qw), shape)
        mul("attn_output", hidden, qw, row_of(self.ATT, qw), row_of(self.TMP, hidden))
        batch.add_rows(row_of(self.TMP, hidden), (batch.attach(layer["attn_output"][2]), 0), 1, hidden)
        batch.add_rows(row_of(self.H, hidden), (row_of(self.TMP, hidden), hidden), 1, hidden)
        batch.copy_rows((row_of(self.H, hidden), hidden), (row_of(self.X, hidden), hidden), 1, hidden)
        batch.rmsnorm_rows((row_of(self.X, hidden), batch.attach(layer["ffn_norm"])), 1, (hidden, hidden), c.eps)

    # -- gpu.rs:829-888 ---------------------------------------------------------------------------
    def encode_routed_experts(self, batch, l: int) -> None:
        c, layer = self.config, self.layers[l]
        hidden, eh, k, count = c.hidden, c.expert_hidden, c.experts_used, c.experts
        f = lambda b, w, rows: Slice(b, 0, rows * w * 4)
        batch.gemv_f32((batch.attach(layer["router"]), batch.attach(layer["router_bias"])), f(self.X, hidden, 1),
                       f(self.ROUTER, count, 1), count, hidden)
        ids, weights = f(self.IDS, k, 1), f(self.WEIGHTS, k, 1)
        batch.topk_softmax(f(self.ROUTER, count, 1), (ids, weights), 1, (count, k))
        ge, gs, gb = (batch.attach(r) for r in layer["ffn_gate_exps"])
        batch.gemv_mxfp4_selected((ge, gs, count), ids, (f(self.X, hidden, 1), 0), f(self.GATE, eh, k), (eh, hidden), k)
        ue, us, ub = (batch.attach(r) for r in layer["ffn_up_exps"])
        batch.gemv_mxfp4_selected((ue, us, count), ids, (f(self.X, hidden, 1), 0), f(self.UP, eh, k), (eh, hidden), k)
        batch.clamped_swiglu_selected((f(self.GATE, eh, k), f(self.UP, eh, k)), (gb, ub, count), ids,
                                      f(self.HIDDEN, eh, k), (k, eh), SWIGLU)
        de, ds, db = (batch.attach(r) for r in layer["ffn_down_exps"])
        batch.gemv_mxfp4_selected((de, ds, count), ids, (f(self.HIDDEN, eh, k), eh), f(self.YE, hidden, k), (hidden, eh), k)
        batch.moe_combine(f(self.H, hidden, 1), (f(self.YE, hidden, k), db, count), (ids, weights), (k, hidden))

    # -- gpu.rs:891-918 ---------------------------------------------------------------------------
    def encode_output(self, batch) -> None:
        c = self.config
        hidden = c.hidden
        one = lambda b, w: Slice(b, 0, w * 4)
        batch.copy_rows((one(self.H, hidden), hidden), (one(self.X, hidden), hidden), 1, hidden)
        batch.rmsnorm_rows((one(self.X, hidden), batch.attach(self.output_norm)), 1, (hidden, hidden), c.eps)
        batch.gemv_q8_0((batch.attach(self.output[0]), batch.attach(self.output[1])), one(self.X, hidden),
                        one(self.LOGITS, c.vocab), c.vocab, hidden)

    def step(self, embedded: np.ndarray) -> np.ndarray:
        """One position: `embedded` is the token's embedding row (the reference widens it on the CPU,
        gpu.rs:681-699); returns the logits.  One submission, as `pass` makes for decoding."""
        c, start = self.config, self.len
        assert start < self.capacity
        self.buffers[self.H].write(np.asarray(embedded, np.float32))
        self.buffers[self.TABLE].write(compute.rope_table(start, 1, head_dim=c.head_dim, theta=c.theta, factor=c.factor,
                                                          original_context=c.original_context))
        batch = self.gpu.batch(self.buffers)
        for l in range(c.layers):
            self.encode_attention(batch, l, start)
            self.encode_routed_experts(batch, l)
        self.encode_output(batch)
        done = batch.run()
        if isinstance(done.gpu_time, Exception):
            raise done.gpu_time
        self.len += 1
        return self.buffers[self.LOGITS].as_f32()[: c.vocab].copy()

    def truncate(self, length: int) -> None:
        """`GpuSession::truncate` for a rewind the sliding rings still cover (gpu.rs:397-412)."""
        assert 0 <= length <= self.len
        self.len = length

    def free(self) -> None:
        for b in self.buffers:
            b.free()
