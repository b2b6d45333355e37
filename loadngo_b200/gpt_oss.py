"""A whole gpt-oss forward pass issued through the batch API exactly as `GpuModel::pass` issues it
(gpt-oss/src/gpu.rs:931-992).  Decoding, one position: per layer `encode_attention`
(gpu.rs:703-827) then `encode_routed_experts` (gpu.rs:829-888), then `encode_output`
(gpu.rs:891-918), one submission per token.  A prompt pass of n positions: per layer one
submission for the attention half, the routing and the gathering of rows by expert on the CPU
(`route_and_gather`, gpu.rs:1187-1227), one submission for the experts (`encode_experts`,
gpu.rs:1229-1286), and the weighted scatter into the residual on the CPU (gpu.rs:1289-1305).
Weights stay as the GGUF stores them: Q8_0 projections, embedding and output matrix, MXFP4
experts, float32 norms, biases, sinks and router.

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

    H, X, Q, K, V, ATT, TMP, TABLE, ROUTER, IDS, WEIGHTS, GATE, UP, HIDDEN, YE, LOGITS, XE, CACHES = range(18)

    def __init__(self, gpu: compute.Gpu, config: Config, tensors: dict, capacity: int, chunk: int = 1):
        """`chunk`: the most positions one pass takes (the reference's 512, gpt-oss/src/engine.rs:51)."""
        c = self.config = config
        self.gpu, self.capacity, self.chunk = gpu, capacity, chunk
        qw, kw = c.heads * c.head_dim, c.kv_heads * c.head_dim
        pad = -(-chunk // 32) * 32 if chunk >= 32 else chunk            # the tiled kernels read whole tiles of 32 rows
        # rows the gathered buffers need: every position goes to `experts_used` experts, and each
        # expert's run is rounded up to 32 rows when it is 32 or longer (gpu.rs:1208-1214)
        gathered = chunk * c.experts_used + 32 * c.experts
        k = c.experts_used
        rows_widths = [(pad, c.hidden), (pad, c.hidden), (pad, qw), (pad, kw), (pad, kw), (pad, qw), (pad, c.hidden),
                       (pad, c.head_dim), (1, c.experts), (1, 16), (1, 16), (max(gathered, k), c.expert_hidden),
                       (max(gathered, k), c.expert_hidden), (max(gathered, k), c.expert_hidden), (max(gathered, k), c.hidden),
                       (pad, c.vocab), (gathered, c.hidden)]
        self.buffers = [gpu.buffer(max(r * w, 4) * 4) for r, w in rows_widths]
        for b in self.buffers:
            b.zero()
        # the caches: sliding layers a ring of (window + chunk) rows rounded up to 32, full layers
        # `capacity` rounded up to 32 (gpu.rs:567-578)
        self.slots = []
        for l in range(c.layers):
            slots = -(-(c.window + chunk) // 32) * 32 if c.is_sliding(l) else -(-capacity // 32) * 32
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
            layer["router_host"] = (np.asarray(t("ffn_gate_inp.weight"), np.float32).reshape(c.experts, c.hidden),
                                    np.asarray(t("ffn_gate_inp.bias"), np.float32))
            for name in ("ffn_gate_exps", "ffn_up_exps", "ffn_down_exps"):
                elements, scales = ggml_to_ocp(t(f"{name}.weight"))
                layer[name] = (res(elements), res(scales), res(np.asarray(t(f"{name}.bias"), np.float32)))
            self.layers.append(layer)
        codes, scales = split_q8_0(tensors["output.weight"])
        self.output = (res(codes), res(scales))
        self.output_norm = res(np.asarray(tensors["output_norm.weight"], np.float32))
        self.len = 0

    # -- gpu.rs:703-827 ---------------------------------------------------------------------------
    def encode_attention(self, batch, l: int, start: int, n: int = 1) -> None:
        c, layer, slots = self.config, self.layers[l], self.slots[l]
        hidden, qw, kw = c.hidden, c.heads * c.head_dim, c.kv_heads * c.head_dim
        kc, vc = self.CACHES + 2 * l, self.CACHES + 2 * l + 1
        f = lambda b, row, w, rows: Slice(b, row * w * 4, rows * w * 4)
        rows_of = lambda b, w: f(b, 0, w, n)

        def mul(name, rows, cols, x, y):                  # Q8::mul (gpu.rs:121-137)
            tiled = n >= 32
            n_run = -(-n // 32) * 32 if tiled else n
            x, y = Slice(x.buffer, x.offset, n_run * cols * 4), Slice(y.buffer, y.offset, n_run * rows * 4)
            m = (batch.attach(layer[name][0]), batch.attach(layer[name][1]))
            if n == 1:
                batch.gemv_q8_0(m, x, y, rows, cols)
            elif tiled:
                batch.gemm_q8_0_tiled(m, x, y, rows, cols, n_run, (cols, rows))
            else:
                batch.gemm_q8_0(m, x, y, rows, cols, n, (cols, rows))

        batch.copy_rows((rows_of(self.H, hidden), hidden), (rows_of(self.X, hidden), hidden), n, hidden)
        batch.rmsnorm_rows((rows_of(self.X, hidden), batch.attach(layer["attn_norm"])), n, (hidden, hidden), c.eps)
        mul("attn_q", qw, hidden, rows_of(self.X, hidden), rows_of(self.Q, qw))
        mul("attn_k", kw, hidden, rows_of(self.X, hidden), rows_of(self.K, kw))
        mul("attn_v", kw, hidden, rows_of(self.X, hidden), rows_of(self.V, kw))
        for buf, name, width in ((self.Q, "attn_q", qw), (self.K, "attn_k", kw), (self.V, "attn_v", kw)):
            batch.add_rows(rows_of(buf, width), (batch.attach(layer[name][2]), 0), n, width)
        table = rows_of(self.TABLE, c.head_dim)
        batch.rotate_halves(rows_of(self.Q, qw), table, n, (c.heads, c.head_dim))
        batch.rotate_halves(rows_of(self.K, kw), table, n, (c.kv_heads, c.head_dim))
        done = 0
        while done < n:                                   # position s goes to row s % slots, in at most two runs
            row = (start + done) % slots
            run = min(n - done, slots - row)
            for src, dst in ((self.K, kc), (self.V, vc)):
                batch.copy_rows((f(src, done, kw, run), kw), (f(dst, row, kw, run), kw), run, kw)
            done += run
        shape = GroupedShape(n, start, c.heads, c.kv_heads, c.head_dim, c.window if c.is_sliding(l) else FULL, slots,
                             1.0 / float(np.sqrt(np.float32(c.head_dim))))
        sinks = batch.attach(layer["sinks"])
        if n >= 32:
            padded, end = -(-n // 32) * 32, start + n
            rows = slots if slots < end else -(-end // 32) * 32
            batch.attention_grouped_tiled_with_sinks((f(self.Q, 0, qw, padded), f(kc, 0, kw, rows), f(vc, 0, kw, rows)),
                                                     sinks, f(self.ATT, 0, qw, padded), shape)
        else:
            rows = min(slots, start + n)
            batch.attention_grouped_with_sinks((rows_of(self.Q, qw), f(kc, 0, kw, rows), f(vc, 0, kw, rows)), sinks,
                                               rows_of(self.ATT, qw), shape)
        mul("attn_output", hidden, qw, rows_of(self.ATT, qw), rows_of(self.TMP, hidden))
        batch.add_rows(rows_of(self.TMP, hidden), (batch.attach(layer["attn_output"][2]), 0), n, hidden)
        batch.add_rows(rows_of(self.H, hidden), (rows_of(self.TMP, hidden), hidden), n, hidden)
        batch.copy_rows((rows_of(self.H, hidden), hidden), (rows_of(self.X, hidden), hidden), n, hidden)
        batch.rmsnorm_rows((rows_of(self.X, hidden), batch.attach(layer["ffn_norm"])), n, (hidden, hidden), c.eps)

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

    # -- gpu.rs:1187-1227 -------------------------------------------------------------------------
    def route_and_gather(self, l: int, n: int):
        """Routes n positions on the CPU from X and gathers their rows into XE by expert, each
        expert's rows padded to 32 when its products run tiled.  Returns (by_expert, runs)."""
        c = self.config
        x = self.buffers[self.X].as_f32()[: n * c.hidden].reshape(n, c.hidden)
        w, bias = self.layers[l]["router_host"]
        logits = (x @ w.T + bias).astype(np.float32)            # `route_all`: the CPU model's router
        by_expert = [[] for _ in range(c.experts)]
        for p in range(n):
            order = sorted(range(c.experts), key=lambda e: (-logits[p, e], e))[: c.experts_used]   # ties: lower index
            weights = np.exp(logits[p, order] - logits[p, order[0]]).astype(np.float32)
            weights = weights / weights.sum(dtype=np.float32)
            for e, wt in zip(order, weights):
                by_expert[e].append((p, np.float32(wt)))
        runs, base = [], 0
        for e, rows in enumerate(by_expert):
            if rows:
                m = len(rows)
                runs.append((e, base, m))
                base += -(-m // 32) * 32 if m >= 32 else m
        gathered = np.zeros((max(base, 1), c.hidden), np.float32)
        for e, at, _ in runs:
            for i, (p, _) in enumerate(by_expert[e]):
                gathered[at + i] = x[p]
        self.buffers[self.XE].write(gathered)
        return by_expert, runs

    # -- gpu.rs:1229-1286 -------------------------------------------------------------------------
    def encode_experts(self, batch, l: int, runs) -> None:
        c, layer = self.config, self.layers[l]
        hidden, eh = c.hidden, c.expert_hidden
        f = lambda b, row, w, rows: Slice(b, row * w * 4, rows * w * 4)
        run_of = lambda m: -(-m // 32) * 32 if m >= 32 else m

        def one(name, e, rows, cols):                    # ExpertMatrices::one: expert e's part of the residents
            el, sc = batch.attach(layer[name][0]), batch.attach(layer[name][1])
            return (Slice(el.buffer, el.offset + e * rows * cols // 2, rows * cols // 2),
                    Slice(sc.buffer, sc.offset + e * rows * cols // 32, rows * cols // 32))

        def mul_mxfp4(matrix, rows, cols, x, y, m):      # gpu.rs:76-96
            tiled = m >= 32
            n_run = run_of(m)
            x, y = Slice(x.buffer, x.offset, n_run * cols * 4), Slice(y.buffer, y.offset, n_run * rows * 4)
            if m == 1:
                batch.gemv_mxfp4(matrix[0], matrix[1], x, y, rows, cols)
            elif tiled:
                batch.gemm_mxfp4_tiled(matrix[0], matrix[1], x, y, rows, cols, n_run, (cols, rows))
            else:
                batch.gemm_mxfp4(matrix[0], matrix[1], x, y, rows, cols, m, (cols, rows))

        part = lambda s_, e, nbytes: Slice(s_.buffer, s_.offset + e * nbytes, nbytes)
        for e, at, m in runs:
            run = run_of(m)
            mul_mxfp4(one("ffn_gate_exps", e, eh, hidden), eh, hidden, f(self.XE, at, hidden, run), f(self.GATE, at, eh, run), m)
            mul_mxfp4(one("ffn_up_exps", e, eh, hidden), eh, hidden, f(self.XE, at, hidden, run), f(self.UP, at, eh, run), m)
        batch.barrier()
        for e, at, m in runs:
            gb = part(batch.attach(layer["ffn_gate_exps"][2]), e, eh * 4)
            ub = part(batch.attach(layer["ffn_up_exps"][2]), e, eh * 4)
            batch.clamped_swiglu((f(self.GATE, at, eh, m), f(self.UP, at, eh, m)), (gb, ub), f(self.HIDDEN, at, eh, m), m, eh,
                                 SWIGLU)
        batch.barrier()
        for e, at, m in runs:
            run = run_of(m)
            mul_mxfp4(one("ffn_down_exps", e, hidden, eh), hidden, eh, f(self.HIDDEN, at, eh, run), f(self.YE, at, hidden, run), m)
        batch.barrier()
        for e, at, m in runs:
            db = part(batch.attach(layer["ffn_down_exps"][2]), e, hidden * 4)
            batch.add_rows(f(self.YE, at, hidden, m), (db, 0), m, hidden)

    # -- gpu.rs:1289-1305 -------------------------------------------------------------------------
    def scatter(self, n: int, by_expert, runs) -> None:
        """Adds each position's weighted expert results to its residual row in H (on the CPU)."""
        c = self.config
        total = max(at + m for _, at, m in runs)
        ye = self.buffers[self.YE].as_f32()[: total * c.hidden].reshape(total, c.hidden)
        h = self.buffers[self.H].as_f32()[: n * c.hidden].reshape(n, c.hidden).copy()
        for e, at, _ in runs:
            for i, (p, w) in enumerate(by_expert[e]):
                h[p] += w * ye[at + i]
        self.buffers[self.H].write(h)

    # -- gpu.rs:891-918 ---------------------------------------------------------------------------
    def encode_output(self, batch, first: int = 0, rows: int = 1) -> None:
        c = self.config
        hidden = c.hidden
        f = lambda b, row, w, r: Slice(b, row * w * 4, r * w * 4)
        batch.copy_rows((f(self.H, first, hidden, rows), hidden), (f(self.X, 0, hidden, rows), hidden), rows, hidden)
        batch.rmsnorm_rows((f(self.X, 0, hidden, rows), batch.attach(self.output_norm)), rows, (hidden, hidden), c.eps)
        codes, scales = batch.attach(self.output[0]), batch.attach(self.output[1])
        tiled = rows >= 32
        n_run = -(-rows // 32) * 32 if tiled else rows
        x, y = f(self.X, 0, hidden, n_run), f(self.LOGITS, 0, c.vocab, n_run)
        if rows == 1:
            batch.gemv_q8_0((codes, scales), x, y, c.vocab, hidden)
        elif tiled:
            batch.gemm_q8_0_tiled((codes, scales), x, y, c.vocab, hidden, n_run, (hidden, c.vocab))
        else:
            batch.gemm_q8_0((codes, scales), x, y, c.vocab, hidden, rows, (hidden, c.vocab))

    def _run(self, batch) -> None:
        done = batch.run()
        if isinstance(done.gpu_time, Exception):
            raise done.gpu_time

    def _table(self, start: int, n: int) -> None:
        c = self.config
        self.buffers[self.TABLE].write(compute.rope_table(start, n, head_dim=c.head_dim, theta=c.theta, factor=c.factor,
                                                          original_context=c.original_context))

    def step(self, embedded: np.ndarray) -> np.ndarray:
        """One position: `embedded` is the token's embedding row (the reference widens it on the CPU,
        gpu.rs:681-699); returns the logits.  One submission, as `pass` makes for decoding."""
        c, start = self.config, self.len
        assert start < self.capacity
        self.buffers[self.H].write(np.asarray(embedded, np.float32))
        self._table(start, 1)
        batch = self.gpu.batch(self.buffers)
        for l in range(c.layers):
            self.encode_attention(batch, l, start)
            self.encode_routed_experts(batch, l)
        self.encode_output(batch)
        self._run(batch)
        self.len += 1
        return self.buffers[self.LOGITS].as_f32()[: c.vocab].copy()

    def prompt_pass(self, embedded: np.ndarray, all_logits: bool = False) -> np.ndarray:
        """A pass of n <= chunk positions (`embedded` [n][hidden]): per layer two submissions with the
        routing, gathering and scattering on the CPU in between, as `pass` does for a prompt
        (gpu.rs:960-992).  Returns the logits of the last position, or of all of them."""
        c, start = self.config, self.len
        n = embedded.shape[0]
        assert 1 <= n <= self.chunk and start + n <= self.capacity
        self.buffers[self.H].write(np.asarray(embedded, np.float32))
        self._table(start, n)
        for l in range(c.layers):
            batch = self.gpu.batch(self.buffers)
            self.encode_attention(batch, l, start, n)
            self._run(batch)
            by_expert, runs = self.route_and_gather(l, n)
            batch = self.gpu.batch(self.buffers)
            self.encode_experts(batch, l, runs)
            self._run(batch)
            self.scatter(n, by_expert, runs)
        first, rows = (0, n) if all_logits else (n - 1, 1)
        batch = self.gpu.batch(self.buffers)
        self.encode_output(batch, first, rows)
        self._run(batch)
        self.len += n
        return self.buffers[self.LOGITS].as_f32()[: rows * c.vocab].reshape(rows, c.vocab).copy()

    def truncate(self, length: int) -> None:
        """`GpuSession::truncate` for a rewind the sliding rings still cover (gpu.rs:397-412)."""
        assert 0 <= length <= self.len
        self.len = length

    def free(self) -> None:
        for b in self.buffers:
            b.free()
