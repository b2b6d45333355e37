"""A gpt-oss model on the GPU, driven through the batch API exactly as `GpuModel` of the
reference drives it (gpt-oss/src/gpu.rs).

* `GpuModel.load(path, chunk, max_context)`: the GGUF header is read by the library's reader
  (`loadngo_b200.gguf`), the shape comes from its metadata (`Config.from_gguf`,
  gpt-oss/src/config.rs:38-97), every tensor goes to GPU memory as the file stores it: Q8_0
  projections and output matrix (codes and scales split, weights/src/q8_0.rs:17-31), MXFP4
  experts (repacked, weights/src/mxfp4.rs:119-149), float32 norms, biases, sinks and router.
* `GpuSession` (gpu.rs:365-413): two sets of working buffers, the key/value caches (sliding
  layers a ring), the position reached; `truncate`, `reset`.
* `GpuModel.feed(session, tokens, which)` (gpu.rs:626-676): passes of at most `chunk` positions.
  Decoding, one position: per layer `encode_attention` (gpu.rs:703-827) then
  `encode_routed_experts` (gpu.rs:829-888), then `encode_output` (gpu.rs:891-918), one
  submission per token.  A prompt pass: per layer one submission for the attention half, the
  routing and the gathering of rows by expert on the CPU (`route_and_gather`, gpu.rs:1187-1227),
  one submission for the experts (`encode_experts`, gpu.rs:1229-1286), and the weighted scatter
  into the residual on the CPU (gpu.rs:1289-1305).  Two consecutive prompt passes interleave
  layer by layer (`pass_pair`, gpu.rs:1004-1183): while the GPU runs one pass's batch the CPU
  routes the other's.

Only call sequencing lives here; every number is computed by libcuda_compute.so.
"""
from __future__ import annotations

import queue
from dataclasses import dataclass

import numpy as np

from . import compute, gguf
from .compute import FULL, Dispatch, GroupedShape, Slice

SWIGLU = (7.0, 1.702)   # limit and alpha of the clamped SwiGLU (gpt-oss/src/gpu.rs `SWIGLU`)
LAST, ALL = "last", "all"   # `Logits` (gpu.rs:319-324): which logits a pass returns


class ConfigError(Exception):
    """`ConfigError` (gpt-oss/src/config.rs:33-35)."""


class Invalid(Exception):
    """`GpuError::Invalid` (gpt-oss/src/gpu.rs:59-66)."""


@dataclass
class Config:
    """`Config` (gpt-oss/src/config.rs:5-25)."""
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
    context_length: int = 0

    def is_sliding(self, layer: int) -> bool:   # config.rs:101-103: even layers slide
        return layer % 2 == 0

    @classmethod
    def from_gguf(cls, g: "gguf.Gguf") -> "Config":
        """`Config::from_gguf` (config.rs:38-97): the same keys, the same refusals."""
        def get(key):
            if g.value_type(f"gpt-oss.{key}") < 0:
                raise ConfigError(f"gpt-oss GGUF: gpt-oss.{key} is missing")
            return g.get(f"gpt-oss.{key}"), g.value_type(f"gpt-oss.{key}")

        def integer(key):
            v, kind = get(key)
            if kind not in (0, 1, 2, 3, 4, 5, 10, 11) or v < 0:
                raise ConfigError(f"gpt-oss GGUF: gpt-oss.{key} is not an integer")
            return v

        def real(key):
            v, kind = get(key)
            if kind not in (6, 12):
                raise ConfigError(f"gpt-oss GGUF: gpt-oss.{key} is not a float")
            return v

        if g.get("general.architecture") != "gpt-oss":
            raise ConfigError("gpt-oss GGUF: general.architecture is not gpt-oss")
        if g.get("gpt-oss.rope.scaling.type") != "yarn":
            raise ConfigError("gpt-oss GGUF: only YaRN rotary scaling is implemented")
        head_dim = integer("attention.key_length")
        if integer("attention.value_length") != head_dim or head_dim % 2:
            raise ConfigError("gpt-oss GGUF: keys and values must share an even width")
        embedding = g.tensor("token_embd.weight")
        if embedding is None or len(embedding.dims) < 2:
            raise ConfigError("gpt-oss GGUF: token_embd.weight is missing")
        c = cls(layers=integer("block_count"), hidden=integer("embedding_length"), heads=integer("attention.head_count"),
                kv_heads=integer("attention.head_count_kv"), head_dim=head_dim, experts=integer("expert_count"),
                experts_used=integer("expert_used_count"), expert_hidden=integer("expert_feed_forward_length"),
                vocab=embedding.dims[1], window=integer("attention.sliding_window"),
                eps=float(np.float32(real("attention.layer_norm_rms_epsilon"))), theta=real("rope.freq_base"),
                original_context=float(integer("rope.scaling.original_context_length")),
                factor=real("rope.scaling.factor"), context_length=integer("context_length"))
        if c.kv_heads == 0 or c.heads % c.kv_heads or c.experts_used > c.experts:
            raise ConfigError("gpt-oss GGUF: inconsistent head or expert counts")
        return c


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


H, X, Q, K, V, ATT, TMP, TABLE, XE, GATE, UP, HIDDEN, YE, LOGITS, ROUTER, IDS, WEIGHTS, CACHES = range(18)   # gpu.rs:228-245
ATTENTION, EXPERTS, OUTPUT, TOKEN = "attention", "experts", "output", "token"   # `Phase`


def f(buffer: int, row: int, width: int, rows: int) -> Slice:
    """Rows `row .. row + rows` of a buffer of float32 rows `width` wide (gpu.rs:326-328)."""
    return Slice(buffer, row * width * 4, rows * width * 4)


def _pad32(n: int) -> int:
    return -(-n // 32) * 32


class GpuSession:
    """`GpuSession` (gpu.rs:365-413): two sets of working buffers, the key/value caches and the
    position reached."""

    def __init__(self, sets, caches, slots, capacity: int, rewind: int):
        self.sets, self.caches, self.slots = sets, caches, slots
        self._len, self._capacity, self.rewind = 0, capacity, rewind

    def __len__(self) -> int:
        return self._len

    def is_empty(self) -> bool:
        return self._len == 0

    def reset(self) -> None:
        """Starts the conversation over; cache rows past the new position are never read before
        they are written again."""
        self._len = 0

    def capacity(self) -> int:
        return self._capacity

    def truncate(self, length: int) -> None:
        """Goes back to position `length` (gpu.rs:397-412): at most one pass back, while the
        sliding layers' rings still hold the window before it."""
        if length > self._len or self._len - length > self.rewind:
            raise Invalid(f"cannot go back from position {self._len} to {length} (at most {self.rewind} back)")
        self._len = length

    def free(self) -> None:
        for b in self.sets[0] + self.sets[1] + self.caches:
            b.free()
        self.sets, self.caches = [[], []], []


class _Lane:
    """One of two interleaved prompt passes, as the scheduler sees it (`Lane`, gpu.rs:430-446)."""

    def __init__(self, tokens, start: int, which, buffers):
        self.tokens, self.start, self.which, self.set = tokens, start, which, buffers
        self.layer, self.ready, self.flight, self.plan, self.logits = 0, True, None, None, []


class GpuModel:
    """`GpuModel` (gpu.rs:342-362).  `tensors[name]` follows the GGUF names
    (`blk.{l}.attn_q.weight` ...); Q8_0 and MXFP4 tensors are the raw block bytes."""

    def __init__(self, gpu: compute.Gpu, config: Config, tensors: dict, chunk: int, max_context: int):
        """`GpuModel::new` (gpu.rs:449-518).  `chunk`: the most positions one pass takes (the
        reference serves with 512, gpt-oss/src/engine.rs:51); `max_context`: the positions a
        conversation can reach."""
        if chunk <= 0 or max_context <= 0:
            raise Invalid("chunk and max_context must be positive")
        c = self.config = config
        self.gpu, self.chunk, self.max_context = gpu, chunk, _pad32(max_context)
        self.gpu_routing = True     # route single positions on the GPU: one submission per token
        self.pipeline = True        # interleave consecutive prompt passes two at a time
        self.submissions = {ATTENTION: 0, EXPERTS: 0, OUTPUT: 0, TOKEN: 0}   # `Profile`, counts only
        res = gpu.resident
        f32 = lambda a, n: self._vector(a, n)
        qw, kw = c.heads * c.head_dim, c.kv_heads * c.head_dim
        self.layers = []
        for l in range(c.layers):
            t = lambda name: tensors[f"blk.{l}.{name}"]
            layer = {}
            for name, rows, cols in (("attn_q", qw, c.hidden), ("attn_k", kw, c.hidden), ("attn_v", kw, c.hidden),
                                     ("attn_output", c.hidden, qw)):
                codes, scales = split_q8_0(self._blocks(t(f"{name}.weight"), rows * cols // 32 * 34, f"blk.{l}.{name}.weight"))
                layer[name] = (res(codes), res(scales), res(f32(t(f"{name}.bias"), rows)))
            layer["attn_norm"] = res(f32(t("attn_norm.weight"), c.hidden))
            layer["ffn_norm"] = res(f32(t("post_attention_norm.weight"), c.hidden))
            layer["sinks"] = res(f32(t("attn_sinks.weight"), c.heads))
            router, router_bias = f32(t("ffn_gate_inp.weight"), c.experts * c.hidden), f32(t("ffn_gate_inp.bias"), c.experts)
            layer["router"], layer["router_bias"] = res(router), res(router_bias)
            layer["router_host"] = (router.reshape(c.experts, c.hidden), router_bias)
            for name, rows, cols in (("ffn_gate_exps", c.expert_hidden, c.hidden), ("ffn_up_exps", c.expert_hidden, c.hidden),
                                     ("ffn_down_exps", c.hidden, c.expert_hidden)):
                elements, scales = ggml_to_ocp(self._blocks(t(f"{name}.weight"), c.experts * rows * cols // 32 * 17,
                                                            f"blk.{l}.{name}.weight"))
                layer[name] = (res(elements), res(scales), res(f32(t(f"{name}.bias"), c.experts * rows)))
            self.layers.append(layer)
        codes, scales = split_q8_0(self._blocks(tensors["output.weight"], c.vocab * c.hidden // 32 * 34, "output.weight"))
        self.output = (res(codes), res(scales))
        self.output_norm = res(f32(tensors["output_norm.weight"], c.hidden))
        # the embedding stays on the CPU, as stored: `Model::embed` widens one row per token
        self.embedding = None
        if "token_embd.weight" in tensors:
            self.embedding = self._blocks(tensors["token_embd.weight"], c.vocab * c.hidden // 32 * 34,
                                          "token_embd.weight").reshape(c.vocab, c.hidden // 32, 34)

    @staticmethod
    def _vector(a, n: int) -> np.ndarray:
        v = np.ascontiguousarray(a).view(np.float32).reshape(-1) if np.asarray(a).dtype == np.uint8 else \
            np.asarray(a, np.float32).reshape(-1)
        if v.size != n:
            raise Invalid(f"want {n} f32, got {v.size}")
        return v

    @staticmethod
    def _blocks(a, nbytes: int, name: str) -> np.ndarray:
        b = np.ascontiguousarray(a, np.uint8).reshape(-1)
        if b.size != nbytes:
            raise Invalid(f"{name}: {b.size} bytes, want {nbytes}")
        return b

    @classmethod
    def load(cls, path: str, chunk: int, max_context: int, gpu: compute.Gpu | None = None) -> "GpuModel":
        """`Model::load` (gpt-oss/src/model.rs:291-309) followed by `GpuModel::new`: the header,
        the shape, then every tensor's bytes; element types and dimensions are checked as
        `Tensors::{vector, matrix, experts}` check them (model.rs:223-271)."""
        g = gguf.open(path)
        try:
            c = Config.from_gguf(g)
            qw, kw = c.heads * c.head_dim, c.kv_heads * c.head_dim
            want = {"token_embd.weight": (gguf.Q8_0, [c.hidden, c.vocab]), "output.weight": (gguf.Q8_0, [c.hidden, c.vocab]),
                    "output_norm.weight": (gguf.F32, c.hidden)}
            for l in range(c.layers):
                b = f"blk.{l}."
                want.update({
                    b + "attn_norm.weight": (gguf.F32, c.hidden), b + "post_attention_norm.weight": (gguf.F32, c.hidden),
                    b + "attn_q.weight": (gguf.Q8_0, [c.hidden, qw]), b + "attn_k.weight": (gguf.Q8_0, [c.hidden, kw]),
                    b + "attn_v.weight": (gguf.Q8_0, [c.hidden, kw]), b + "attn_output.weight": (gguf.Q8_0, [qw, c.hidden]),
                    b + "attn_q.bias": (gguf.F32, qw), b + "attn_k.bias": (gguf.F32, kw), b + "attn_v.bias": (gguf.F32, kw),
                    b + "attn_output.bias": (gguf.F32, c.hidden), b + "attn_sinks.weight": (gguf.F32, c.heads),
                    b + "ffn_gate_inp.weight": (gguf.F32, [c.hidden, c.experts]), b + "ffn_gate_inp.bias": (gguf.F32, c.experts),
                    b + "ffn_gate_exps.weight": (gguf.MXFP4, [c.hidden, c.expert_hidden, c.experts]),
                    b + "ffn_up_exps.weight": (gguf.MXFP4, [c.hidden, c.expert_hidden, c.experts]),
                    b + "ffn_down_exps.weight": (gguf.MXFP4, [c.expert_hidden, c.hidden, c.experts]),
                    b + "ffn_gate_exps.bias": (gguf.F32, c.experts * c.expert_hidden),
                    b + "ffn_up_exps.bias": (gguf.F32, c.experts * c.expert_hidden),
                    b + "ffn_down_exps.bias": (gguf.F32, c.experts * c.hidden)})
            tensors = {}
            for name, (kind, shape) in want.items():
                t = g.tensor(name)
                if t is None:
                    raise Invalid(f"{name} is missing")
                if isinstance(shape, list):
                    if t.dims != shape:
                        raise Invalid(f"{name}: dims {t.dims}, want {shape}")
                elif t.numel() != shape:
                    raise Invalid(f"{name}: want {shape} f32")
                if t.ggml_type != kind:
                    raise Invalid(f"{name}: element type {t.ggml_type}, want {kind}")
                tensors[name] = g.read(t)
        finally:
            g.close()
        return cls(gpu if gpu is not None else compute.Gpu(0), c, tensors, chunk, max_context)

    # -- sessions (gpu.rs:528-587) --------------------------------------------------------------------
    def session(self) -> GpuSession:
        return self.session_holding(self.max_context)

    def session_holding(self, capacity: int) -> GpuSession:
        """A session for at most `capacity` positions (rounded up to 32, no more than
        `max_context`): smaller full-layer caches, for short side conversations."""
        c = self.config
        capacity = min(_pad32(capacity), self.max_context)
        n = _pad32(self.chunk)
        qw, kw = c.heads * c.head_dim, c.kv_heads * c.head_dim
        # every position is routed to `experts_used` experts; each expert's rows are padded to 32
        assigned = n * c.experts_used + 32 * c.experts

        def zeroed(length: int):
            b = self.gpu.buffer(max(length, 16))
            b.zero()
            return b

        def one_set():
            return [zeroed(n * c.hidden * 4), zeroed(n * c.hidden * 4), zeroed(n * qw * 4), zeroed(n * kw * 4),
                    zeroed(n * kw * 4), zeroed(n * qw * 4), zeroed(n * c.hidden * 4), zeroed(n * c.head_dim * 4),
                    zeroed(assigned * c.hidden * 4), zeroed(assigned * c.expert_hidden * 4),
                    zeroed(assigned * c.expert_hidden * 4), zeroed(assigned * c.expert_hidden * 4),
                    zeroed(assigned * c.hidden * 4), zeroed(32 * c.vocab * 4), zeroed(c.experts * 4),
                    zeroed(c.experts_used * 4), zeroed(c.experts_used * 4)]

        sets = [one_set(), one_set()]
        caches, slots = [], []
        for l in range(c.layers):
            rows = _pad32(c.window + self.chunk) if c.is_sliding(l) else capacity
            caches += [zeroed(rows * kw * 4), zeroed(rows * kw * 4)]
            slots.append(rows)
        return GpuSession(sets, caches, slots, capacity, self.chunk)

    # -- gpu.rs:703-827 ---------------------------------------------------------------------------
    def encode_attention(self, batch, l: int, n: int, start: int, slots: int) -> None:
        c, layer = self.config, self.layers[l]
        hidden, qw, kw = c.hidden, c.heads * c.head_dim, c.kv_heads * c.head_dim
        kc, vc = CACHES + 2 * l, CACHES + 2 * l + 1
        rows_of = lambda b, w: f(b, 0, w, n)

        def mul(name, rows, cols, x, y):                  # Q8::mul (gpu.rs:121-137)
            tiled = n >= 32
            n_run = _pad32(n) if tiled else n
            x, y = Slice(x.buffer, x.offset, n_run * cols * 4), Slice(y.buffer, y.offset, n_run * rows * 4)
            m = (batch.attach(layer[name][0]), batch.attach(layer[name][1]))
            if n == 1:
                batch.gemv_q8_0(m, x, y, rows, cols)
            elif tiled:
                batch.gemm_q8_0_tiled(m, x, y, rows, cols, n_run, (cols, rows))
            else:
                batch.gemm_q8_0(m, x, y, rows, cols, n, (cols, rows))

        batch.copy_rows((rows_of(H, hidden), hidden), (rows_of(X, hidden), hidden), n, hidden)
        batch.rmsnorm_rows((rows_of(X, hidden), batch.attach(layer["attn_norm"])), n, (hidden, hidden), c.eps)
        mul("attn_q", qw, hidden, rows_of(X, hidden), rows_of(Q, qw))
        mul("attn_k", kw, hidden, rows_of(X, hidden), rows_of(K, kw))
        mul("attn_v", kw, hidden, rows_of(X, hidden), rows_of(V, kw))
        for buf, name, width in ((Q, "attn_q", qw), (K, "attn_k", kw), (V, "attn_v", kw)):
            batch.add_rows(rows_of(buf, width), (batch.attach(layer[name][2]), 0), n, width)
        table = rows_of(TABLE, c.head_dim)
        batch.rotate_halves(rows_of(Q, qw), table, n, (c.heads, c.head_dim))
        batch.rotate_halves(rows_of(K, kw), table, n, (c.kv_heads, c.head_dim))
        done = 0
        while done < n:                                   # position s goes to row s % slots, in at most two runs
            row = (start + done) % slots
            run = min(n - done, slots - row)
            for src, dst in ((K, kc), (V, vc)):
                batch.copy_rows((f(src, done, kw, run), kw), (f(dst, row, kw, run), kw), run, kw)
            done += run
        shape = GroupedShape(n, start, c.heads, c.kv_heads, c.head_dim, c.window if c.is_sliding(l) else FULL, slots,
                             1.0 / float(np.sqrt(np.float32(c.head_dim))))
        sinks = batch.attach(layer["sinks"])
        if n >= 32:
            padded, end = _pad32(n), start + n
            rows = slots if slots < end else _pad32(end)
            batch.attention_grouped_tiled_with_sinks((f(Q, 0, qw, padded), f(kc, 0, kw, rows), f(vc, 0, kw, rows)),
                                                     sinks, f(ATT, 0, qw, padded), shape)
        else:
            rows = min(slots, start + n)
            batch.attention_grouped_with_sinks((rows_of(Q, qw), f(kc, 0, kw, rows), f(vc, 0, kw, rows)), sinks,
                                               rows_of(ATT, qw), shape)
        mul("attn_output", hidden, qw, rows_of(ATT, qw), rows_of(TMP, hidden))
        batch.add_rows(rows_of(TMP, hidden), (batch.attach(layer["attn_output"][2]), 0), n, hidden)
        batch.add_rows(rows_of(H, hidden), (rows_of(TMP, hidden), hidden), n, hidden)
        batch.copy_rows((rows_of(H, hidden), hidden), (rows_of(X, hidden), hidden), n, hidden)
        batch.rmsnorm_rows((rows_of(X, hidden), batch.attach(layer["ffn_norm"])), n, (hidden, hidden), c.eps)

    # -- gpu.rs:829-888 ---------------------------------------------------------------------------
    def encode_routed_experts(self, batch, l: int) -> None:
        c, layer = self.config, self.layers[l]
        hidden, eh, k, count = c.hidden, c.expert_hidden, c.experts_used, c.experts
        g = lambda b, w, rows: Slice(b, 0, rows * w * 4)
        batch.gemv_f32((batch.attach(layer["router"]), batch.attach(layer["router_bias"])), g(X, hidden, 1),
                       g(ROUTER, count, 1), count, hidden)
        ids, weights = g(IDS, k, 1), g(WEIGHTS, k, 1)
        batch.topk_softmax(g(ROUTER, count, 1), (ids, weights), 1, (count, k))
        ge, gs, gb = (batch.attach(r) for r in layer["ffn_gate_exps"])
        batch.gemv_mxfp4_selected((ge, gs, count), ids, (g(X, hidden, 1), 0), g(GATE, eh, k), (eh, hidden), k)
        ue, us, ub = (batch.attach(r) for r in layer["ffn_up_exps"])
        batch.gemv_mxfp4_selected((ue, us, count), ids, (g(X, hidden, 1), 0), g(UP, eh, k), (eh, hidden), k)
        batch.clamped_swiglu_selected((g(GATE, eh, k), g(UP, eh, k)), (gb, ub, count), ids, g(HIDDEN, eh, k), (k, eh), SWIGLU)
        de, ds, db = (batch.attach(r) for r in layer["ffn_down_exps"])
        batch.gemv_mxfp4_selected((de, ds, count), ids, (g(HIDDEN, eh, k), eh), g(YE, hidden, k), (hidden, eh), k)
        batch.moe_combine(g(H, hidden, 1), (g(YE, hidden, k), db, count), (ids, weights), (k, hidden))

    # -- gpu.rs:1187-1227 -------------------------------------------------------------------------
    def route_and_gather(self, buffers, l: int, n: int):
        """Routes n positions on the CPU from X and gathers their rows into XE by expert, each
        expert's rows padded to 32 when its products run tiled.  Returns (by_expert, runs):
        `(position, weight)` per expert and `(expert, first row, rows)` per expert with positions."""
        c = self.config
        x = buffers[X].as_f32()[: n * c.hidden].reshape(n, c.hidden)
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
                base += _pad32(m) if m >= 32 else m
        gathered = np.zeros((max(base, 1), c.hidden), np.float32)
        for e, at, _ in runs:
            for i, (p, _) in enumerate(by_expert[e]):
                gathered[at + i] = x[p]
        buffers[XE].write(gathered)
        return by_expert, runs

    # -- gpu.rs:1229-1286 -------------------------------------------------------------------------
    def encode_experts(self, batch, l: int, plan) -> None:
        c, layer, (_, runs) = self.config, self.layers[l], plan
        hidden, eh = c.hidden, c.expert_hidden
        run_of = lambda m: _pad32(m) if m >= 32 else m

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
            mul_mxfp4(one("ffn_gate_exps", e, eh, hidden), eh, hidden, f(XE, at, hidden, run), f(GATE, at, eh, run), m)
            mul_mxfp4(one("ffn_up_exps", e, eh, hidden), eh, hidden, f(XE, at, hidden, run), f(UP, at, eh, run), m)
        batch.barrier()
        for e, at, m in runs:
            gb = part(batch.attach(layer["ffn_gate_exps"][2]), e, eh * 4)
            ub = part(batch.attach(layer["ffn_up_exps"][2]), e, eh * 4)
            batch.clamped_swiglu((f(GATE, at, eh, m), f(UP, at, eh, m)), (gb, ub), f(HIDDEN, at, eh, m), m, eh, SWIGLU)
        batch.barrier()
        for e, at, m in runs:
            run = run_of(m)
            mul_mxfp4(one("ffn_down_exps", e, hidden, eh), hidden, eh, f(HIDDEN, at, eh, run), f(YE, at, hidden, run), m)
        batch.barrier()
        for e, at, m in runs:
            db = part(batch.attach(layer["ffn_down_exps"][2]), e, hidden * 4)
            batch.add_rows(f(YE, at, hidden, m), (db, 0), m, hidden)

    # -- gpu.rs:1289-1305 -------------------------------------------------------------------------
    def scatter(self, buffers, plan, n: int) -> None:
        """Adds each position's weighted expert results to its residual row in H (on the CPU)."""
        c, (by_expert, runs) = self.config, plan
        total = max(at + m for _, at, m in runs)
        ye = buffers[YE].as_f32()[: total * c.hidden].reshape(total, c.hidden)
        h = buffers[H].as_f32()[: n * c.hidden].reshape(n, c.hidden).copy()
        for e, at, _ in runs:
            for i, (p, w) in enumerate(by_expert[e]):
                h[p] += w * ye[at + i]
        buffers[H].write(h)

    # -- gpu.rs:891-918 ---------------------------------------------------------------------------
    def encode_output(self, batch, first: int, rows: int) -> None:
        c = self.config
        hidden = c.hidden
        batch.copy_rows((f(H, first, hidden, rows), hidden), (f(X, 0, hidden, rows), hidden), rows, hidden)
        batch.rmsnorm_rows((f(X, 0, hidden, rows), batch.attach(self.output_norm)), rows, (hidden, hidden), c.eps)
        codes, scales = batch.attach(self.output[0]), batch.attach(self.output[1])
        tiled = rows >= 32
        n_run = _pad32(rows) if tiled else rows
        x, y = f(X, 0, hidden, n_run), f(LOGITS, 0, c.vocab, n_run)
        if rows == 1:
            batch.gemv_q8_0((codes, scales), x, y, c.vocab, hidden)
        elif tiled:
            batch.gemm_q8_0_tiled((codes, scales), x, y, c.vocab, hidden, n_run, (hidden, c.vocab))
        else:
            batch.gemm_q8_0((codes, scales), x, y, c.vocab, hidden, rows, (hidden, c.vocab))

    @staticmethod
    def _gathered_rows(plan) -> int:
        return max(at + (_pad32(m) if m >= 32 else m) for _, at, m in plan[1])

    @staticmethod
    def _read_back(batch, what) -> None:
        """Has the batch copy the rows the CPU reads next to the buffers' host mirrors (device and
        host memory are not one here as they are for the reference's GPU), so that reading them
        after completion does not wait for whatever the other pass has in flight."""
        for buffer, width, rows in what:
            batch.read_back(f(buffer, 0, width, rows))

    # -- submitting (gpu.rs:589-624) ----------------------------------------------------------------
    def _run(self, batch, phase: str):
        """Commits `batch` and waits until the GPU has finished; returns the buffers."""
        self.submissions[phase] += 1
        done = batch.run()
        if isinstance(done.gpu_time, Exception):
            raise done.gpu_time
        return done.buffers

    def _submit(self, batch, arrivals: "queue.Queue", lane: int, phase: str) -> None:
        """Commits `batch`; its completion arrives in `arrivals`, tagged `lane`."""
        self.submissions[phase] += 1
        batch.commit(lambda done: arrivals.put((lane, done)))

    # -- gpu.rs:626-676 ---------------------------------------------------------------------------
    def feed(self, session: GpuSession, tokens, which: str = LAST) -> list:
        """Feeds `tokens` at the session's next positions, in passes of at most `chunk`, and returns
        the logits after the last one (`LAST`) or after each (`ALL`), one array per position."""
        tokens = list(tokens)
        if len(session) + len(tokens) > session.capacity():
            raise Invalid(f"{len(session) + len(tokens)} positions exceed the session's {session.capacity()}")
        parts = [tokens[i:i + self.chunk] for i in range(0, len(tokens), self.chunk)]
        want = lambda i: ALL if which == ALL else (LAST if i + 1 == len(parts) else None)
        out, i = [], 0
        while i < len(parts):
            # two prompt passes interleave; a single position (decoding) or a last odd pass runs alone
            if self.pipeline and i + 1 < len(parts) and len(parts[i]) > 1:
                out += self.pass_pair(session, [parts[i], parts[i + 1]], [want(i), want(i + 1)])
                i += 2
            else:
                out += self.pass_(session, parts[i], want(i))
                i += 1
        return out

    def embed(self, token: int) -> np.ndarray:
        """`Model::embed` (gpt-oss/src/model.rs:501-503): the token's Q8_0 row widened, each code
        times its block's binary16 scale in float32 (weights/src/q8_0.rs:80-95)."""
        if self.embedding is None:
            raise Invalid("the model was built without token_embd.weight")
        row = self.embedding[token]
        scales = np.ascontiguousarray(row[:, :2]).view(np.float16).astype(np.float32)       # [blocks][1]
        return (scales * row[:, 2:].view(np.int8).astype(np.float32)).reshape(-1)

    def prepare(self, buffers, tokens, start: int) -> None:
        """Writes the embedding rows of `tokens` (ids, or rows already widened) and the rotary table
        for positions `start..` into a buffer set (gpu.rs:678-700)."""
        c = self.config
        rows = np.stack([self.embed(t) if np.ndim(t) == 0 else np.asarray(t, np.float32) for t in tokens])
        buffers[H].write(rows)
        buffers[TABLE].write(compute.rope_table(start, len(tokens), head_dim=c.head_dim, theta=c.theta, factor=c.factor,
                                                original_context=c.original_context))

    @staticmethod
    def _wanted(which, n: int) -> range:
        return range(0) if which is None else (range(n - 1, n) if which == LAST else range(n))

    # -- gpu.rs:929-992 ---------------------------------------------------------------------------
    def pass_(self, session: GpuSession, tokens, which) -> list:
        """One pass on its own: decoding (one submission per token when routed on the GPU) or a
        prompt pass, one submission after another."""
        c, n, start = self.config, len(tokens), len(session)
        self.prepare(session.sets[0], tokens, start)
        buffers = session.sets[0] + session.caches
        out = []
        if n == 1 and self.gpu_routing:
            batch = self.gpu.batch(buffers, Dispatch.Serial)
            for l, slots in enumerate(session.slots):
                self.encode_attention(batch, l, 1, start, slots)
                self.encode_routed_experts(batch, l)
            if which is not None:
                self.encode_output(batch, 0, 1)
                self._read_back(batch, ((LOGITS, c.vocab, 1),))
            self._run(batch, TOKEN)
            if which is not None:
                out.append(buffers[LOGITS].as_f32()[: c.vocab].copy())
        else:
            for l, slots in enumerate(session.slots):
                batch = self.gpu.batch(buffers, Dispatch.Serial)
                self.encode_attention(batch, l, n, start, slots)
                self._read_back(batch, ((X, c.hidden, n), (H, c.hidden, n)))
                self._run(batch, ATTENTION)
                plan = self.route_and_gather(buffers, l, n)
                batch = self.gpu.batch(buffers, Dispatch.Concurrent)
                self.encode_experts(batch, l, plan)
                self._read_back(batch, ((YE, c.hidden, self._gathered_rows(plan)),))
                self._run(batch, EXPERTS)
                self.scatter(buffers, plan, n)
            wanted = self._wanted(which, n)
            for first in range(wanted.start, wanted.stop, 32):
                rows = min(wanted.stop - first, 32)
                batch = self.gpu.batch(buffers, Dispatch.Serial)
                self.encode_output(batch, first, rows)
                self._read_back(batch, ((LOGITS, c.vocab, rows),))
                self._run(batch, OUTPUT)
                logits = buffers[LOGITS].as_f32()
                out += [logits[r * c.vocab:(r + 1) * c.vocab].copy() for r in range(rows)]
        session._len += n
        return out

    # -- gpu.rs:1004-1183 -------------------------------------------------------------------------
    def pass_pair(self, session: GpuSession, parts, which) -> list:
        """Two consecutive prompt passes interleaved layer by layer.  Each submission's completion
        arrives through a queue, and each one triggers the next step:
        - an attention batch finishing hands the caches to the other pass's attention when that is
          due, then the CPU routes this pass while the GPU works;
        - an experts batch finishing adds the results to the residual and makes this pass ready for
          the next layer's attention.
        Attention runs in order: first pass, then second, layer by layer.  The caches go to one
        attention batch at a time."""
        c, layers = self.config, len(self.layers)
        lanes = []
        for i in range(2):
            start = len(session) + (0 if i == 0 else len(parts[0]))
            self.prepare(session.sets[i], parts[i], start)
            lanes.append(_Lane(parts[i], start, which[i], session.sets[i]))
        caches = session.caches          # None while an attention batch holds them
        due = [0, 0]                     # the next attention due: (pass, layer)
        arrivals: "queue.Queue" = queue.Queue()
        failure = None

        def try_attention():
            """Submits the due attention when its pass is ready and the caches are free."""
            nonlocal caches
            i, l = due
            lane = lanes[i]
            if l >= layers or caches is None or not lane.ready or lane.layer != l or lane.set is None:
                return
            batch = self.gpu.batch(lane.set + caches, Dispatch.Serial)
            lane.set, caches = None, None
            self.encode_attention(batch, l, len(lane.tokens), lane.start, session.slots[l])
            self._read_back(batch, ((X, c.hidden, len(lane.tokens)), (H, c.hidden, len(lane.tokens))))
            lane.ready, lane.flight = False, ATTENTION
            self._submit(batch, arrivals, i, ATTENTION)
            due[:] = [1, l] if i == 0 else [0, l + 1]

        try_attention()
        while any(lane.layer <= layers for lane in lanes):
            i, done = arrivals.get(timeout=120)
            lane = lanes[i]
            phase, lane.flight = lane.flight, None
            if isinstance(done.gpu_time, Exception):
                # keep driving the other pass to completion so every buffer comes back, then report
                failure = failure or done.gpu_time
            if phase == ATTENTION:
                lane.set, caches = done.buffers[:CACHES], done.buffers[CACHES:]
                try_attention()              # keep the GPU fed before the CPU works
                buffers, lane.set = lane.set, None
                lane.plan = self.route_and_gather(buffers, lane.layer, len(lane.tokens))
                batch = self.gpu.batch(buffers, Dispatch.Concurrent)
                self.encode_experts(batch, lane.layer, lane.plan)
                self._read_back(batch, ((YE, c.hidden, self._gathered_rows(lane.plan)),))
                lane.flight = EXPERTS
                self._submit(batch, arrivals, i, EXPERTS)
            elif phase == EXPERTS:
                buffers = done.buffers
                self.scatter(buffers, lane.plan, len(lane.tokens))
                lane.plan = None
                lane.layer += 1
                lane.ready = True
                if lane.layer == layers:
                    wanted = self._wanted(lane.which, len(lane.tokens))
                    if len(wanted) == 0:
                        lane.layer += 1
                        lane.set = buffers
                    else:
                        # at most 32 rows a submission: the first group here, the rest as each completes
                        batch = self.gpu.batch(buffers, Dispatch.Serial)
                        self.encode_output(batch, wanted.start, min(len(wanted), 32))
                        self._read_back(batch, ((LOGITS, c.vocab, min(len(wanted), 32)),))
                        lane.flight = OUTPUT
                        self._submit(batch, arrivals, i, OUTPUT)
                else:
                    lane.set = buffers
                    try_attention()
            else:
                wanted = self._wanted(lane.which, len(lane.tokens))
                first = wanted.start + len(lane.logits)
                rows = min(wanted.stop - first, 32)
                buffers = done.buffers
                logits = buffers[LOGITS].as_f32()
                lane.logits += [logits[r * c.vocab:(r + 1) * c.vocab].copy() for r in range(rows)]
                if first + rows < wanted.stop:
                    batch = self.gpu.batch(buffers, Dispatch.Serial)
                    self.encode_output(batch, first + rows, min(wanted.stop - first - rows, 32))
                    self._read_back(batch, ((LOGITS, c.vocab, min(wanted.stop - first - rows, 32)),))
                    lane.flight = OUTPUT
                    self._submit(batch, arrivals, i, OUTPUT)
                else:
                    lane.layer += 1
                    lane.set = buffers
        if failure is not None:
            raise failure
        session._len += len(parts[0]) + len(parts[1])
        return lanes[0].logits + lanes[1].logits

    def free(self) -> None:
        """Gives the weights' GPU memory back (sessions are freed on their own)."""
        held = [self.output_norm, *self.output]
        for layer in self.layers:
            for value in layer.values():
                held += [r for r in (value if isinstance(value, tuple) else (value,)) if isinstance(r, compute.Resident)]
        for r in held:
            r.free()
        self.layers = []
