"""The host side of a conversation without a GPU: `GpuSession`, `feed`'s splitting into passes and
the scheduler that interleaves two prompt passes (gpt-oss/src/gpu.rs:365-413, 626-676, 1004-1183),
run against a stand-in for the device that computes nothing but enforces the batch API's
ownership rule: a buffer belongs to one batch from `Gpu::batch` until that batch's completion,
and the CPU touches it only in between (metal-compute/src/apple.rs:365-390, 536-539)."""
import json
import os
import random
import threading
import time

import numpy as np
import pytest

from loadngo_b200.compute import Completed, Slice
from loadngo_b200.gpt_oss import ALL, CACHES, LAST, Config, GpuModel, Invalid

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "tiny_block.npz")


class FakeBuffer:
    def __init__(self, length):
        self.data, self.owner = np.zeros(-(-length // 4), np.float32), None

    def _mine(self):
        assert self.owner is None, "the CPU touched a buffer a batch owns"

    def as_f32(self):
        self._mine()
        return self.data

    def write(self, array, offset=0):
        self._mine()
        flat = np.ascontiguousarray(array, np.float32).reshape(-1)
        self.data[offset // 4: offset // 4 + flat.size] = flat

    def zero(self):
        self._mine()
        self.data[:] = 0

    def free(self):
        self._mine()


class FakeBatch:
    def __init__(self, gpu, buffers, dispatch):
        for b in buffers:
            assert b.owner is None, "a buffer was given to two batches at once"
            b.owner = self
        self.gpu, self.buffers, self.dispatch, self.calls = gpu, list(buffers), dispatch, []

    def attach(self, resident):
        return Slice(len(self.buffers) + resident, 0, 0)

    def __getattr__(self, name):                    # every dispatch is recorded, none computes
        def record(*args):
            self.calls.append((name, args))
        return record

    def _finish(self):
        for b in self.buffers:
            b.owner = None
        return Completed(self.buffers, 1e-6)

    def run(self):
        self.gpu.log.append(("run", self))
        return self._finish()

    def commit(self, callback):
        self.gpu.log.append(("commit", self))
        self.gpu.pending.append((self, callback))
        self.gpu.wake.set()


class FakeGpu:
    """One queue: batches finish in commit order, each after a short random time, and the
    completion runs on another thread, as the library's completion thread does."""

    def __init__(self):
        self.log, self.pending, self.wake, self.residents = [], [], threading.Event(), 0
        self.stop = False
        self.thread = threading.Thread(target=self._completions, daemon=True)
        self.thread.start()

    def _completions(self):
        rng = random.Random(7)
        while not self.stop:
            self.wake.wait(0.05)
            self.wake.clear()
            while self.pending:
                batch, callback = self.pending.pop(0)
                time.sleep(rng.random() * 0.002)
                self.log.append(("done", batch))
                callback(batch._finish())

    def buffer(self, length):
        return FakeBuffer(length)

    def resident(self, data):
        self.residents += 1
        return self.residents

    def batch(self, buffers, dispatch=0):
        return FakeBatch(self, buffers, dispatch)


@pytest.fixture()
def model():
    g = np.load(GOLDEN)
    m = json.loads(str(g["meta"]))
    cfg = Config(layers=m["layers"], hidden=m["hidden"], heads=m["heads"], kv_heads=m["kv_heads"], head_dim=m["dim"],
                 window=m["window"], eps=m["eps"], experts=m["experts"], experts_used=m["experts_used"],
                 expert_hidden=m["expert_hidden"], vocab=m["vocab"], theta=m["theta"], factor=m["factor"],
                 original_context=float(m["original_context"]))
    tensors = {"output.weight": g["output_q8_0"], "output_norm.weight": g["output_norm"], "token_embd.weight": g["token_embd_q8_0"]}
    for l in range(cfg.layers):
        for name in ("attn_q", "attn_k", "attn_v", "attn_output"):
            tensors[f"blk.{l}.{name}.weight"] = g[f"l{l}_{name}_q8_0"]
            tensors[f"blk.{l}.{name}.bias"] = g[f"l{l}_{name}_bias"]
        for name, key in (("attn_norm.weight", "attn_norm"), ("post_attention_norm.weight", "ffn_norm"),
                          ("attn_sinks.weight", "sinks"), ("ffn_gate_inp.weight", "router"), ("ffn_gate_inp.bias", "router_bias")):
            tensors[f"blk.{l}.{name}"] = g[f"l{l}_{key}"]
        for name in ("ffn_gate_exps", "ffn_up_exps", "ffn_down_exps"):
            tensors[f"blk.{l}.{name}.weight"] = g[f"l{l}_{name}_mxfp4"]
            tensors[f"blk.{l}.{name}.bias"] = g[f"l{l}_{name}_bias"]
    gpu = FakeGpu()
    made = lambda chunk, max_context=64: GpuModel(gpu, cfg, tensors, chunk, max_context)
    yield made, gpu, [int(t) for t in g["ids"]], g
    gpu.stop = True


def test_embedding_rows_are_the_stored_blocks_widened(model):
    made, _, ids, g = model
    m = made(8)
    for p in (0, 7, 39):
        assert np.array_equal(m.embed(ids[p]), g["embedded"][p])     # bit for bit what the oracle's replay embedded


def test_a_session_has_the_reference_buffers_and_rings(model):
    made, _, _, _ = model
    m = made(8, 100)
    assert m.max_context == 128
    s = m.session()
    c = m.config
    assert len(s.sets[0]) == len(s.sets[1]) == CACHES and len(s.caches) == 2 * c.layers
    # sliding layers: window + chunk rounded up to 32 rows; full layers: the capacity
    assert s.slots == [32, 128, 32, 128] and s.capacity() == 128 and s.rewind == 8
    assert m.session_holding(40).slots == [32, 64, 32, 64]
    assert m.session_holding(4000).capacity() == 128
    n, kw = 32, c.kv_heads * c.head_dim
    assigned = n * c.experts_used + 32 * c.experts
    sizes = [b.data.size for b in s.sets[0]]
    assert sizes[:8] == [n * c.hidden, n * c.hidden, n * c.heads * c.head_dim, n * kw, n * kw, n * c.heads * c.head_dim,
                         n * c.hidden, n * c.head_dim]
    assert sizes[8:13] == [assigned * c.hidden] + [assigned * c.expert_hidden] * 3 + [assigned * c.hidden]
    assert sizes[13:] == [32 * c.vocab, 4, 4, 4]
    assert [b.data.size for b in s.caches[:4]] == [32 * kw, 32 * kw, 128 * kw, 128 * kw]
    with pytest.raises(Invalid, match="positive"):
        made(0)


def test_truncate_and_reset_follow_the_reference_rules(model):
    made, _, ids, _ = model
    m = made(8)
    s = m.session()
    assert s.is_empty() and len(m.feed(s, ids[:30], LAST)) == 1 and len(s) == 30
    with pytest.raises(Invalid, match="cannot go back from position 30 to 12"):
        s.truncate(12)
    with pytest.raises(Invalid):
        s.truncate(31)
    s.truncate(22)
    assert len(s) == 22
    assert len(m.feed(s, ids[22:27], ALL)) == 5 and len(s) == 27
    s.reset()
    assert s.is_empty()
    with pytest.raises(Invalid, match="65 positions exceed the session's 64"):
        m.feed(s, [1] * 65, LAST)
    assert s.is_empty()


def phases(gpu):
    """The committed or run batches, each as (what it is, its first dispatch's row count)."""
    out = []
    for kind, batch in gpu.log:
        if kind == "done":
            continue
        names = [name for name, _ in batch.calls]
        if "moe_combine" in names:
            what = "token"
        elif "rotate_halves" in names:
            what = "attention"
        elif "clamped_swiglu" in names:
            what = "experts"
        else:
            what = "output"
        out.append(what)
    return out


def test_feed_splits_into_passes_and_returns_the_logits_asked_for(model):
    made, gpu, ids, _ = model
    m = made(16)
    m.pipeline = False
    s = m.session()
    assert len(m.feed(s, ids[:40], ALL)) == 40
    # 16 + 16 + 8 positions: per pass 4 x (attention, experts), then one output submission each
    assert phases(gpu) == (["attention", "experts"] * 4 + ["output"]) * 3
    assert m.submissions == {"attention": 12, "experts": 12, "output": 3, "token": 0}
    del gpu.log[:]
    s.reset()
    assert len(m.feed(s, ids[:40], LAST)) == 1
    assert phases(gpu) == ["attention", "experts"] * 8 + (["attention", "experts"] * 4 + ["output"])   # only the last pass's
    del gpu.log[:]
    assert len(m.feed(s, ids[:3], LAST)) == 1 and len(s) == 43
    assert phases(gpu) == ["attention", "experts"] * 4 + ["output"]
    del gpu.log[:]
    assert len(m.feed(s, [ids[3]], LAST)) == 1                # decoding: one submission with everything in it
    assert phases(gpu) == ["token"]
    m.gpu_routing = False
    del gpu.log[:]
    assert len(m.feed(s, [ids[4]], LAST)) == 1                # routed on the CPU: as a prompt pass of one
    assert phases(gpu) == ["attention", "experts"] * 4 + ["output"]


@pytest.mark.parametrize("chunk, which", [(8, ALL), (16, ALL), (16, LAST), (32, ALL), (5, LAST)])
def test_two_passes_interleave_layer_by_layer(model, chunk, which):
    made, gpu, ids, _ = model
    m = made(chunk)
    s = m.session()
    logits = m.feed(s, ids[:40], which)
    assert len(logits) == (40 if which == ALL else 1) and len(s) == 40
    parts = -(-40 // chunk)
    per_pass_outputs = lambda n: -(-n // 32) if which == ALL else 0
    sizes = [min(chunk, 40 - i * chunk) for i in range(parts)]
    outputs = sum(per_pass_outputs(n) for n in sizes) if which == ALL else 1
    layers = m.config.layers
    assert m.submissions == {"attention": parts * layers, "experts": parts * layers, "output": outputs, "token": 0}
    # attention batches take the caches in order: first pass, second pass, layer by layer
    order = []
    for kind, batch in gpu.log:
        if kind != "done" and any(name == "rotate_halves" for name, _ in batch.calls):
            shape = next(args for name, args in batch.calls if name.startswith("attention_grouped"))[-1]
            order.append((shape.start, shape.t))
    starts = [sum(sizes[:i]) for i in range(parts)]
    want = []
    for pair in range(0, parts - 1, 2):
        for _ in range(layers):
            want += [(starts[pair], sizes[pair]), (starts[pair + 1], sizes[pair + 1])]
    if parts % 2:
        want += [(starts[-1], sizes[-1])] * layers
    assert order == want
    # while a pair was in flight two batches were outstanding at some point: the passes overlapped
    if parts >= 2:
        outstanding, most = 0, 0
        for kind, _ in gpu.log:
            outstanding += {"commit": 1, "done": -1, "run": 0}[kind]
            most = max(most, outstanding)
        assert most == 2
    # every buffer came back
    assert all(b.owner is None for b in s.sets[0] + s.sets[1] + s.caches)
    assert len(s.sets[0]) == len(s.sets[1]) == CACHES and len(s.caches) == 2 * layers


def test_a_failed_batch_is_reported_after_every_buffer_came_back(model):
    made, gpu, ids, _ = model
    m = made(8)
    s = m.session()
    real = FakeBatch._finish
    count = {"n": 0}

    def sometimes_fails(self):
        done = real(self)
        count["n"] += 1
        if count["n"] == 5:
            return Completed(done.buffers, RuntimeError("the GPU reported an error"))
        return done

    FakeBatch._finish = sometimes_fails
    try:
        with pytest.raises(RuntimeError, match="reported an error"):
            m.feed(s, ids[:16], ALL)
    finally:
        FakeBatch._finish = real
    assert len(s) == 0, "a failed pair does not advance the session"
    assert all(b.owner is None for b in s.sets[0] + s.sets[1] + s.caches)


def test_host_repacking_is_the_oracles(model):
    """The two repackings done while loading (Q8_0 blocks split into codes and scales,
    weights/src/q8_0.rs:17-31; MXFP4 blocks from ggml's nibble order to pairs,
    weights/src/mxfp4.rs:119-149) against the oracle's restatements, on the fixture's tensors."""
    from loadngo_b200.gpt_oss import ggml_to_ocp, split_q8_0
    from oracle import oracle
    _, _, _, g = model
    blocks = np.ascontiguousarray(g["l1_attn_q_q8_0"])
    n = blocks.size // 34
    codes, scales = np.zeros(n * 32, np.uint8), np.zeros(n * 2, np.uint8)
    oracle.lib().oracle_q8_0_split(blocks, n, codes, scales)
    mine = split_q8_0(blocks)
    assert np.array_equal(mine[0], codes) and np.array_equal(mine[1], scales)
    mx = np.ascontiguousarray(g["l2_ffn_down_exps_mxfp4"])
    want = oracle.mxfp4_ggml_to_ocp(mx)
    got = ggml_to_ocp(mx)
    assert np.array_equal(got[0], want[0]) and np.array_equal(got[1], want[1])


def test_cpu_routing_of_a_prompt_pass_is_the_oracles_and_gathers_rows_by_expert(model):
    """`route_and_gather` (gpt-oss/src/gpu.rs:1187-1227) on the fixture's inputs of layer 1's experts:
    the experts and weights of every position are the oracle's router's (ties to the lower index,
    softmax over the chosen ones), and the gathered buffer holds each expert's rows together, an
    expert with 32 rows or more padded to a multiple of 32."""
    from loadngo_b200.gpt_oss import X, XE
    from oracle import oracle
    made, _, _, g = model
    m = made(40)
    s = m.session()
    c, layer, n = m.config, 1, 40
    x = np.ascontiguousarray(g["l1_x_ffn"][:n], np.float32)
    s.sets[0][X].write(x)
    by_expert, runs = m.route_and_gather(s.sets[0], layer, n)
    w, bias = g["l1_router"].reshape(c.experts, c.hidden), g["l1_router_bias"]
    chosen = {}
    for e, rows in enumerate(by_expert):
        for p, weight in rows:
            chosen.setdefault(p, []).append((e, weight))
    for p in range(n):
        logits = np.ascontiguousarray((x[p] @ w.T + bias).astype(np.float32))
        ids, weights = np.zeros(c.experts_used, np.int32), np.zeros(c.experts_used, np.float32)
        oracle.lib().oracle_route(logits, c.experts, c.experts_used, ids, weights)
        got = dict(chosen[p])
        assert sorted(got) == sorted(int(i) for i in ids)
        for i, wt in zip(ids, weights):
            assert abs(got[int(i)] - wt) <= 1e-6
        assert abs(sum(got.values()) - 1.0) <= 1e-6
    # rows of an expert lie together, in position order, runs of 32 or more padded to 32
    gathered = s.sets[0][XE].as_f32()
    at = 0
    for e, first, count in runs:
        assert first == at and count == len(by_expert[e])
        for i, (p, _) in enumerate(by_expert[e]):
            assert np.array_equal(gathered[(first + i) * c.hidden:(first + i + 1) * c.hidden], x[p])
        at += -(-count // 32) * 32 if count >= 32 else count
    assert sum(count for _, _, count in runs) == n * c.experts_used
    # a tie goes to the expert with the lower index
    logits = np.array([1.0, 3.0, 3.0, 0.5], np.float32)
    ids, weights = np.zeros(2, np.int32), np.zeros(2, np.float32)
    oracle.lib().oracle_route(logits, 4, 2, ids, weights)
    assert list(ids) == [1, 2] and weights[0] == weights[1] == 0.5
