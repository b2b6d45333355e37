"""The float32 entry points with metal-compute's own shapes and semantics, checked the way the
reference checks its kernels: against the float64 definition written in its tests
(metal-compute/tests/attention_grouped.rs, q8_0_and_gpt_oss_glue.rs), with the same
deterministic inputs, ring layouts (NaN in rows the plain kernel must never read), shape lists
and tolerances; then the reference's tiny end-to-end fixture replayed through the call sequence
of `GpuModel::encode_attention` (gpt-oss/src/gpu.rs:741-806)."""
import json
import os

import numpy as np
import pytest

from loadngo_b200 import compute
from loadngo_b200.compute import FULL, GroupedShape, Slice
from oracle import oracle
from tests.helpers import xorshift_values as values

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "tiny_attention.npz")


def shape(t, start, heads, kv_heads, dim, window, slots, scale=1.0):
    return GroupedShape(t, start, heads, kv_heads, dim, window, slots, scale)


def ring(all_rows, s: GroupedShape, tiled: bool):
    """attention_grouped.rs:47-63: the newest `slots` positions laid into their ring rows; rows
    the tiled kernel reads past the end are zero, rows the plain kernel must not read are NaN."""
    row = s.kv_heads * s.dim
    end = s.start + s.t
    if not tiled:
        rows = min(s.slots, end)
    elif s.slots < end:
        rows = s.slots
    else:
        rows = -(-end // 32) * 32
    out = np.full((rows, row), 0.0 if tiled else np.nan, np.float32)
    for p in range(max(0, end - s.slots), end):
        out[p % s.slots] = all_rows[p]
    return out


def max_error(gpu, s: GroupedShape, sharp, tiled, sinks=None):
    end = s.start + s.t
    rows = -(-s.t // 32) * 32 if tiled else s.t
    q = values(1, s.t * s.heads * s.dim) * np.float32(sharp)
    want_q = q.reshape(s.t, s.heads, s.dim)
    q = np.concatenate([q, np.zeros((rows - s.t) * s.heads * s.dim, np.float32)])
    k = values(2, end * s.kv_heads * s.dim).reshape(end, s.kv_heads * s.dim)
    v = values(3, end * s.kv_heads * s.dim).reshape(end, s.kv_heads * s.dim)
    kr, vr = ring(k, s, tiled), ring(v, s, tiled)
    out_len = rows * s.heads * s.dim * 4
    buffers = [gpu.upload(q), gpu.upload(kr), gpu.upload(vr), gpu.buffer(out_len),
               gpu.upload(sinks if sinks is not None else np.zeros(1, np.float32))]
    batch = gpu.batch(buffers)
    qs, ks, vs, os_ = Slice(0, 0, q.nbytes), Slice(1, 0, kr.nbytes), Slice(2, 0, vr.nbytes), Slice(3, 0, out_len)
    sink_slice = Slice(4, 0, s.heads * 4)
    if tiled and sinks is None:
        batch.attention_grouped_tiled(qs, ks, vs, os_, s)
    elif tiled:
        batch.attention_grouped_tiled_with_sinks((qs, ks, vs), sink_slice, os_, s)
    elif sinks is None:
        batch.attention_grouped(qs, ks, vs, os_, s)
    else:
        batch.attention_grouped_with_sinks((qs, ks, vs), sink_slice, os_, s)
    done = batch.run()
    assert not isinstance(done.gpu_time, Exception), done.gpu_time
    window = 0 if s.window >= FULL else s.window
    want = oracle.attention_f64(want_q, k.reshape(end, s.kv_heads, s.dim), v.reshape(end, s.kv_heads, s.dim),
                                start=s.start, window=window, scale=s.scale, sinks=sinks)
    got = done.buffers[3].as_f32()[: want.size].reshape(want.shape).copy()   # the view dies with the buffer
    for b in buffers:
        b.free()
    if np.isnan(got).any():
        return float("inf")
    return float(np.abs(got - want).max())


def test_matches_the_float64_definition(gpu):
    # attention_grouped.rs:181-203 (tolerance 2e-5)
    for s, sharp in [
        (shape(1, 0, 32, 4, 512, FULL, 1), 1.0),
        (shape(1, 700, 32, 4, 512, FULL, 701), 0.05),
        (shape(37, 300, 32, 4, 512, FULL, 337), 0.05),
        (shape(1, 3000, 32, 16, 256, 1024, 1536), 0.08),
        (shape(200, 1400, 32, 16, 256, 1024, 1536), 0.08),
        (shape(512, 0, 32, 16, 256, 1024, 1536), 0.08),
        (shape(5, 97, 4, 1, 64, 7, 12), 3.0),
        (shape(3, 2, 8, 2, 32, 16, 40), 1.0),
    ]:
        error = max_error(gpu, s, sharp, False)
        assert error < 2e-5, f"{s} sharp {sharp}: max error {error}"


def test_tiled_matches_the_float64_definition(gpu):
    # attention_grouped.rs:206-226 (tolerance 1e-4)
    for s, sharp in [
        (shape(512, 0, 32, 4, 512, FULL, 512), 0.05),
        (shape(77, 700, 32, 4, 512, FULL, 4096), 0.05),
        (shape(33, 5, 32, 4, 512, FULL, 40), 0.05),
        (shape(512, 2600, 32, 16, 256, 1024, 1536), 0.08),
        (shape(200, 1400, 32, 16, 256, 1024, 1536), 0.08),
        (shape(512, 0, 32, 16, 256, 1024, 1536), 0.08),
        (shape(40, 97, 4, 1, 64, 7, 64), 3.0),
    ]:
        error = max_error(gpu, s, sharp, True)
        assert error < 1e-4, f"{s} sharp {sharp}: max error {error}"


def test_sinks_take_probability_without_value_on_gpt_oss_shapes(gpu):
    # attention_grouped.rs:229-253: 64 heads over 8, 64 wide, scale 1/8, sinks from -3 to 3
    sinks = values(4, 64) * np.float32(3.0)
    g = lambda t, start, window, slots: shape(t, start, 64, 8, 64, window, slots, 0.125)
    for s, tiled in [
        (g(1, 0, 128, 640), False),
        (g(1, 3000, 128, 640), False),
        (g(9, 700, 128, 640), False),
        (g(512, 0, 128, 640), True),
        (g(512, 2600, 128, 640), True),
        (g(1, 4095, FULL, 4096), False),
        (g(300, 200, FULL, 4096), True),
    ]:
        error = max_error(gpu, s, 1.0, tiled, sinks)
        assert error < 1e-4, f"{s} tiled {tiled}: max error {error}"


def test_rejects_shapes_it_cannot_run(gpu):
    # attention_grouped.rs:255-275
    for s in [
        shape(1, 0, 6, 4, 64, 8, 8),     # heads not a multiple of KV heads
        shape(1, 0, 4, 4, 48, 8, 8),     # dim not a multiple of 32
        shape(1, 0, 4, 4, 544, 8, 8),    # dim over 512
        shape(4, 100, 4, 4, 64, 8, 10),  # ring smaller than window + t
        shape(0, 0, 4, 4, 64, 8, 8),     # nothing to do
    ]:
        buffers = [gpu.buffer(1 << 20) for _ in range(4)]
        batch = gpu.batch(buffers)
        sl = lambda b: Slice(b, 0, 1 << 20)
        with pytest.raises(compute.DispatchError):
            batch.attention_grouped(sl(0), sl(1), sl(2), sl(3), s)
        batch.drop()
        for b in buffers:
            b.free()


def test_glue_rotates_adds_copies_and_norms_as_defined(gpu):
    # q8_0_and_gpt_oss_glue.rs:190-297
    rows, heads, dim, width = 3, 4, 64, 96
    x = values(1, rows * heads * dim)
    bias = values(2, width)
    h = values(3, rows * width)
    i = np.arange(rows * dim // 2, dtype=np.float64) * 0.37
    table = np.stack([np.cos(i).astype(np.float32) * np.float32(1.3), np.sin(i).astype(np.float32) * np.float32(1.3)],
                     axis=1).reshape(-1)
    wide = values(8, rows * 160)          # rows 160 apart, only 96 columns touched
    weight = values(9, width)
    buffers = [gpu.upload(x), gpu.upload(table), gpu.upload(h), gpu.upload(bias), gpu.upload(wide),
               gpu.upload(weight), gpu.buffer(rows * 160 * 4)]
    gpu_copy = buffers[6]
    gpu_copy.write(np.full(rows * 160, 7.0, np.float32))
    batch = gpu.batch(buffers)
    f = lambda b, n, off=0: Slice(b, off * 4, n * 4)
    batch.rotate_halves(f(0, x.size), f(1, table.size), rows, (heads, dim))
    batch.add_rows(f(2, h.size), (f(3, width), 0), rows, width)
    batch.copy_rows((f(4, (rows - 1) * 160 + width), 160), (f(6, (rows - 1) * 160 + width), 160), rows, width)
    batch.rmsnorm_rows((f(4, (rows - 1) * 160 + width), f(5, width)), rows, (width, 160), 1e-5)
    done = batch.run()
    assert not isinstance(done.gpu_time, Exception), done.gpu_time
    half = dim // 2
    rotated = buffers[0].as_f32()[: x.size].reshape(rows, heads, dim)
    xs = x.reshape(rows, heads, dim).astype(np.float64)
    t64 = table.reshape(rows, half, 2).astype(np.float64)
    for r in range(rows):
        c, s = t64[r, :, 0], t64[r, :, 1]
        for hd in range(heads):
            a, b = xs[r, hd, :half], xs[r, hd, half:]
            assert np.abs(rotated[r, hd, :half] - (a * c - b * s)).max() < 1e-6
            assert np.abs(rotated[r, hd, half:] - (b * c + a * s)).max() < 1e-6
    added = buffers[2].as_f32()[: rows * width]
    assert np.array_equal(added, h + np.tile(bias, rows))
    copied = buffers[6].as_f32()[: rows * 160].reshape(rows, 160)
    src = wide.reshape(rows, 160)
    assert np.array_equal(copied[:, :width], src[:, :width])
    assert np.all(copied[:, width:] == 7.0)              # nothing outside its columns
    normed = buffers[4].as_f32()[: rows * 160].reshape(rows, 160)
    for r in range(rows):
        v64 = src[r, :width].astype(np.float64)
        want = v64 / np.sqrt(np.mean(v64 ** 2) + 1e-5) * weight.astype(np.float64)
        assert np.abs(normed[r, :width] - want).max() < 1e-5
    assert np.array_equal(normed[:, width:], src[:, width:])
    for b in buffers:
        b.free()


def test_output_must_not_alias_inputs_or_residents(gpu):
    buffers = [gpu.buffer(4096), gpu.buffer(4096)]
    res = gpu.resident(np.zeros(1024, np.float32))
    batch = gpu.batch(buffers)
    rs = batch.attach(res)
    with pytest.raises(compute.DispatchError):     # output overlapping its input
        batch.copy_rows((Slice(0, 0, 1024), 256), (Slice(0, 512, 1024), 256), 1, 256)
    with pytest.raises(compute.DispatchError):     # writing into resident memory
        batch.copy_rows((Slice(0, 0, 1024), 256), (Slice(rs.buffer, 0, 1024), 256), 1, 256)
    with pytest.raises(compute.DispatchError):     # a slice shorter than the shape needs
        batch.copy_rows((Slice(0, 0, 1000), 256), (Slice(1, 0, 1024), 256), 1, 256)
    with pytest.raises(compute.DispatchError):     # misaligned offset
        batch.copy_rows((Slice(0, 2, 1024), 256), (Slice(1, 0, 1024), 256), 1, 256)
    batch.copy_rows((Slice(rs.buffer, 0, 1024), 256), (Slice(1, 0, 1024), 256), 1, 256)   # reading one is fine
    assert batch.dispatches == 1
    assert buffers[0].as_bytes is not None
    done = batch.run()
    assert not isinstance(done.gpu_time, Exception)
    res.free()
    for b in buffers:
        b.free()


def test_completion_callback_hands_buffers_back(gpu):
    import threading
    a = gpu.upload(np.arange(256, dtype=np.float32))
    b = gpu.buffer(1024)
    batch = gpu.batch([a, b])
    batch.copy_rows((Slice(0, 0, 1024), 256), (Slice(1, 0, 1024), 256), 1, 256)
    box, event = {}, threading.Event()

    def done(completed):
        box["done"] = completed
        event.set()

    batch.commit(done)                      # returns at once; the callback runs on the completion thread
    assert event.wait(30)
    assert isinstance(box["done"].gpu_time, float) and box["done"].gpu_time >= 0
    assert np.array_equal(box["done"].buffers[1].as_f32()[:256], np.arange(256, dtype=np.float32))
    a.free(); b.free()


@pytest.mark.parametrize("chunks", [[1] * 40, [8] * 5, [33, 7]])
def test_tiny_fixture_through_the_reference_call_sequence(gpu, chunks):
    """The attention of the reference's tiny end-to-end fixture (4 query heads over 2 KV heads of
    32, window 8 on even layers), fed as gpt-oss/tests/gpu_oracle.rs:76-145 feeds it: one
    position at a time through a wrapping ring, in chunks of 8, and as 33 + 7; each pass issues
    what encode_attention issues: rotate_halves on Q and K, copy_rows into the ring in at most
    two runs, then grouped attention with sinks (the tiled entry from 32 positions)."""
    g = np.load(GOLDEN)
    meta = json.loads(str(g["meta"]))
    heads, kv_heads, dim, positions = meta["heads"], meta["kv_heads"], meta["dim"], meta["positions"]
    qw, kw = heads * dim, kv_heads * dim
    rope = dict(head_dim=dim, theta=meta["theta"], factor=meta["factor"],
                original_context=float(meta["original_context"]))
    chunk = max(chunks)
    pad = -(-chunk // 32) * 32
    for l in range(meta["layers"]):
        sliding = l % 2 == 0
        window = meta["window"] if sliding else FULL
        slots = -(-(meta["window"] + chunk) // 32) * 32 if sliding else -(-positions // 32) * 32
        Q, K, V, ATT, TABLE, KC, VC, SINKS = range(8)
        buffers = [gpu.buffer(pad * qw * 4), gpu.buffer(pad * kw * 4), gpu.buffer(pad * kw * 4),
                   gpu.buffer(pad * qw * 4), gpu.buffer(pad * dim * 4), gpu.buffer(slots * kw * 4),
                   gpu.buffer(slots * kw * 4), gpu.upload(g[f"l{l}_sinks"])]
        for b in (buffers[KC], buffers[VC], buffers[Q], buffers[ATT]):
            b.zero()
        start, worst = 0, 0.0
        for n in chunks:
            buffers[Q].write(g[f"l{l}_q"][start:start + n])
            buffers[K].write(g[f"l{l}_k"][start:start + n])
            buffers[V].write(g[f"l{l}_v"][start:start + n])
            buffers[TABLE].write(compute.rope_table(start, n, **rope))
            batch = gpu.batch(buffers)
            f = lambda b, row, w, rows: Slice(b, row * w * 4, rows * w * 4)
            table = f(TABLE, 0, dim, n)
            batch.rotate_halves(f(Q, 0, qw, n), table, n, (heads, dim))
            batch.rotate_halves(f(K, 0, kw, n), table, n, (kv_heads, dim))
            done_rows = 0
            while done_rows < n:                      # gpu.rs:744-759
                row = (start + done_rows) % slots
                run = min(n - done_rows, slots - row)
                for src, dst in ((K, KC), (V, VC)):
                    batch.copy_rows((f(src, done_rows, kw, run), kw), (f(dst, row, kw, run), kw), run, kw)
                done_rows += run
            s = GroupedShape(n, start, heads, kv_heads, dim, window, slots, 1.0 / float(np.sqrt(np.float32(dim))))
            sinks = Slice(SINKS, 0, heads * 4)
            if n >= 32:
                padded = -(-n // 32) * 32
                end = start + n
                rows = slots if slots < end else -(-end // 32) * 32
                batch.attention_grouped_tiled_with_sinks((f(Q, 0, qw, padded), f(KC, 0, kw, rows), f(VC, 0, kw, rows)),
                                                         sinks, f(ATT, 0, qw, padded), s)
            else:
                rows = min(slots, start + n)
                batch.attention_grouped_with_sinks((f(Q, 0, qw, n), f(KC, 0, kw, rows), f(VC, 0, kw, rows)), sinks,
                                                   f(ATT, 0, qw, n), s)
            done = batch.run()
            assert not isinstance(done.gpu_time, Exception), done.gpu_time
            got = buffers[ATT].as_f32()[: n * qw].reshape(n, heads, dim)
            worst = max(worst, float(np.abs(got - g[f"l{l}_out"][start:start + n]).max()))
            start += n
        assert worst < 1e-4, f"layer {l}: worst attention error {worst}"
        for b in buffers:
            b.free()


BLOCK_GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "tiny_block.npz")


def _split_q8_0(blocks: np.ndarray):
    """`split_blocks` (weights/src/q8_0.rs:17-31) through the oracle."""
    n = blocks.size // 34
    codes, scales = np.zeros(n * 32, np.uint8), np.zeros(n * 2, np.uint8)
    oracle.lib().oracle_q8_0_split(np.ascontiguousarray(blocks), n, codes, scales)
    return codes, scales


@pytest.mark.parametrize("chunks", [[1] * 40, [8] * 5, [33, 7]])
def test_tiny_fixture_whole_encode_attention_with_the_stored_q8_0_weights(gpu, chunks):
    """Everything `GpuModel::encode_attention` records (gpt-oss/src/gpu.rs:703-827), call for call,
    on the tiny fixture's own weights as the GGUF stores them (Q8_0 projections with biases):
    copy H to X, RMSNorm, the three projections (gemv for one position, the plain product below
    32, the tiled one on n rounded up to 32 from there), biases, rotary, the ring append,
    grouped attention with sinks, output projection, bias, residual add, and the copy + norm that
    leaves the experts' input in X.  The residual stream going in is the golden one of each
    layer (the experts between the layers are not part of this path); H and X coming out are
    compared with the golden vectors made by the pinned oracle replay."""
    g = np.load(BLOCK_GOLDEN)
    meta = json.loads(str(g["meta"]))
    hidden, heads, kv_heads, dim, positions = (meta[k] for k in ("hidden", "heads", "kv_heads", "dim", "positions"))
    qw, kw, eps = heads * dim, kv_heads * dim, meta["eps"]
    rope = dict(head_dim=dim, theta=meta["theta"], factor=meta["factor"], original_context=float(meta["original_context"]))
    chunk = max(chunks)
    pad = -(-chunk // 32) * 32
    f = lambda b, row, w, rows: Slice(b, row * w * 4, rows * w * 4)
    for l in range(meta["layers"]):
        sliding = l % 2 == 0
        window = meta["window"] if sliding else FULL
        slots = -(-(meta["window"] + chunk) // 32) * 32 if sliding else -(-positions // 32) * 32
        H, X, Q, K, V, ATT, TMP, TABLE, KC, VC = range(10)
        buffers = [gpu.buffer(pad * w * 4) for w in (hidden, hidden, qw, kw, kw, qw, hidden, dim)]
        buffers += [gpu.buffer(slots * kw * 4), gpu.buffer(slots * kw * 4)]
        for b in buffers:
            b.zero()
        # the layer's weights as residents, as `GpuModel::load` keeps them
        res = {}
        for name in ("attn_q", "attn_k", "attn_v", "attn_output"):
            codes, scales = _split_q8_0(g[f"l{l}_{name}_q8_0"])
            res[name] = (gpu.resident(codes), gpu.resident(scales), gpu.resident(g[f"l{l}_{name}_bias"]))
        res["attn_norm"], res["ffn_norm"] = gpu.resident(g[f"l{l}_attn_norm"]), gpu.resident(g[f"l{l}_ffn_norm"])
        res["sinks"] = gpu.resident(g[f"l{l}_sinks"])

        def mul(batch, name, rows, cols, x, y, n):           # Q8::mul, gpu.rs:121-137
            tiled = n >= 32
            n_run = -(-n // 32) * 32 if tiled else n
            x, y = Slice(x.buffer, x.offset, n_run * cols * 4), Slice(y.buffer, y.offset, n_run * rows * 4)
            m = (batch.attach(res[name][0]), batch.attach(res[name][1]))
            if n == 1:
                batch.gemv_q8_0(m, x, y, rows, cols)
            elif tiled:
                batch.gemm_q8_0_tiled(m, x, y, rows, cols, n_run, (cols, rows))
            else:
                batch.gemm_q8_0(m, x, y, rows, cols, n, (cols, rows))

        start, worst_h, worst_x = 0, 0.0, 0.0
        for n in chunks:
            buffers[H].write(g[f"l{l}_h_in"][start:start + n])
            buffers[TABLE].write(compute.rope_table(start, n, **rope))
            batch = gpu.batch(buffers)
            rows_of = lambda b, w: f(b, 0, w, n)
            batch.copy_rows((rows_of(H, hidden), hidden), (rows_of(X, hidden), hidden), n, hidden)
            batch.rmsnorm_rows((rows_of(X, hidden), batch.attach(res["attn_norm"])), n, (hidden, hidden), eps)
            mul(batch, "attn_q", qw, hidden, rows_of(X, hidden), rows_of(Q, qw), n)
            mul(batch, "attn_k", kw, hidden, rows_of(X, hidden), rows_of(K, kw), n)
            mul(batch, "attn_v", kw, hidden, rows_of(X, hidden), rows_of(V, kw), n)
            for buf, name, width in ((Q, "attn_q", qw), (K, "attn_k", kw), (V, "attn_v", kw)):
                batch.add_rows(rows_of(buf, width), (batch.attach(res[name][2]), 0), n, width)
            table = rows_of(TABLE, dim)
            batch.rotate_halves(rows_of(Q, qw), table, n, (heads, dim))
            batch.rotate_halves(rows_of(K, kw), table, n, (kv_heads, dim))
            done_rows = 0
            while done_rows < n:
                row = (start + done_rows) % slots
                run = min(n - done_rows, slots - row)
                for src, dst in ((K, KC), (V, VC)):
                    batch.copy_rows((f(src, done_rows, kw, run), kw), (f(dst, row, kw, run), kw), run, kw)
                done_rows += run
            s = GroupedShape(n, start, heads, kv_heads, dim, window, slots, 1.0 / float(np.sqrt(np.float32(dim))))
            sinks = batch.attach(res["sinks"])
            if n >= 32:
                padded, end = -(-n // 32) * 32, start + n
                rows = slots if slots < end else -(-end // 32) * 32
                batch.attention_grouped_tiled_with_sinks((f(Q, 0, qw, padded), f(KC, 0, kw, rows), f(VC, 0, kw, rows)),
                                                         sinks, f(ATT, 0, qw, padded), s)
            else:
                rows = min(slots, start + n)
                batch.attention_grouped_with_sinks((rows_of(Q, qw), f(KC, 0, kw, rows), f(VC, 0, kw, rows)), sinks,
                                                   rows_of(ATT, qw), s)
            mul(batch, "attn_output", hidden, qw, rows_of(ATT, qw), rows_of(TMP, hidden), n)
            batch.add_rows(rows_of(TMP, hidden), (batch.attach(res["attn_output"][2]), 0), n, hidden)
            batch.add_rows(rows_of(H, hidden), (rows_of(TMP, hidden), hidden), n, hidden)
            batch.copy_rows((rows_of(H, hidden), hidden), (rows_of(X, hidden), hidden), n, hidden)
            batch.rmsnorm_rows((rows_of(X, hidden), batch.attach(res["ffn_norm"])), n, (hidden, hidden), eps)
            done = batch.run()
            assert not isinstance(done.gpu_time, Exception), done.gpu_time
            got_h = buffers[H].as_f32()[: n * hidden].reshape(n, hidden)
            got_x = buffers[X].as_f32()[: n * hidden].reshape(n, hidden)
            worst_h = max(worst_h, float(np.abs(got_h - g[f"l{l}_h_att"][start:start + n]).max()))
            worst_x = max(worst_x, float(np.abs(got_x - g[f"l{l}_x_ffn"][start:start + n]).max()))
            start += n
        assert worst_h < 2e-4 and worst_x < 2e-4, f"layer {l}: residual {worst_h}, experts' input {worst_x}"
        for b in buffers:
            b.free()
        for v in res.values():
            for r in (v if isinstance(v, tuple) else (v,)):
                r.free()


def test_host_ranges_of_any_size_and_offset_reach_the_device_and_come_back(gpu):
    """A buffer's two copies stay in step however the host writes it: whole, a few bytes at an odd
    offset (the range is rounded out to 16 bytes for the copy kernel; the bytes around it must
    survive), next to a range the device wrote in the meantime, and as a range large enough to go
    through the copy engine instead.  Read back lazily and with an explicit read-back."""
    rng = np.random.default_rng(4)
    n = 1000                                           # not a multiple of 16: the tail is padding
    a, b = gpu.buffer(n), gpu.buffer(n)
    want = rng.integers(0, 256, n, dtype=np.uint8)
    a.write(want)

    def copy(src, dst, read_back=False):               # dst <- src on the device (250 floats)
        batch = gpu.batch([src, dst])
        batch.copy_rows((Slice(0, 0, n), 250), (Slice(1, 0, n), 250), 1, 250)
        if read_back:
            batch.read_back(Slice(1, 0, n))
        assert not isinstance(batch.run().gpu_time, Exception)

    copy(a, b)
    assert np.array_equal(b.as_bytes()[:n], want)
    # six bytes at an odd offset
    patch = np.array([1, 2, 3, 4, 5, 6], np.uint8)
    a.write(patch, offset=35)
    want[35:41] = patch
    copy(a, b, read_back=True)
    assert np.array_equal(b.as_bytes()[:n], want)
    # the device writes a range of `a` (rows 4..7 of b's floats), then the host writes beside it
    batch = gpu.batch([b, a])
    batch.copy_rows((Slice(0, 400, 64), 16), (Slice(1, 64, 64), 16), 1, 16)
    assert not isinstance(batch.run().gpu_time, Exception)
    want[64:128] = want[400:464]
    a.write(np.array([9, 8, 7], np.uint8), offset=129)
    want[129:132] = [9, 8, 7]
    a.write(np.array([42], np.uint8), offset=n - 1)    # the last byte before the padding
    want[n - 1] = 42
    copy(a, b)
    assert np.array_equal(b.as_bytes()[:n], want)
    assert np.array_equal(a.as_bytes()[:n], want)
    # a range above the copy kernel's limit takes the copy engine
    big_n = (3 << 20) + 8
    big, back = gpu.buffer(big_n), gpu.buffer(big_n)
    data = rng.integers(0, 256, big_n, dtype=np.uint8)
    big.write(data)
    batch = gpu.batch([big, back])
    batch.copy_rows((Slice(0, 0, big_n), big_n // 4), (Slice(1, 0, big_n), big_n // 4), 1, big_n // 4)
    batch.read_back(Slice(1, 0, big_n))
    assert not isinstance(batch.run().gpu_time, Exception)
    assert np.array_equal(back.as_bytes()[:big_n], data)
    for buf in (a, b, big, back):
        buf.free()
