"""The GGUF reader (host code of libcuda_compute.so) against files written by the tests' own
writer, in the cases the reference's reader is tested on (weights/src/gguf.rs:493-571), and
against the reference's tiny model file where the reference checkout is present."""
import os
import struct

import numpy as np
import pytest

from loadngo_b200 import gguf

from tests import gguf_writer as w

# a loadngo checkout named by LOADNGO_REFERENCE, or lying beside this repository
REFERENCE = os.environ.get("LOADNGO_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(
    os.path.abspath(__file__)))), "reference")
TINY = os.path.join(REFERENCE, "gpt-oss", "tests", "fixtures", "tiny", "model.gguf")


def sample() -> bytes:
    return w.file(
        [("general.architecture", w.STRING, "gpt-oss"),
         ("gpt-oss.block_count", w.U32, 24),
         ("gpt-oss.rope.freq_base", w.F32, 150000.0),
         ("tokenizer.ggml.merges", w.ARRAY, (w.STRING, ["a b", "é"]))],
        [("norm", [3], gguf.F32, np.array([1.0, 2.0, 3.0], np.float32)),
         ("q", [32, 2], gguf.Q8_0, bytes(range(68))),
         ("odd", [5], 2, bytes([9] * 18))])


def test_metadata_and_tensors_parse_with_absolute_aligned_offsets():
    raw = sample()
    g = gguf.Gguf.parse(raw, len(raw))
    assert g.version == 3 and g.alignment == 32
    assert g.get("general.architecture") == "gpt-oss"
    assert g.get("gpt-oss.block_count") == 24
    assert g.get("gpt-oss.rope.freq_base") == 150000.0
    assert g.get("tokenizer.ggml.merges") == ["a b", "é"]
    assert g.get("absent") is None
    assert g.keys() == sorted(["general.architecture", "gpt-oss.block_count", "gpt-oss.rope.freq_base",
                               "tokenizer.ggml.merges"])
    assert g.data_offset % 32 == 0
    norm = g.tensor("norm")
    assert (norm.ggml_type, norm.len, norm.dims) == (gguf.F32, 12, [3])
    assert raw[norm.offset:norm.offset + 4] == struct.pack("<f", 1.0)
    q = g.tensor("q")
    assert (q.ggml_type, q.len, q.numel()) == (gguf.Q8_0, 68, 64)
    assert q.offset - g.data_offset == 32
    assert raw[q.offset + 67] == 67
    assert g.tensor("odd").len is None, "Q4_0 is not sized here"
    assert g.tensor("nothing") is None


def test_a_short_prefix_asks_for_more_and_bad_files_are_refused():
    raw = sample()
    with pytest.raises(gguf.Truncated, match="40 bytes"):
        gguf.Gguf.parse(raw[:40], len(raw))
    with pytest.raises(gguf.Magic):
        gguf.Gguf.parse(b"X" + raw[1:], len(raw))
    with pytest.raises(gguf.Version, match="version 1"):
        gguf.Gguf.parse(raw[:4] + struct.pack("<I", 1) + raw[8:], len(raw))
    with pytest.raises(gguf.Invalid, match="past the end"):
        gguf.Gguf.parse(raw, len(raw) - 70)          # the file is cut inside q, the last sized tensor
    with pytest.raises(gguf.Invalid, match="inside its header"):
        gguf.Gguf.parse(raw, 100)


def test_a_file_is_read_in_growing_pieces(tmp_path):
    path = tmp_path / "m.gguf"
    path.write_bytes(sample())
    whole = gguf.open(path)
    small = gguf.open(path, first_read=16)
    assert small.tensors == whole.tensors and small.keys() == whole.keys()
    assert bytes(small.read(small.tensor("q"))) == bytes(range(68))
    with pytest.raises(gguf.Invalid):
        small.read(small.tensor("odd"))
    with pytest.raises(gguf.Read):
        gguf.open(tmp_path / "absent.gguf")
    parsed = gguf.Gguf.parse(sample(), len(sample()))
    with pytest.raises(gguf.Read):
        parsed.read(parsed.tensor("q"))               # parsed from bytes: there is no file to read


def test_every_value_type_and_its_conversions():
    raw = w.file([("u8", w.U8, 200), ("i8", w.I8, -5), ("u16", w.U16, 60000), ("i16", w.I16, -300),
                  ("u32", w.U32, 4000000000), ("i32", w.I32, -7), ("f32", w.F32, 0.5), ("yes", w.BOOL, 1),
                  ("no", w.BOOL, 0), ("u64", w.U64, 2 ** 63 + 1), ("i64", w.I64, -2 ** 40), ("f64", w.F64, 1e300),
                  ("ints", w.ARRAY, (w.I32, [3, -4, 5])), ("floats", w.ARRAY, (w.F32, [0.25, -2.0])),
                  ("empty", w.ARRAY, (w.U8, [])), ("text", w.STRING, "")], [])
    g = gguf.Gguf.parse(raw, len(raw))
    assert [g.get(k) for k in ("u8", "i8", "u16", "i16", "u32", "i32")] == [200, -5, 60000, -300, 4000000000, -7]
    assert (g.get("f32"), g.get("yes"), g.get("no"), g.get("u64"), g.get("i64"), g.get("f64")) == \
        (0.5, True, False, 2 ** 63 + 1, -2 ** 40, 1e300)
    assert g.get("ints") == [3, -4, 5] and g.get("floats") == [0.25, -2.0] and g.get("empty") == [] and g.get("text") == ""
    # `as_u64` takes any integer that is not negative; `as_f64` only floats
    from ctypes import byref, c_double, c_uint64
    from loadngo_b200 import compute
    L, v, d = compute.lib(), c_uint64(), c_double()
    assert L.cc_gguf_get_u64(g._h, b"i16", -1, byref(v)) == 0
    assert L.cc_gguf_get_u64(g._h, b"u8", -1, byref(v)) == 1 and v.value == 200
    assert L.cc_gguf_get_u64(g._h, b"ints", 2, byref(v)) == 1 and v.value == 5
    assert L.cc_gguf_get_u64(g._h, b"ints", 1, byref(v)) == 0
    assert L.cc_gguf_get_u64(g._h, b"ints", 3, byref(v)) == 0
    assert L.cc_gguf_get_f64(g._h, b"u32", -1, byref(d)) == 0
    assert L.cc_gguf_get_f64(g._h, b"f64", -1, byref(d)) == 1 and d.value == 1e300


@pytest.mark.parametrize("metadata, tensors, alignment, error, text", [
    ([("a", w.ARRAY, (w.ARRAY, [(w.U8, [1])]))], [], 32, gguf.Invalid, "nested"),
    ([("a", w.U8, 1), ("a", w.U8, 2)], [], 32, gguf.Invalid, "repeats"),
    ([("flag", w.BOOL, 2)], [], 32, gguf.Invalid, "bool byte 2"),
    ([("a", 13, b"\0\0\0\0")], [], 32, gguf.ValueType, "13"),
    ([("bad", w.STRING, b"\xff\xfe")], [], 32, gguf.Utf8, "UTF-8"),
    ([("bad", w.STRING, b"\xed\xa0\x80")], [], 32, gguf.Utf8, "UTF-8"),          # a surrogate
    ([("bad", w.STRING, b"\xc0\x80")], [], 32, gguf.Utf8, "UTF-8"),              # an overlong form
    ([("general.alignment", w.U32, 24)], [], 32, gguf.Invalid, "general.alignment"),
    ([("general.alignment", w.STRING, "32")], [], 32, gguf.Invalid, "general.alignment"),
    ([], [("t", [33], gguf.Q8_0, bytes(34))], 32, gguf.Invalid, "whole blocks of 32"),
    ([], [("t", [16], gguf.MXFP4, bytes(17))], 32, gguf.Invalid, "whole blocks of 32"),
    ([], [("t", [], gguf.F32, bytes(4))], 32, gguf.Invalid, "0 dimensions"),
    ([], [("t", [1] * 9, gguf.F32, bytes(4))], 32, gguf.Invalid, "9 dimensions"),
    ([], [("t", [2 ** 40, 2 ** 40], gguf.F32, bytes(4))], 32, gguf.Invalid, "overflows"),
])
def test_what_cannot_be_right_is_refused(metadata, tensors, alignment, error, text):
    raw = w.file(metadata, tensors, alignment)
    with pytest.raises(error, match=text):
        gguf.Gguf.parse(raw, len(raw))


def test_alignment_from_the_metadata_places_the_data():
    raw = w.file([("general.alignment", w.U32, 64)],
                 [("a", [2], gguf.BF16, bytes([1, 2, 3, 4])), ("b", [32], gguf.MXFP4, bytes(range(17)))], alignment=64)
    g = gguf.Gguf.parse(raw, len(raw))
    assert g.alignment == 64 and g.data_offset % 64 == 0
    a, b = g.tensor("a"), g.tensor("b")
    assert (a.len, b.len) == (4, 17) and b.offset - a.offset == 64
    assert raw[b.offset:b.offset + 17] == bytes(range(17))
    # an offset that is not a multiple of the alignment
    wrong = w.file([], [("a", [2], gguf.BF16, bytes(4)), ("b", [32], gguf.MXFP4, bytes(17))], offsets=[0, 48])
    with pytest.raises(gguf.Invalid, match="b: unaligned"):
        gguf.Gguf.parse(wrong, len(wrong))


def test_version_2_shares_the_layout():
    raw = w.file([("k", w.U32, 7)], [("t", [4], gguf.F16, bytes(8))], version=2)
    g = gguf.Gguf.parse(raw, len(raw))
    assert g.version == 2 and g.get("k") == 7 and g.tensor("t").len == 8


@pytest.mark.skipif(not os.path.exists(TINY), reason="the reference checkout is not mounted")
def test_the_reference_tiny_model_reads_like_the_gguf_package_reads_it():
    ref = pytest.importorskip("gguf")
    theirs = ref.GGUFReader(TINY)
    ours = gguf.open(TINY, first_read=512)           # the header is 5.6 KB: several doublings
    assert ours.data_offset == theirs.data_offset and ours.alignment == theirs.alignment
    for key, field in theirs.fields.items():
        if key.startswith("GGUF."):
            continue
        want = field.contents()
        got = ours.get(key)
        assert got == pytest.approx(want) if isinstance(want, float) else got == want, key
    assert [t.name for t in ours.tensors] == [t.name for t in theirs.tensors]
    for mine, t in zip(ours.tensors, theirs.tensors):
        assert mine.dims == [int(d) for d in t.shape] and mine.ggml_type == int(t.tensor_type)
        assert mine.offset == t.data_offset and mine.len == t.n_bytes
        assert np.array_equal(ours.read(mine), np.asarray(t.data).view(np.uint8).reshape(-1)), mine.name


GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "tiny_block.npz")


def test_the_tiny_model_written_from_the_golden_vectors_gives_the_reference_shape(tmp_path):
    """The model file the GPU tests load: its header parses, `Config.from_gguf` reads the shape the
    reference's fixture has, and (where the reference checkout is present) every tensor's bytes
    are the reference file's."""
    import json
    from loadngo_b200.gpt_oss import Config, ConfigError
    golden = np.load(GOLDEN)
    path = tmp_path / "tiny.gguf"
    w.tiny_model(golden, path)
    g = gguf.open(path, first_read=1024)
    c = Config.from_gguf(g)
    meta = json.loads(str(golden["meta"]))
    assert (c.layers, c.hidden, c.heads, c.kv_heads, c.head_dim, c.window) == \
        (meta["layers"], meta["hidden"], meta["heads"], meta["kv_heads"], meta["dim"], meta["window"]) == (4, 128, 4, 2, 32, 8)
    assert (c.experts, c.experts_used, c.expert_hidden, c.vocab, c.context_length) == (4, 2, 64, 512, 2048)
    assert (c.theta, c.factor, c.original_context) == (150000.0, 32.0, 64.0) and c.eps == float(np.float32(1e-5))
    assert [c.is_sliding(l) for l in range(4)] == [True, False, True, False]
    if os.path.exists(TINY):
        theirs = gguf.open(TINY)
        assert Config.from_gguf(theirs) == c
        assert [(t.name, t.dims, t.ggml_type, t.len) for t in theirs.tensors] == \
            [(t.name, t.dims, t.ggml_type, t.len) for t in g.tensors]
        for mine, t in zip(g.tensors, theirs.tensors):
            assert np.array_equal(g.read(mine), theirs.read(t)), t.name
    # the refusals of config.rs:52-95
    for drop, text in (("gpt-oss.block_count", "block_count is missing"), ("gpt-oss.rope.scaling.type", "YaRN")):
        raw = path.read_bytes().replace(drop.encode(), drop.encode()[:-1] + b"_")
        with pytest.raises(ConfigError, match=text):
            Config.from_gguf(gguf.Gguf.parse(raw, len(raw)))
    raw = path.read_bytes().replace(b"\x07\x00\x00\x00\x00\x00\x00\x00gpt-oss", b"\x07\x00\x00\x00\x00\x00\x00\x00gpt-0ss", 1)
    with pytest.raises(ConfigError, match="architecture"):
        Config.from_gguf(gguf.Gguf.parse(raw, len(raw)))


def test_damaged_headers_are_refused_or_read_never_worse():
    """The reader is native code that reads files nobody vouches for: every truncation of a valid
    file and a few thousand seeded byte changes either parse (and then every sized tensor lies inside
    the file) or are refused with one of the reader's errors."""
    raw = sample()
    rng = np.random.default_rng(12)
    cases = [raw[:n] for n in range(0, len(raw), 3)]
    for _ in range(3000):
        damaged = bytearray(raw)
        for _ in range(int(rng.integers(1, 4))):
            at = int(rng.integers(0, 400))              # the header: counts, lengths, types, offsets
            damaged[at] = int(rng.integers(0, 256))
        cases.append(bytes(damaged))
    parsed = refused = 0
    for data in cases:
        try:
            g = gguf.Gguf.parse(data, len(data))
        except gguf.GgufError:
            refused += 1
            continue
        parsed += 1
        for t in g.tensors:
            assert t.len is None or t.offset + t.len <= len(data)
        for key in g.keys():
            g.get(key)
        g.close()
    assert parsed > 0 and refused > 0
