"""Writes GGUF v3 files for the tests (an independent statement of the layout the reader parses:
ggml's docs/gguf.md, version 3)."""
from __future__ import annotations

import struct

import numpy as np

U8, I8, U16, I16, U32, I32, F32, BOOL, STRING, ARRAY, U64, I64, F64 = range(13)
_FMT = {U8: "<B", I8: "<b", U16: "<H", I16: "<h", U32: "<I", I32: "<i", F32: "<f", BOOL: "<B", U64: "<Q", I64: "<q",
        F64: "<d"}


def string(s) -> bytes:
    raw = s if isinstance(s, bytes) else s.encode()
    return struct.pack("<Q", len(raw)) + raw


def value(kind: int, v) -> bytes:
    """The encoded value (without its type word). Arrays are `(element kind, [values])`."""
    if kind == STRING:
        return string(v)
    if kind == ARRAY:
        element, items = v
        return struct.pack("<IQ", element, len(items)) + b"".join(value(element, x) for x in items)
    return struct.pack(_FMT[kind], v)


def file(metadata, tensors, alignment: int = 32, version: int = 3, offsets=None) -> bytes:
    """metadata: [(key, kind, value)]; tensors: [(name, dims, ggml type id, bytes)]; `offsets` overrides
    the offsets written in the tensor descriptions (to write a file that is wrong)."""
    pad = lambda n: -n % alignment
    out = b"GGUF" + struct.pack("<IQQ", version, len(tensors), len(metadata))
    for key, kind, v in metadata:
        out += string(key) + struct.pack("<I", kind) + (v if isinstance(v, bytes) and kind != STRING else value(kind, v))
    data = b""
    for i, (name, dims, kind, raw) in enumerate(tensors):
        out += string(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims)
        out += struct.pack("<IQ", kind, len(data) if offsets is None else offsets[i])
        raw = np.ascontiguousarray(raw).tobytes() if isinstance(raw, np.ndarray) else bytes(raw)
        data += raw + b"\0" * pad(len(raw))
    out += b"\0" * pad(len(out))
    return out + data


def tiny_model(golden, path) -> None:
    """Writes the tiny gpt-oss model of tests/golden/tiny_block.npz (`golden`: the loaded npz) as a
    GGUF file with the tensor names, element types, dimensions and metadata keys a gpt-oss GGUF
    has (the ones `Config::from_gguf`, gpt-oss/src/config.rs:38-97, and `Model::from_tensors`,
    gpt-oss/src/model.rs:311-380, ask for)."""
    import json
    m = json.loads(str(golden["meta"]))
    hidden, qw, kw = m["hidden"], m["heads"] * m["dim"], m["kv_heads"] * m["dim"]
    eh, experts = m["expert_hidden"], m["experts"]
    metadata = [
        ("general.architecture", STRING, "gpt-oss"), ("gpt-oss.block_count", U32, m["layers"]),
        ("gpt-oss.context_length", U32, m["context_length"]), ("gpt-oss.embedding_length", U32, hidden),
        ("gpt-oss.feed_forward_length", U32, m["feed_forward_length"]), ("gpt-oss.attention.head_count", U32, m["heads"]),
        ("gpt-oss.attention.head_count_kv", U32, m["kv_heads"]), ("gpt-oss.rope.freq_base", F32, m["theta"]),
        ("gpt-oss.attention.layer_norm_rms_epsilon", F32, m["eps"]), ("gpt-oss.expert_count", U32, experts),
        ("gpt-oss.expert_used_count", U32, m["experts_used"]), ("gpt-oss.attention.key_length", U32, m["dim"]),
        ("gpt-oss.attention.value_length", U32, m["dim"]), ("gpt-oss.attention.sliding_window", U32, m["window"]),
        ("gpt-oss.expert_feed_forward_length", U32, eh), ("gpt-oss.rope.scaling.type", STRING, "yarn"),
        ("gpt-oss.rope.scaling.factor", F32, m["factor"]),
        ("gpt-oss.rope.scaling.original_context_length", U32, m["original_context"])]
    Q8, MX, F = 8, 39, 0
    tensors = [("token_embd.weight", [hidden, m["vocab"]], Q8, golden["token_embd_q8_0"]),
               ("output.weight", [hidden, m["vocab"]], Q8, golden["output_q8_0"]),
               ("output_norm.weight", [hidden], F, golden["output_norm"])]
    for l in range(m["layers"]):
        g = lambda name: golden[f"l{l}_{name}"]
        b = f"blk.{l}."
        tensors += [
            (b + "attn_norm.weight", [hidden], F, g("attn_norm")),
            (b + "attn_q.weight", [hidden, qw], Q8, g("attn_q_q8_0")), (b + "attn_k.weight", [hidden, kw], Q8, g("attn_k_q8_0")),
            (b + "attn_v.weight", [hidden, kw], Q8, g("attn_v_q8_0")),
            (b + "attn_output.weight", [qw, hidden], Q8, g("attn_output_q8_0")),
            (b + "attn_q.bias", [qw], F, g("attn_q_bias")), (b + "attn_k.bias", [kw], F, g("attn_k_bias")),
            (b + "attn_v.bias", [kw], F, g("attn_v_bias")), (b + "attn_output.bias", [hidden], F, g("attn_output_bias")),
            (b + "attn_sinks.weight", [m["heads"]], F, g("sinks")),
            (b + "post_attention_norm.weight", [hidden], F, g("ffn_norm")),
            (b + "ffn_gate_inp.weight", [hidden, experts], F, g("router")), (b + "ffn_gate_inp.bias", [experts], F, g("router_bias")),
            (b + "ffn_gate_exps.weight", [hidden, eh, experts], MX, g("ffn_gate_exps_mxfp4")),
            (b + "ffn_up_exps.weight", [hidden, eh, experts], MX, g("ffn_up_exps_mxfp4")),
            (b + "ffn_down_exps.weight", [eh, hidden, experts], MX, g("ffn_down_exps_mxfp4")),
            (b + "ffn_gate_exps.bias", [eh, experts], F, g("ffn_gate_exps_bias")),
            (b + "ffn_up_exps.bias", [eh, experts], F, g("ffn_up_exps_bias")),
            (b + "ffn_down_exps.bias", [hidden, experts], F, g("ffn_down_exps_bias"))]
    with open(path, "wb") as fh:
        fh.write(file(metadata, tensors))
