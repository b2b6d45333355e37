"""Pins the CPU oracle to the reference's own end-to-end fixture and writes golden vectors.

Run where the reference checkout is mounted:

    python tests/golden/make_tiny_golden.py <loadngo checkout>

It replays `gpt-oss/tests/fixtures/tiny` (a 4-layer random-weight gpt-oss: 4 query heads over
2 key/value heads of 32, window 8 on even layers, YaRN with original context 64, 40 tokens;
made by the reference's `scripts/gpt_oss_tiny_oracle.py`) one position at a time, exactly as
`gpt-oss/tests/tiny_oracle.rs:10-41` does, with every step of `Model::step`
(`gpt-oss/src/model.rs:408-478`) restated in NumPy EXCEPT attention, RoPE and the cache
append, which are done by the C oracle (`oracle/oracle.c`).  The logits must match the
fixture's `logits.f32` (transformers' fp32 eager output) within the reference's own 2e-3.

Only then does it store, per layer, what went into and came out of the oracle's attention
(`tiny_attention.npz`: q, k, v before rotation, sinks, outputs, rotated q, cache rows), so that
the tests can replay them anywhere - the reference checkout does not travel.

It also checks that each of the attention-relevant deliberate bugs listed in the reference's
`docs/GPT_OSS.md:112-121` breaks the 2e-3 match, so the pin is known to be sensitive to them;
the worst logit error of each is stored in the same file.
"""
from __future__ import annotations

import json
import os
import sys

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))
from oracle import oracle  # noqa: E402


def load(reference_root: str):
    import gguf
    from gguf.quants import dequantize

    d = os.path.join(reference_root, "gpt-oss", "tests", "fixtures", "tiny")
    reader = gguf.GGUFReader(os.path.join(d, "model.gguf"))
    meta = {k: f.contents() for k, f in reader.fields.items() if k.startswith("gpt-oss.")}
    tensors = {t.name: np.array(dequantize(t.data, t.tensor_type), np.float32) for t in reader.tensors}
    # the attention projections also as they are stored: ggml Q8_0 blocks, row after row
    for t in reader.tensors:
        if t.tensor_type == gguf.GGMLQuantizationType.Q8_0:
            tensors[t.name + ":q8_0"] = np.ascontiguousarray(t.data, np.uint8).reshape(-1)
        if t.tensor_type == gguf.GGMLQuantizationType.MXFP4:
            tensors[t.name + ":mxfp4"] = np.ascontiguousarray(t.data, np.uint8).reshape(-1)
    with open(os.path.join(d, "oracle.json")) as fh:
        ids = json.load(fh)["ids"]
    logits = np.fromfile(os.path.join(d, "logits.f32"), np.float32)
    return meta, tensors, ids, logits


def rms_norm(x, w, eps):
    # model.rs:274-280: f64 mean of squares, f32 1/sqrt, x * scale * w
    mean = np.sum(x.astype(np.float64) ** 2) / x.size
    scale = np.float32(1.0 / np.sqrt(mean + np.float64(np.float32(eps))))
    return (x * scale * w).astype(np.float32)


def experts(T, l, x, used):
    # model.rs:482-548: top-k router logits (ties: lower index first), softmax over those,
    # down((clamp(up,-7,7)+1) * g * sigmoid(1.702 g)), g = min(gate, 7)
    router = T[f"blk.{l}.ffn_gate_inp.weight"] @ x + T[f"blk.{l}.ffn_gate_inp.bias"]
    order = sorted(range(router.size), key=lambda e: (-router[e], e))[:used]
    w = np.exp(router[order] - router[order[0]]).astype(np.float32)
    w = w / w.sum(dtype=np.float32)
    out = np.zeros_like(x)
    for e, we in zip(order, w):
        g = T[f"blk.{l}.ffn_gate_exps.weight"][e] @ x + T[f"blk.{l}.ffn_gate_exps.bias"][e]
        u = T[f"blk.{l}.ffn_up_exps.weight"][e] @ x + T[f"blk.{l}.ffn_up_exps.bias"][e]
        g = np.minimum(g, np.float32(7.0))
        u = np.clip(u, np.float32(-7.0), np.float32(7.0))
        hidden = ((u + 1) * g / (1 + np.exp(np.float32(-1.702) * g))).astype(np.float32)
        y = T[f"blk.{l}.ffn_down_exps.weight"][e] @ hidden + T[f"blk.{l}.ffn_down_exps.bias"][e]
        out += we * y.astype(np.float32)
    return out


def replay(meta, T, ids, mutation: str | None = None, record: dict | None = None):
    layers = meta["gpt-oss.block_count"]
    heads = meta["gpt-oss.attention.head_count"]
    kv_heads = meta["gpt-oss.attention.head_count_kv"]
    dim = meta["gpt-oss.attention.key_length"]
    window = meta["gpt-oss.attention.sliding_window"]
    eps = meta["gpt-oss.attention.layer_norm_rms_epsilon"]
    used = meta["gpt-oss.expert_used_count"]
    factor = meta["gpt-oss.rope.scaling.factor"]
    if mutation == "no_yarn_interpolation":
        # plain RoPE frequencies, YaRN's cos/sin factor kept
        rope = oracle.Rope(dim, meta["gpt-oss.rope.freq_base"], factor,
                           float(meta["gpt-oss.rope.scaling.original_context_length"]),
                           beta_fast=1e-9, beta_slow=1e-10)
    else:
        rope = oracle.Rope(dim, meta["gpt-oss.rope.freq_base"], factor,
                           float(meta["gpt-oss.rope.scaling.original_context_length"]))
    sessions = []
    for l in range(layers):
        sliding = (l % 2 == 0) if mutation != "sliding_on_odd" else (l % 2 == 1)
        w = window if mutation != "window_one_narrower" else window - 1
        sinks = T[f"blk.{l}.attn_sinks.weight"] if mutation != "no_sinks" else None
        s = oracle.Session(heads, kv_heads, dim, len(ids), window=w if sliding else 0,
                           sinks=sinks, rope=rope)
        if mutation == "no_yarn_scale":
            s._rope_scale = 1.0
        if mutation == "flipped_rotation_sign":
            s._inv = -s._inv
        sessions.append(s)
    all_logits = []
    for pos, token in enumerate(ids):
        h = T["token_embd.weight"][token].copy()
        for l in range(layers):
            if record is not None:
                record.setdefault(f"l{l}_h_in", []).append(h.copy())
            x = rms_norm(h, T[f"blk.{l}.attn_norm.weight"], eps)
            q = T[f"blk.{l}.attn_q.weight"] @ x + T[f"blk.{l}.attn_q.bias"]
            k = T[f"blk.{l}.attn_k.weight"] @ x + T[f"blk.{l}.attn_k.bias"]
            v = T[f"blk.{l}.attn_v.weight"] @ x + T[f"blk.{l}.attn_v.bias"]
            q = q.astype(np.float32).reshape(1, heads, dim)
            k = k.astype(np.float32).reshape(1, kv_heads, dim)
            v = v.astype(np.float32).reshape(1, kv_heads, dim)
            att, q_rot = sessions[l].feed(q, k, v)
            if record is not None:
                for name, val in (("q", q), ("k", k), ("v", v), ("out", att), ("q_rot", q_rot)):
                    record.setdefault(f"l{l}_{name}", []).append(val[0])
            o = T[f"blk.{l}.attn_output.weight"] @ att.reshape(-1) + T[f"blk.{l}.attn_output.bias"]
            h = h + o.astype(np.float32)
            x = rms_norm(h, T[f"blk.{l}.post_attention_norm.weight"], eps)
            if record is not None:
                record.setdefault(f"l{l}_h_att", []).append(h.copy())
                record.setdefault(f"l{l}_x_ffn", []).append(x.copy())
            h = h + experts(T, l, x, used)
            if record is not None:
                record.setdefault(f"l{l}_h_out", []).append(h.copy())
        x = rms_norm(h, T["output_norm.weight"], eps)
        all_logits.append((T["output.weight"] @ x).astype(np.float32))
    if record is not None:
        for l in range(layers):
            record[f"l{l}_kcache"] = sessions[l].keys.copy()
            record[f"l{l}_vcache"] = sessions[l].values.copy()
            record[f"l{l}_sinks"] = T[f"blk.{l}.attn_sinks.weight"].astype(np.float32)
    return np.stack(all_logits)


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: make_tiny_golden.py <loadngo checkout>")
    root = sys.argv[1]
    meta, T, ids, want = load(root)
    want = want.reshape(len(ids), -1)
    record: dict = {}
    got = replay(meta, T, ids, record=record)
    worst = float(np.abs(got - want).max())
    print(f"tiny fixture: worst logit error over {len(ids)} positions = {worst:.3e} (tolerance 2e-3)")
    assert worst < 2e-3, "the oracle does not reproduce the reference's fixture"
    out = {k: np.stack(v) if isinstance(v, list) else v for k, v in record.items()}
    mutations = ["no_sinks", "window_one_narrower", "sliding_on_odd", "flipped_rotation_sign",
                 "no_yarn_scale", "no_yarn_interpolation"]
    errs = []
    for m in mutations:
        e = float(np.abs(replay(meta, T, ids, mutation=m) - want).max())
        print(f"  mutation {m}: worst logit error {e:.3e}")
        assert e > 2e-3, f"mutation {m} was not detected"
        errs.append(e)
    out["meta"] = np.array(json.dumps({
        "layers": meta["gpt-oss.block_count"], "heads": meta["gpt-oss.attention.head_count"],
        "kv_heads": meta["gpt-oss.attention.head_count_kv"],
        "dim": meta["gpt-oss.attention.key_length"],
        "window": meta["gpt-oss.attention.sliding_window"],
        "theta": meta["gpt-oss.rope.freq_base"], "factor": meta["gpt-oss.rope.scaling.factor"],
        "original_context": meta["gpt-oss.rope.scaling.original_context_length"],
        "positions": len(ids), "worst_logit_error": worst,
        "mutations": dict(zip(mutations, errs)),
    }))
    # the block-level vectors (residual stream in and out of the attention half of each layer, the
    # Q8_0 projections as stored) go to a file of their own
    block = {k: out.pop(k) for k in [k for k in out if k.endswith(("_h_in", "_h_att", "_x_ffn", "_h_out"))]}
    for l in range(meta["gpt-oss.block_count"]):
        for name in ("attn_q", "attn_k", "attn_v", "attn_output"):
            block[f"l{l}_{name}_q8_0"] = T[f"blk.{l}.{name}.weight:q8_0"]
            block[f"l{l}_{name}_bias"] = T[f"blk.{l}.{name}.bias"].astype(np.float32)
        block[f"l{l}_attn_norm"] = T[f"blk.{l}.attn_norm.weight"].astype(np.float32)
        block[f"l{l}_ffn_norm"] = T[f"blk.{l}.post_attention_norm.weight"].astype(np.float32)
        block[f"l{l}_sinks"] = out[f"l{l}_sinks"]
        # the experts as stored: router (f32), ggml MXFP4 blocks of all experts, biases
        block[f"l{l}_router"] = T[f"blk.{l}.ffn_gate_inp.weight"].astype(np.float32)
        block[f"l{l}_router_bias"] = T[f"blk.{l}.ffn_gate_inp.bias"].astype(np.float32)
        for name in ("ffn_gate_exps", "ffn_up_exps", "ffn_down_exps"):
            block[f"l{l}_{name}_mxfp4"] = T[f"blk.{l}.{name}.weight:mxfp4"]
            block[f"l{l}_{name}_bias"] = T[f"blk.{l}.{name}.bias"].astype(np.float32)
    # what surrounds the layers: embedding rows of the prompt's tokens (widened), the final norm,
    # the output matrix as stored, and the logits the reference's fixture holds
    block["embedded"] = np.stack([T["token_embd.weight"][t] for t in ids]).astype(np.float32)
    block["output_norm"] = T["output_norm.weight"].astype(np.float32)
    block["output_q8_0"] = T["output.weight:q8_0"]
    # the embedding as stored and the prompt's token ids: with them the tests can write the whole
    # model as a GGUF file again and load it the way the reference loads its fixture
    block["token_embd_q8_0"] = T["token_embd.weight:q8_0"]
    block["ids"] = np.array(ids, np.uint32)
    block["logits"] = want.astype(np.float32)
    block["meta"] = np.array(json.dumps({
        "layers": meta["gpt-oss.block_count"], "hidden": int(T["token_embd.weight"].shape[1]),
        "heads": meta["gpt-oss.attention.head_count"], "kv_heads": meta["gpt-oss.attention.head_count_kv"],
        "dim": meta["gpt-oss.attention.key_length"], "window": meta["gpt-oss.attention.sliding_window"],
        "eps": float(meta["gpt-oss.attention.layer_norm_rms_epsilon"]),
        "theta": meta["gpt-oss.rope.freq_base"], "factor": meta["gpt-oss.rope.scaling.factor"],
        "original_context": meta["gpt-oss.rope.scaling.original_context_length"], "positions": len(ids),
        "experts": meta["gpt-oss.expert_count"], "experts_used": meta["gpt-oss.expert_used_count"],
        "expert_hidden": meta["gpt-oss.expert_feed_forward_length"], "vocab": int(want.shape[1]),
        "feed_forward_length": meta["gpt-oss.feed_forward_length"], "context_length": meta["gpt-oss.context_length"]}))
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "tiny_attention.npz")
    np.savez_compressed(path, **out)
    print(f"wrote {path} ({os.path.getsize(path)} bytes)")
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "tiny_block.npz")
    np.savez_compressed(path, **block)
    print(f"wrote {path} ({os.path.getsize(path)} bytes)")


if __name__ == "__main__":
    main()
