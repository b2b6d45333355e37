"""A second opinion on the oracle: the attention, the sink and the YaRN rotation of transformers'
gpt-oss (the implementation the reference's own fixture was generated with,
scripts/gpt_oss_tiny_oracle.py:94-137, fp32 eager) against the C oracle on seeded random inputs at
gpt-oss shapes.  Harness only: nothing of it is shipped or timed."""
import types

import numpy as np
import pytest

from oracle import oracle

torch = pytest.importorskip("torch")
modeling = pytest.importorskip("transformers.models.gpt_oss.modeling_gpt_oss")

H, G, D = 64, 8, 64


def test_yarn_frequencies_and_factor_match_transformers_rope_init():
    from transformers import GptOssConfig
    try:
        cfg = GptOssConfig(hidden_size=128, num_attention_heads=H, num_key_value_heads=G, head_dim=D, num_hidden_layers=2,
                           max_position_embeddings=131072, rope_theta=150000.0,
                           rope_scaling={"rope_type": "yarn", "factor": 32.0, "beta_fast": 32.0, "beta_slow": 1.0,
                                         "truncate": False, "original_max_position_embeddings": 4096})
        rope = modeling.GptOssRotaryEmbedding(cfg)
    except Exception as e:      # the constructor's arguments moved between releases
        pytest.skip(f"this transformers builds its rotary embedding differently: {e}")
    want_inv, want_scale = oracle.Rope().inv_freq()
    assert np.allclose(rope.inv_freq.double().numpy(), want_inv, rtol=2e-6, atol=0)
    assert abs(float(rope.attention_scaling) - want_scale) < 1e-6


@pytest.mark.parametrize("window", [0, 128])
def test_attention_with_sinks_and_window_matches_transformers_eager(window):
    rng = np.random.default_rng(17)
    T = 200
    q = rng.standard_normal((T, H, D)).astype(np.float32)
    k = rng.standard_normal((T, G, D)).astype(np.float32)
    v = rng.standard_normal((T, G, D)).astype(np.float32)
    sinks = rng.standard_normal(H).astype(np.float32)
    # the oracle, reference-faithful mode (f32 cache), no rotation: a table of cos = 1, sin = 0 is what
    # a rope with all-zero frequencies gives; easier: rotate by position 0 only through attention_f64
    want = oracle.attention_f64(q, k, v, start=0, window=window if window else 2 ** 62, scale=0.125, sinks=sinks)
    module = types.SimpleNamespace(num_key_value_groups=H // G, sinks=torch.from_numpy(sinks), training=False)
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    visible = (j <= i) & ((j > i - window) if window else torch.ones_like(j, dtype=torch.bool))
    mask = torch.zeros(T, T).masked_fill(~visible, float("-inf"))[None, None]
    out, _ = modeling.eager_attention_forward(module, torch.from_numpy(q).permute(1, 0, 2)[None],
                                              torch.from_numpy(k).permute(1, 0, 2)[None],
                                              torch.from_numpy(v).permute(1, 0, 2)[None], mask, scaling=0.125, dropout=0.0)
    got = out[0].numpy()                                   # [T][H][D]
    assert got.shape == (T, H, D)
    assert np.abs(got - want).max() < 2e-5


def test_the_c_oracle_session_agrees_with_the_float64_definition_it_is_checked_with():
    rng = np.random.default_rng(3)
    T = 150
    q = rng.standard_normal((T, H, D)).astype(np.float32)
    k = rng.standard_normal((T, G, D)).astype(np.float32)
    v = rng.standard_normal((T, G, D)).astype(np.float32)
    sinks = rng.standard_normal(H).astype(np.float32)
    for window in (0, 128):
        s = oracle.Session(H, G, D, T, window=window, sinks=sinks, rope=oracle.Rope())
        got, q_rot = s.feed(q, k, v)
        want = oracle.attention_f64(q_rot, s.keys[:T], s.values[:T], start=0, window=window if window else 2 ** 62,
                                    scale=0.125, sinks=sinks)
        assert np.abs(got - want).max() < 2e-5
