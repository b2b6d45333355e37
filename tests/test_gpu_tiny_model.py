"""The whole model on the GPU against transformers' logits on the reference's tiny random model,
in the feeding patterns of gpt-oss/tests/gpu_oracle.rs:76-145: one position at a time with a
sliding ring that wraps (routed on the GPU and on the CPU), passes large enough for the tiled
kernels, consecutive passes interleaved two at a time against the same passes one after
another, and a session that goes back.  The model is loaded from a GGUF file (written from the
golden vectors, tensor for tensor the reference's file) through the library's reader."""
import os

import numpy as np
import pytest

from loadngo_b200 import compute
from loadngo_b200.gpt_oss import ALL, LAST, GpuModel, Invalid
from tests import gguf_writer

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "tiny_block.npz")
TOLERANCE = 2e-3


@pytest.fixture(scope="module")
def fixture(tmp_path_factory):
    golden = np.load(GOLDEN)
    path = tmp_path_factory.mktemp("tiny") / "model.gguf"
    gguf_writer.tiny_model(golden, path)
    return str(path), [int(t) for t in golden["ids"]], golden["logits"]


def largest_error(fixture, gpu, chunk, parts, gpu_routing=True, pipeline=True):
    """Feeds the fixture's tokens in parts of the given sizes; returns the largest logit error and
    the submissions made (gpu_oracle.rs:48-74)."""
    path, ids, want = fixture
    model = GpuModel.load(path, chunk, 64, gpu)
    model.gpu_routing, model.pipeline = gpu_routing, pipeline
    session = model.session()
    at, worst = 0, 0.0
    for part in parts:
        logits = model.feed(session, ids[at:at + part], ALL)
        assert len(logits) == part
        for i, row in enumerate(logits):
            error = float(np.abs(row - want[at + i]).max())
            assert error < TOLERANCE, f"position {at + i}: max error {error}"
            worst = max(worst, error)
        at += part
    assert at == len(ids) == len(session)
    session.free()
    model.free()
    return worst, dict(model.submissions)


def test_one_position_at_a_time_through_a_wrapping_ring(fixture, gpu):
    # chunk 8: sliding layers keep (8 + 8) rounded up to 32 rows, so 40 positions wrap
    worst, made = largest_error(fixture, gpu, 8, [1] * 40, gpu_routing=True)
    print(f"\none at a time, routed on the GPU: largest logit error {worst:.3e}")
    assert made == {"token": 40, "attention": 0, "experts": 0, "output": 0}      # each token one submission
    worst, made = largest_error(fixture, gpu, 8, [1] * 40, gpu_routing=False)
    print(f"one at a time, routed on the CPU: largest logit error {worst:.3e}")
    assert made == {"token": 0, "attention": 160, "experts": 160, "output": 40}


def test_passes_on_the_tiled_kernels_and_after_them(fixture, gpu):
    worst, made = largest_error(fixture, gpu, 40, [33, 7])
    print(f"\n33 then 7: largest logit error {worst:.3e}")
    assert made["output"] == 3                       # 33 rows of logits leave in groups of 32
    worst, _ = largest_error(fixture, gpu, 8, [8, 8, 3, 8, 8, 5])
    print(f"chunks of 8: largest logit error {worst:.3e}")
    worst, _ = largest_error(fixture, gpu, 22, [16, 1, 1, 22])
    print(f"a pass, two tokens, a pass: largest logit error {worst:.3e}")


@pytest.mark.parametrize("chunk, label", [(8, "chunks of 8: two pairs and one alone"), (16, "chunks of 16: a pair and one alone"),
                                          (32, "chunks of 32: a tiled pair")])
def test_consecutive_passes_interleave(fixture, gpu, chunk, label):
    """One call, several passes: pairs of passes interleaved layer by layer (and a last odd one
    alone), against the same passes one after another: the same submissions, the same logits."""
    paired, made_paired = largest_error(fixture, gpu, chunk, [40], pipeline=True)
    alone, made_alone = largest_error(fixture, gpu, chunk, [40], pipeline=False)
    print(f"\n{label}: largest logit error {paired:.3e} interleaved, {alone:.3e} one after another")
    assert made_paired == made_alone


def test_a_session_goes_back_and_reads_on_as_if_never_ahead(fixture, gpu):
    path, ids, want = fixture
    # a sliding ring of (8 + 8) rounded up to 32 rows; 30 positions in, back 6
    model = GpuModel.load(path, 8, 64, gpu)
    session = model.session_holding(64)
    assert session.capacity() == 64 and session.is_empty()
    last = model.feed(session, ids[:30], LAST)
    assert len(last) == 1 and float(np.abs(last[0] - want[29]).max()) < TOLERANCE
    with pytest.raises(Invalid, match="at most 8 back"):
        session.truncate(12)                                                   # further back than the ring allows
    with pytest.raises(Invalid):
        session.truncate(31)                                                   # ahead of the session
    session.truncate(24)
    for i, row in enumerate(model.feed(session, ids[24:27], ALL)):
        assert float(np.abs(row - want[24 + i]).max()) < TOLERANCE, f"position {24 + i}"
    # a smaller session for a side conversation, started over once
    side = model.session_holding(20)
    assert side.capacity() == 32
    with pytest.raises(Invalid, match="exceed the session's 32"):
        model.feed(side, ids[:33], LAST)
    for _ in range(2):
        row = model.feed(side, ids[:12], LAST)[0]
        assert float(np.abs(row - want[11]).max()) < TOLERANCE
        side.reset()
    session.free()
    side.free()
    model.free()


def test_a_model_file_that_is_not_the_shape_it_claims_is_refused(fixture, gpu, tmp_path):
    path = fixture[0]
    raw = open(path, "rb").read()
    wrong = tmp_path / "wrong.gguf"
    wrong.write_bytes(raw.replace(b"blk.2.attn_sinks.weight", b"blk.2.attn_sinkz.weight"))
    with pytest.raises(Invalid, match="blk.2.attn_sinks.weight is missing"):
        GpuModel.load(str(wrong), 8, 64, gpu)
    with pytest.raises(Invalid, match="positive"):
        GpuModel.load(path, 0, 64, gpu)
