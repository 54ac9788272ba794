"""The CPU restatements of the text encoder and the codec decoder against outputs of the
reference's own encode_text / decode_codec (tests/golden/golden_frontend.npz, made by
tests/golden/make_golden_frontend.py), and against the compiled reference where it is present."""
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
import make_golden_frontend as G  # noqa: E402
from mynah_tts_b200 import synth  # noqa: E402
from oracle import oracle as O  # noqa: E402

GOLDEN = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "golden_frontend.npz"))


def test_port_text_encoder_equals_golden():
    enc = synth.TINY_ENCODER
    tensors = synth.add_encoder(None, enc, seed=G.ENCODER_SEED)
    for count in G.ENCODER_COUNTS:
        got = O.Port.get().encode_text(tensors, enc, G.encoder_ids(count))
        assert np.array_equal(got, GOLDEN[f"encoder_{count}"]), count


def test_port_codec_equals_golden():
    """FSQ de-index, causal convolutions as unfolded scalar products, grouped transposed
    convolution, half-Snake in the CPU backend's reciprocal form, residual layers, clip:
    bit for bit at the reference's fixed size."""
    shape = synth.CodecShape()
    tensors = synth.add_codec(None, shape, seed=G.CODEC_SEED)
    for frames in G.CODEC_FRAMES[:1]:
        codes = synth.make_codec_codes(shape, G.CODES_SEED, frames)
        got = O.Port.get().codec_decode(tensors, shape, codes)
        want = GOLDEN[f"codec_{frames}"]
        assert got.shape == want.shape == (frames * 1024,)
        assert np.array_equal(got, want)
        assert np.abs(want).max() <= 1.0 and want.std() > 0.05      # a live signal, clipped


def test_port_codec_equals_reference():
    if not O.have_ref("strict"):
        pytest.skip("compiled reference absent")
    shape = synth.CodecShape()
    model = G.bare_model(lambda m: synth.add_codec(m, shape, seed=11))
    rm = O.RefModel(model, O.F32, "strict")
    codes = synth.make_codec_codes(shape, 9, 2)
    want = rm.decode_codec(codes)
    got = O.Port.get().codec_decode(model.tensors, shape, codes)
    assert np.array_equal(got, want)
    rm.close()


def test_port_codec_is_causal_and_stagewise_consistent():
    """Every operation of the codec is causal, so the samples of the first frames do not
    depend on later frames; and the stage outputs chain (small shape)."""
    shape = synth.TINY_CODEC
    tensors = synth.add_codec(None, shape, seed=2)
    codes = synth.make_codec_codes(shape, 4, 5)
    whole = O.Port.get().codec_decode(tensors, shape, codes)
    head = O.Port.get().codec_decode(tensors, shape, codes[:, :2])
    assert np.array_equal(whole[:2 * 1024], head)
    pre = O.Port.get().codec_decode(tensors, shape, codes, stop_after=1)
    assert pre.shape == (shape.base, 5)
    last = O.Port.get().codec_decode(tensors, shape, codes, stop_after=6)
    assert last.shape == (shape.base // 32, 5 * 1024)
