"""The text encoder (encode_text, src/graph.c:709-748) on the GPU against the CPU restatement,
which tests/test_oracle.py pins bit for bit against the reference's own encode_text."""
import numpy as np
import pytest

from conftest import rel_err
from mynah_tts_b200 import synth
from mynah_tts_b200.backend import Backend, TextEncoder
from oracle import oracle as O

pytestmark = pytest.mark.gpu

WIDE = synth.EncoderShape(layers=2, width=768, vocab=96, max_length=160)


@pytest.mark.parametrize("shape,counts", [(synth.TINY_ENCODER, (1, 2, 19, 33, 48)), (WIDE, (1, 31, 97, 160))],
                         ids=["tiny", "width768"])
@pytest.mark.parametrize("strict,no_tc", [pytest.param(True, False, id="strict"),
                                           pytest.param(False, False, id="fast-tensor-core"),
                                           pytest.param(False, True, id="fast-simt")])
def test_text_encoder_matches_oracle(shape, counts, strict, no_tc, monkeypatch):
    """Strict: sequential f32 sums, bit for bit.  Fast: the layer's products on the tensor cores
    over split f16 planes (the kernel-3 convolutions without an unfolded copy), or SIMT FMAs
    with MYNAH_B200_NO_TC."""
    if no_tc:
        monkeypatch.setenv("MYNAH_B200_NO_TC", "1")
    tensors = synth.add_encoder(None, shape, seed=91)
    be = Backend("int8", strict=strict)          # the weight format must not matter: the encoder is f32
    enc = TextEncoder(be, tensors, shape)
    rng = np.random.default_rng(5)
    for count in counts:
        ids = rng.integers(0, shape.vocab, size=count).astype(np.int32)
        want = O.Port.get().encode_text(tensors, shape, ids)
        got = enc.encode(ids)
        if strict:
            assert np.array_equal(got, want), count          # bit for bit
        else:
            assert rel_err(got, want) < 2e-4, count          # f32 sums in another order
    # a second pass over the first length: no state is carried between requests
    ids = rng.integers(0, shape.vocab, size=counts[1]).astype(np.int32)
    a = enc.encode(ids)
    assert np.array_equal(a, enc.encode(ids))
    enc.close(); be.close()


def test_text_encoder_refusals():
    shape = synth.TINY_ENCODER
    tensors = synth.add_encoder(None, shape, seed=3)
    be = Backend("f32", strict=True)
    enc = TextEncoder(be, tensors, shape)
    with pytest.raises(RuntimeError, match="text length"):
        enc.encode(np.zeros(shape.max_length + 1, np.int32))
    with pytest.raises(RuntimeError, match="text length"):
        enc.encode(np.zeros(0, np.int32))
    with pytest.raises(RuntimeError, match="outside vocabulary"):
        enc.encode(np.array([0, shape.vocab], np.int32))
    with pytest.raises(RuntimeError, match="outside vocabulary"):
        enc.encode(np.array([-1], np.int32))
    assert enc.encode(np.array([1, 2, 3], np.int32)).shape == (3, shape.width)
    enc.close(); be.close()
