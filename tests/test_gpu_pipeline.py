"""A whole request on the GPU -- text ids -> text encoder -> cross K/V of the decoder slot ->
greedy decoder frames -> codec -> audio samples -- against the same chain of CPU restatements
(each pinned against the reference's own function: encode_text, decoder_cache_init /
decoder_step_batch with the logit heads, decode_codec).  Strict mode, full size, two requests
of different text lengths stepped together: every stage bit for bit."""
import numpy as np
import pytest

from mynah_tts_b200 import synth
from mynah_tts_b200.backend import Backend, Codec, Decoder, TextEncoder
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def test_text_to_audio_matches_the_cpu_chain():
    shape = synth.MAGPIE_357M
    model = synth.make_model(shape, seed=51)
    eshape = synth.EncoderShape(layers=2, max_length=shape.memory_length)      # two layers keep the CPU side short
    etensors = synth.add_encoder(None, eshape, seed=52)
    cshape = synth.CodecShape()
    ctensors = synth.add_codec(None, cshape, seed=53)
    frames = 5
    rng = np.random.default_rng(54)
    texts = [rng.integers(0, eshape.vocab, size=n).astype(np.int32) for n in (19, 40)]
    start = synth.make_codes(shape, seed=55, frames=2)                          # one start frame per request

    be = Backend("int8", strict=True)
    enc = TextEncoder(be, etensors, eshape)
    dec = Decoder(be, model, capacity=16, slots=2)
    codec = Codec(be, ctensors, cshape, max_frames=frames)
    pm = O.PortModel(model, O.INT8)
    port = O.Port.get()

    # ---- text encoder, then the slots' cross K/V made on the device from the states
    streams = []
    for slot, ids in enumerate(texts):
        states = enc.encode(ids)
        want_states = port.encode_text(etensors, eshape, ids)
        assert np.array_equal(states, want_states), slot
        dec.slot_prefill(slot, states)
        streams.append(pm.new_stream(want_states, 16))
        ck, cv = dec.slot_read_cross(slot)
        n = len(ids)
        assert np.array_equal(ck[:, :n], streams[slot].cross_k) and np.array_equal(cv[:, :n], streams[slot].cross_v)

    # ---- greedy frames, both requests stepped together
    tokens, eos, _, _ = dec.greedy([0, 1], start, frames, min_frames=10 ** 6)
    assert tokens.shape == (frames, 2, shape.tables) and (eos == -1).all()
    for slot in range(2):
        codes = start[slot].copy()
        for f in range(frames):
            want, _, _ = streams[slot].greedy_frame(codes, allow_eos=False)
            assert np.array_equal(tokens[f, slot], want), (slot, f)
            codes = np.where(want < shape.codebook_size, want, 0).astype(np.uint32)

    # ---- codec: the 8 codebook indices of every frame are the FSQ indices of the 8 groups
    for slot in range(2):
        fsq = np.ascontiguousarray(np.minimum(tokens[:, slot, :cshape.groups], cshape.fsq_codes - 1).T)   # [groups, frames]
        samples = codec.decode(fsq)
        want = port.codec_decode(ctensors, cshape, fsq)
        assert samples.shape == (frames * 1024,)
        assert np.array_equal(samples, want), slot
    for st in streams:
        st.close()
    pm.close(); codec.close(); dec.close(); enc.close(); be.close()
