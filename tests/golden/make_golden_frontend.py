"""Generates tests/golden/golden_frontend.npz from the REFERENCE's own code: the text encoder
(encode_text, src/graph.c:709-748 in mynah-tts) and the codec decoder (decode_codec,
src/graph.c:2640-2780) -- the two ends of a request around the decoder loop.

Run where a mynah-tts checkout is mounted (compiled into oracle/_ref by `make -C oracle ref`):

    python tests/golden/make_golden_frontend.py

Everything stored is an output of the reference's sources (strict host build, `-std=c11 -O2`)
on seeded synthetic weights (mynah_tts_b200.synth.add_encoder / add_codec):
  * text encoder, tiny shape (2 layers, width 192), 1 / 19 / 40 ids: the states;
  * codec at the reference's fixed size (base 864), 1 and 3 frames: the samples.
"""
from __future__ import annotations

import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from mynah_tts_b200 import synth  # noqa: E402
from oracle import oracle as O  # noqa: E402

OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden_frontend.npz")
ENCODER_SEED, ENCODER_COUNTS, IDS_SEED = 91, (1, 19, 40), 5
CODEC_SEED, CODEC_FRAMES, CODES_SEED = 7, (1, 3), 5


def bare_model(tensors_from):
    """A model whose file holds only what `tensors_from` draws into it."""
    base = synth.make_model(synth.TINY, seed=3)
    model = type(base)(shape=base.shape, seed=base.seed, tensors={})
    tensors_from(model)
    return model


def encoder_ids(count):
    return np.random.default_rng([IDS_SEED, count]).integers(0, synth.TINY_ENCODER.vocab, size=count).astype(np.int32)


def main():
    assert O.have_ref("strict"), "build the reference first: make -C oracle ref"
    out = {}
    model = bare_model(lambda m: synth.add_encoder(m, synth.TINY_ENCODER, seed=ENCODER_SEED))
    rm = O.RefModel(model, O.F32, "strict")
    for count in ENCODER_COUNTS:
        out[f"encoder_{count}"] = rm.encode_text(synth.TINY_ENCODER, encoder_ids(count))
    rm.close()
    shape = synth.CodecShape()
    model = bare_model(lambda m: synth.add_codec(m, shape, seed=CODEC_SEED))
    rm = O.RefModel(model, O.F32, "strict")
    for frames in CODEC_FRAMES:
        out[f"codec_{frames}"] = rm.decode_codec(synth.make_codec_codes(shape, CODES_SEED, frames))
    rm.close()
    np.savez_compressed(OUT, **out)
    print("wrote", OUT, os.path.getsize(OUT), "bytes")


if __name__ == "__main__":
    main()
