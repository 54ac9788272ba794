"""Generates tests/golden/golden_local.npz from the REFERENCE's own code: the
local transformer and its sampler (src/graph.c:806-1656 in mynah-tts).

Run where a mynah-tts checkout is mounted (compiled into oracle/_ref by
`make -C oracle ref`):

    python tests/golden/make_golden_local.py

Everything stored is an output of the reference's sources (strict host build,
`-std=c11 -O2`) on seeded synthetic weights; see make_golden.py.  Cases:
  * tiny shape, each weight format: one local step per request (hidden row),
    stacked frames for six requests with mixed greedy / top-k settings;
  * tiny shape: a generation loop (embed -> decoder step -> local frame) of 24
    frames for four requests stepped together;
  * full-size shape (16 stacked streams, 2 local layers), int8: 12 frames of the
    same loop for three requests, one greedy and two sampling.
"""
from __future__ import annotations

import os
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from mynah_tts_b200 import synth  # noqa: E402
from oracle import oracle as O  # noqa: E402

OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden_local.npz")
QT = {"f32": O.F32, "int8": O.INT8, "int4": O.INT4}

# per-request sampler settings of the tiny frame case: temperature, top-k, rng seed, EOS allowed
TINY_LANES = [(0.0, 0, 1, 1), (0.7, 8, 0x1234, 1), (1.3, 5, 0x9E3779B97F4A7C15, 0),
              (0.0, 0, 5, 0), (0.5, 56, 77, 1), (2.0, 64, 99, 1)]


def generate(rm, model, memories, start_codes, frames, lanes, min_frames, capacity):
    """The reference's synthesis loop without the codec: per frame embed the stored
    codes, one batched decoder step, one batched local frame."""
    shape = model.shape
    batch = len(memories)
    decoders = [rm.new_decoder(m, capacity) for m in memories]
    top = max(min(k, shape.vocab) for _, k, _, _ in lanes)
    locals_ = [rm.new_local(top) for _ in range(batch)]
    codes = np.array(start_codes, np.uint32).copy()
    rng = [seed for _, _, seed, _ in lanes]
    all_codes = np.zeros((frames, batch, shape.tables), np.uint32)
    hidden = np.zeros((frames, batch, shape.width), np.float32)
    saw = np.zeros((frames, batch), np.int32)
    for f in range(frames):
        rows = np.stack([rm.embed_frame(codes[b]) for b in range(batch)])
        out = rm.step_batch(decoders, rows)
        hidden[f] = out
        allow = [int(f >= min_frames)] * batch
        codes, s, _, rng = rm.local_frame(locals_, out, [t for t, _, _, _ in lanes],
                                          [k for _, k, _, _ in lanes], rng, allow)
        all_codes[f] = codes
        saw[f] = s
    for d in decoders:
        d.close()
    for l in locals_:
        l.close()
    return all_codes, hidden, saw, np.array(rng, np.uint64)


def main():
    assert O.have_ref("strict"), "build the reference first: make -C oracle ref"
    out = {}
    t0 = time.time()
    shape = synth.TINY_LOCAL
    model = synth.make_model(shape, seed=3)
    rng = np.random.default_rng(41)
    rows = rng.normal(0.0, 1.0, size=(len(TINY_LANES), shape.width)).astype(np.float32)
    out["tiny_rows"] = rows
    for name, qt in QT.items():
        rm = O.RefModel(model, qt, "strict")
        locals_ = [rm.new_local(shape.vocab) for _ in TINY_LANES]
        out[f"tiny_{name}_step"] = rm.local_step_batch(locals_, rows)
        for l in locals_:
            l.length = 0
        codes, saw, eos, rng_out = rm.local_frame(
            locals_, rows, [t for t, _, _, _ in TINY_LANES], [k for _, k, _, _ in TINY_LANES],
            [s for _, _, s, _ in TINY_LANES], [a for _, _, _, a in TINY_LANES])
        out[f"tiny_{name}_frame_codes"] = codes
        out[f"tiny_{name}_frame_saw_eos"] = saw.astype(np.int32)
        out[f"tiny_{name}_frame_eos_frame"] = eos.astype(np.int64)
        out[f"tiny_{name}_frame_rng"] = np.array(rng_out, np.uint64)
        for l in locals_:
            l.close()
        # generation loop, four requests
        lanes = TINY_LANES[:4]
        memories = [synth.make_memory(shape, seed=300 + b) for b in range(4)]
        start = np.stack([synth.make_codes(shape, seed=400 + b, frames=1)[0] for b in range(4)])
        gc, gh, gs, gr = generate(rm, model, memories, start, 24, lanes, 4, 32)
        out[f"tiny_{name}_gen_codes"] = gc
        out[f"tiny_{name}_gen_hidden"] = gh[[0, 1, 23]]
        out[f"tiny_{name}_gen_saw_eos"] = gs
        out[f"tiny_{name}_gen_rng"] = gr
        rm.close()
        print(f"tiny {name}: {time.time() - t0:.0f}s", flush=True)
    # ---- full size, int8 ---------------------------------------------------------
    shape = synth.MAGPIE_357M_LOCAL
    model = synth.make_model(shape, seed=31)
    rm = O.RefModel(model, O.INT8, "strict")
    lanes = [(0.0, 0, 1, 1), (0.6, 80, 0xABCDEF, 1), (1.0, 40, 424242, 1)]
    memories = [synth.make_memory(shape, seed=500 + b) for b in range(3)]
    start = np.stack([synth.make_codes(shape, seed=600 + b, frames=1)[0] for b in range(3)])
    gc, gh, gs, gr = generate(rm, model, memories, start, 12, lanes, 2, 20)
    out["full_int8_gen_codes"] = gc.astype(np.uint16)
    out["full_int8_gen_hidden"] = gh[[0, 11]]
    out["full_int8_gen_saw_eos"] = gs
    out["full_int8_gen_rng"] = gr
    rm.close()
    print(f"full int8: {time.time() - t0:.0f}s", flush=True)
    np.savez_compressed(OUT, **out)
    print("wrote", OUT, os.path.getsize(OUT), "bytes")


if __name__ == "__main__":
    main()
