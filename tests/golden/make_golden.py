"""Generates tests/golden/golden.npz from the REFERENCE's own code.

Run where a mynah-tts checkout is mounted (it is compiled into oracle/_ref by
`make -C oracle ref`):

    python tests/golden/make_golden.py

Everything stored here is an output of the reference's sources built with the
host flags of its CUDA variant (`-std=c11 -O2`, no SIMD, no -ffast-math) on
seeded synthetic weights (mynah_tts_b200/synth.py); nothing is produced by this
repository's own arithmetic.  The fixtures pin oracle/mynah_oracle.c on
machines without a reference checkout and give the GPU tests token streams and
hidden states to compare against at sizes the CPU needs minutes for.
"""
from __future__ import annotations

import os
import sys
import time
import zlib

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from mynah_tts_b200 import synth  # noqa: E402
from oracle import oracle as O  # noqa: E402

OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden.npz")
QT = {"f32": O.F32, "int8": O.INT8, "int4": O.INT4}
KEEP_HIDDEN = (0, 1, 63, 64, 255, 256, 511)


def crc(a: np.ndarray) -> np.uint32:
    return np.uint32(zlib.crc32(np.ascontiguousarray(a).tobytes()))


def margins(logits: np.ndarray, shape, allow_eos: bool) -> float:
    """Smallest top-1/top-2 gap over the tables, among allowed candidates."""
    worst = np.inf
    for t in range(shape.tables):
        cand = list(range(shape.codebook_size)) + ([shape.eos_id] if allow_eos else [])
        v = np.sort(logits[t, cand])
        worst = min(worst, float(v[-1] - v[-2]))
    return worst


def greedy(model, rm, memory, codes0, frames, min_frames, capacity, keep=()):
    """Frame-by-frame greedy decode through the reference: embed (its
    embed_audio_frame), decoder_step_batch, heads; returns tokens, the margin
    per frame and selected hidden states."""
    s = model.shape
    rd = rm.new_decoder(memory, capacity)
    codes = codes0.astype(np.uint32).copy()
    toks = np.zeros((frames, s.tables), np.uint32)
    marg = np.zeros((frames,), np.float32)
    hid = {}
    import ctypes as C
    lib = rm.ref.lib
    lib.ref_embed_audio_frame.argtypes = [C.c_void_p, O.c_uint_p, C.c_size_t, C.c_size_t,
                                          O.c_float_p, C.c_char_p, C.c_size_t]
    cb = s.tables // 2
    n = frames
    for f in range(frames):
        # stream = fs * codebooks + codebook  ->  codes[codebook * 2 + fs]
        fc = np.zeros((s.tables,), np.uint32)
        for fs in range(2):
            for c in range(cb):
                fc[c * 2 + fs] = codes[fs * cb + c]
        row = np.empty((s.width,), np.float32)
        err = C.create_string_buffer(256)
        assert lib.ref_embed_audio_frame(rm.handle, fc.ctypes.data_as(O.c_uint_p), 2, 0,
                                         O._fp(row), err, 256) == 0, err.value
        h = rd.step(row)
        allow = f >= min_frames
        tok, logits = rm.heads_argmax(h, allow)
        toks[f] = tok
        marg[f] = margins(logits, s, allow)
        if f in keep:
            hid[f] = h.copy()
        codes = np.where(tok < s.codebook_size, tok, 0).astype(np.uint32)
        if (tok == s.eos_id).any():
            n = f + 1
            break
    kv_crc = crc(rd.self_k[:, :n]) ^ crc(rd.self_v[:, :n])
    rd.close()
    return toks[:n], marg[:n], hid, kv_crc


def main():
    assert O.have_ref("strict"), "build the reference first: make -C oracle ref"
    ref = O.Ref.get("strict")
    rc, msg = ref.self_tests()
    assert rc == 0, msg
    out = {}
    t0 = time.time()
    # ---- single op (the [3072,768] LayerNorm + linear case) -------------------
    x, w, gain, bias = synth.make_linear_case(seed=1)
    nrm = ref.layernorm(x, gain)
    out["linear_ln"] = nrm[0]
    q8, s8 = ref.quantize_weight_int8(w)
    q4, s4 = ref.quantize_weight_int4(w)
    out["linear_pack_crc"] = np.array([crc(q8), crc(s8), crc(q4), crc(s4)], np.uint32)
    qa, sx = ref.quantize_act_int8(nrm[0])
    out["linear_act_q"] = qa
    out["linear_act_sx"] = np.float32(sx)
    for name, qt in QT.items():
        out[f"linear_y_{name}"] = ref.qmat_linear(qt, w, nrm, bias)[0]
    # ---- tiny decoder: every mode, teacher-forced frames + greedy tokens --------
    shape = synth.TINY
    model = synth.make_model(shape, seed=3)
    memory = synth.make_memory(shape, seed=5)
    forced = synth.make_codes(shape, seed=7, frames=10)
    start = synth.make_codes(shape, seed=9, frames=1)[0]
    for name, qt in QT.items():
        rm = O.RefModel(model, qt, "strict")
        rd = rm.new_decoder(memory, 64)
        if name == "f32":
            out["tiny_cross_k"] = rd.cross_k.copy()
            out["tiny_cross_v"] = rd.cross_v.copy()
        pm = O.PortModel(model, qt)   # only for the embedding gather (checked against the ref below)
        hidden = np.zeros((10, shape.width), np.float32)
        tokens = np.zeros((10, shape.tables), np.uint32)
        for f in range(10):
            hidden[f] = rd.step(pm.embed_frame(forced[f]))
            tokens[f], _ = rm.heads_argmax(hidden[f], True)
        out[f"tiny_{name}_forced_hidden"] = hidden
        out[f"tiny_{name}_forced_tokens"] = tokens
        out[f"tiny_{name}_forced_kv_crc"] = crc(rd.self_k[:, :10]) ^ crc(rd.self_v[:, :10])
        # per-layer hidden states of one further step (position 10)
        row = pm.embed_frame(forced[0])
        per_layer = np.zeros((shape.layers, shape.width), np.float32)
        for n in range(1, shape.layers + 1):
            rd.length = 10
            rd.set_layers(n)
            per_layer[n - 1] = rd.step(row)
        out[f"tiny_{name}_layers"] = per_layer
        rd.close()
        toks, marg, _, kv = greedy(model, rm, memory, start, 64, 4, 80)
        out[f"tiny_{name}_greedy_tokens"] = toks
        out[f"tiny_{name}_greedy_margin"] = marg
        rm.close()
        pm.close()
        print(f"tiny {name}: {len(toks)} greedy frames, {time.time() - t0:.0f}s", flush=True)
    # ---- Magpie-357M shape: 512 greedy frames --------------------------------
    shape = synth.MAGPIE_357M
    plan = [("int8", 21), ("int8", 22), ("int8", 23), ("f32", 21), ("int4", 21)]
    models = {}
    for name, seed in plan:
        if seed not in models:
            models[seed] = synth.make_model(shape, seed=seed)
        model = models[seed]
        memory = synth.make_memory(shape, seed=seed + 100)
        start = synth.make_codes(shape, seed=seed + 200, frames=1)[0]
        rm = O.RefModel(model, QT[name], "strict")
        toks, marg, hid, kv = greedy(model, rm, memory, start, 512, 10 ** 6, 520, keep=KEEP_HIDDEN)
        rm.close()
        key = f"full_{name}_s{seed}"
        out[f"{key}_tokens"] = toks.astype(np.uint16)
        out[f"{key}_margin"] = marg
        out[f"{key}_hidden"] = np.stack([hid[f] for f in KEEP_HIDDEN])
        out[f"{key}_kv_crc"] = kv
        print(f"{key}: done, min margin {marg.min():.2e}, {time.time() - t0:.0f}s", flush=True)
        np.savez_compressed(OUT, **out)
    np.savez_compressed(OUT, **out)
    print("wrote", OUT, os.path.getsize(OUT), "bytes")


if __name__ == "__main__":
    main()
