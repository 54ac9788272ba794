"""GPU parity tests of the local transformer and its sampler (src/graph.c:806-1656 in
mynah-tts) through the C ABI.

Strict mode must reproduce the reference bit for bit: hidden rows, greedy picks,
top-k draws (so the xorshift64 states too), stored codes and EOS reports, at any
batch.  The checker is the CPU port (oracle/mynah_oracle.c) and the fixtures
generated from the reference's own functions (tests/golden/golden_local.npz)."""
import os
import sys

import numpy as np
import pytest

from mynah_tts_b200 import synth
from oracle import oracle as O

pytestmark = pytest.mark.gpu

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
from make_golden_local import TINY_LANES  # noqa: E402

GOLDEN_LOCAL = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "golden_local.npz")
QT = {"f32": O.F32, "int8": O.INT8, "int4": O.INT4}


@pytest.fixture(scope="module")
def gl():
    return np.load(GOLDEN_LOCAL)


@pytest.fixture(scope="module")
def tiny_local_model():
    return synth.make_model(synth.TINY_LOCAL, seed=3)


def make(name, model, strict=True, slots=8, capacity=40):
    from mynah_tts_b200.backend import Backend, Decoder
    be = Backend(name, strict=strict)
    return be, Decoder(be, model, capacity=capacity, slots=slots)


@pytest.mark.parametrize("name", ["int8", "int4", "f32"])
def test_local_frame_matches_reference_fixture(name, gl, tiny_local_model):
    shape = synth.TINY_LOCAL
    be, dec = make(name, tiny_local_model)
    assert dec.has_local
    rows = gl["tiny_rows"]
    codes, values, saw, eos, rng = dec.local_frame(rows, TINY_LANES)
    if name != "f32":      # f32 products are equal to rounding only; picks may differ on near ties
        assert np.array_equal(codes, gl[f"tiny_{name}_frame_codes"])
        assert np.array_equal(saw, gl[f"tiny_{name}_frame_saw_eos"])
        assert np.array_equal(eos, gl[f"tiny_{name}_frame_eos_frame"])
        assert np.array_equal(np.array(rng, np.uint64), gl[f"tiny_{name}_frame_rng"])
    assert np.array_equal(codes, np.where(values < shape.codebook_size, values, 0))
    for b, (_, _, _, allow) in enumerate(TINY_LANES):
        if not allow:
            assert not (values[b] == shape.eos_id).any()
    dec.close(); be.close()


@pytest.mark.parametrize("name", ["int8", "int4"])
def test_local_frame_does_not_depend_on_batch(name, tiny_local_model):
    """A request's frame is the same alone and among 2, 5, 16 and 17 others (the
    reference batches the projections across requests, src/graph.c:1227-1233)."""
    shape = synth.TINY_LOCAL
    rng = np.random.default_rng(12)
    rows = rng.normal(0, 1, size=(17, shape.width)).astype(np.float32)
    lanes = [(0.8, 12, 1000 + b, 1) if b % 3 else (0.0, 0, 0, 1) for b in range(17)]
    pm = O.PortModel(tiny_local_model, QT[name])
    pl = O.PortLocal(pm, 16)
    for strict in (True, False):
        from mynah_tts_b200.backend import Backend, Decoder
        be = Backend(name, strict=strict)
        dec = Decoder(be, tiny_local_model, capacity=24, slots=17)
        solo = [dec.local_frame(rows[b:b + 1], lanes[b:b + 1]) for b in range(17)]
        for batch in (2, 5, 16, 17):
            codes, values, saw, eos, states = dec.local_frame(rows[:batch], lanes[:batch])
            for b in range(batch):
                assert np.array_equal(codes[b], solo[b][0][0]), (strict, batch, b)
                assert np.array_equal(values[b], solo[b][1][0])
                assert saw[b] == solo[b][2][0] and eos[b] == solo[b][3][0] and states[b] == solo[b][4][0]
        if strict:
            for b in range(17):
                c, v, s_, e, r = pl.frame(rows[b], *lanes[b][:3], bool(lanes[b][3]))
                assert np.array_equal(solo[b][0][0], c) and np.array_equal(solo[b][1][0], v)
                assert bool(solo[b][2][0]) == s_ and solo[b][3][0] == e and solo[b][4][0] == r
        dec.close(); be.close()
    pl.close(); pm.close()


@pytest.mark.parametrize("name", ["int8", "int4"])
def test_generation_loop_matches_reference_fixture(name, gl, tiny_local_model):
    """embed -> decoder step -> local frame, 24 frames, four requests stepped together
    with mixed greedy / top-k settings: tokens, EOS frames and rng states."""
    shape = synth.TINY_LOCAL
    be, dec = make(name, tiny_local_model, capacity=32, slots=4)
    pm = O.PortModel(tiny_local_model, QT[name])
    for b in range(4):
        st = pm.new_stream(synth.make_memory(shape, seed=300 + b), 8)
        dec.slot_load(b, st.cross_k.copy(), st.cross_v.copy())
        st.close()
    start = np.stack([synth.make_codes(shape, seed=400 + b, frames=1)[0] for b in range(4)])
    lanes = TINY_LANES[:4]
    tokens, eos, ms, last, states = dec.generate([0, 1, 2, 3], start, 24, min_frames=4, samplers=lanes)
    want = gl[f"tiny_{name}_gen_codes"]
    stored = np.where(tokens < shape.codebook_size, tokens, 0)
    assert np.array_equal(stored, want)
    assert np.array_equal(last, want[-1])
    assert np.array_equal(np.array(states, np.uint64), gl[f"tiny_{name}_gen_rng"])
    saw = gl[f"tiny_{name}_gen_saw_eos"]
    for b in range(4):
        first = np.flatnonzero(saw[:, b])
        assert eos[b] == (first[0] if first.size else -1)
    # ragged lengths: a lane that stops early leaves the others' streams unchanged
    for b in range(4):
        dec.slot_set_length(b, 0)
    t2, _, _, _, _ = dec.generate([0, 1, 2, 3], start, [24, 7, 24, 13], min_frames=4, samplers=lanes)
    assert np.array_equal(t2[:, 0], tokens[:, 0]) and np.array_equal(t2[:, 2], tokens[:, 2])
    assert np.array_equal(t2[:7, 1], tokens[:7, 1]) and not t2[7:, 1].any()
    assert np.array_equal(t2[:13, 3], tokens[:13, 3])
    pm.close(); dec.close(); be.close()


def test_full_size_generation_matches_reference_fixture(gl):
    """Magpie-357M shape with 16 stacked streams and 2 local layers, int8, strict:
    12 frames for one greedy and two sampling requests."""
    shape = synth.MAGPIE_357M_LOCAL
    model = synth.make_model(shape, seed=31)
    be, dec = make("int8", model, capacity=20, slots=3)
    pm = O.PortModel(model, O.INT8)
    for b in range(3):
        st = pm.new_stream(synth.make_memory(shape, seed=500 + b), 4)
        dec.slot_load(b, st.cross_k.copy(), st.cross_v.copy())
        st.close()
    pm.close()
    start = np.stack([synth.make_codes(shape, seed=600 + b, frames=1)[0] for b in range(3)])
    lanes = [(0.0, 0, 1, 1), (0.6, 80, 0xABCDEF, 1), (1.0, 40, 424242, 1)]
    tokens, eos, ms, last, states = dec.generate([0, 1, 2], start, 12, min_frames=2, samplers=lanes)
    stored = np.where(tokens < shape.codebook_size, tokens, 0)
    assert np.array_equal(stored, gl["full_int8_gen_codes"].astype(np.uint32))
    assert np.array_equal(np.array(states, np.uint64), gl["full_int8_gen_rng"])
    dec.close(); be.close()


def test_full_size_top_k_with_tied_logits_matches_port():
    """The sampler's top-k on 2048 candidates (register-resident warp sorts and top-128
    merges) against the CPU port, strict, with exact ties among the logits: half of every
    table's projection rows are copies of other rows, so equal logits sit inside and at the
    edge of the top k and the earlier index has to win.  k = 2, 40, 80, 128 take the
    merge path, k = 200 the block-wide sort."""
    import copy
    shape = synth.MAGPIE_357M_LOCAL
    model = copy.copy(synth.make_model(shape, seed=33))
    model.tensors = dict(model.tensors)
    rng = np.random.default_rng(5)
    for t in range(shape.tables):
        w = model.tensors[f"local_transformer_out_projections.{t}.weight"].copy()
        b = model.tensors[f"local_transformer_out_projections.{t}.bias"].copy()
        src = rng.permutation(shape.codebook_size)[:1000]
        dst = rng.permutation(shape.codebook_size)[:1000]
        w[dst] = w[src]
        b[dst] = b[src]
        model.tensors[f"local_transformer_out_projections.{t}.weight"] = w
        model.tensors[f"local_transformer_out_projections.{t}.bias"] = b
    rows = rng.normal(0, 1, size=(5, shape.width)).astype(np.float32)
    lanes = [(0.7, 80, 11, 1), (1.0, 128, 12, 1), (0.5, 40, 13, 0), (1.3, 200, 14, 1), (0.9, 2, 15, 1)]
    be, dec = make("int8", model, strict=True, slots=5, capacity=8)
    codes, values, saw, eos, states = dec.local_frame(rows, lanes)
    pm = O.PortModel(model, O.INT8)
    pl = O.PortLocal(pm, 256)         # room for the largest top-k of the lanes
    for b in range(5):
        c, v, s_, e, r = pl.frame(rows[b], *lanes[b][:3], bool(lanes[b][3]))
        assert np.array_equal(codes[b], c), b
        assert np.array_equal(values[b], v), b
        assert bool(saw[b]) == s_ and eos[b] == e and states[b] == r, b
    pl.close(); pm.close()
    dec.close(); be.close()


def test_local_requests_are_refused_without_local_weights(tiny_model):
    from mynah_tts_b200.backend import Backend, Decoder
    from mynah_tts_b200.capi import MynahB200Error
    be = Backend("int8", strict=True)
    dec = Decoder(be, tiny_model, capacity=8, slots=2)
    assert not dec.has_local
    with pytest.raises(MynahB200Error):
        dec.local_frame(np.zeros((1, synth.TINY.width), np.float32))
    with pytest.raises(MynahB200Error):
        dec.generate([0], np.zeros((1, synth.TINY.tables), np.uint32), 2)
    dec.close(); be.close()


def test_continuous_batching_gives_each_request_its_solo_result(tiny_local_model):
    """Eight requests over three slots: a request enters when a slot frees up, leaves on
    EOS or at its frame limit, and its codes are what the reference's functions give
    for the request alone (port loop: embed -> decoder step -> local frame)."""
    from mynah_tts_b200.backend import Backend, Decoder
    shape = synth.TINY_LOCAL
    pm = O.PortModel(tiny_local_model, O.INT8)
    reqs, want = [], []
    for i in range(8):
        memory = synth.make_memory(shape, seed=700 + i)
        start = synth.make_codes(shape, seed=800 + i, frames=1)[0]
        sampler = (0.9, 12, 5000 + i) if i % 2 else (0.0, 0, 0)
        max_frames, min_frames = 6 + 3 * i, 2 + (i % 3)
        reqs.append({"memory": memory, "start_codes": start, "max_frames": max_frames,
                     "min_frames": min_frames, "sampler": sampler})
        st = pm.new_stream(memory, max_frames + 2)
        pl = O.PortLocal(pm, 16)
        codes, rng, out, eos_at = start.copy(), sampler[2], [], -1
        for f in range(max_frames):
            hidden = st.step(pm.embed_frame(codes))
            codes, _, saw, _, rng = pl.frame(hidden, sampler[0], sampler[1], rng, f >= min_frames)
            out.append(codes.copy())
            if saw:
                eos_at = f
                break
        want.append((np.stack(out), eos_at, rng))
        st.close(); pl.close()
    pm.close()
    be = Backend("int8", strict=True)
    dec = Decoder(be, tiny_local_model, capacity=40, slots=3)
    results, steps = dec.serve(reqs)
    for i, (codes, eos_frame, admitted_at, rng) in enumerate(results):
        assert np.array_equal(codes, want[i][0]), i
        assert eos_frame == want[i][1] and rng == want[i][2]
        assert (admitted_at == 0) == (i < 3)
    total = sum(len(w[0]) for w in want)
    assert max(len(w[0]) for w in want) <= steps < total      # requests overlapped
    dec.close(); be.close()
