"""CPU tests of the local-transformer part of the parity checker: the C
restatement (oracle/mynah_oracle.c, orc_local_*) against fixtures generated from
the reference's own sample_local_frame_batch / local_step_batch
(tests/golden/make_golden_local.py), and against the compiled reference bit for
bit where oracle/_ref exists."""
import os
import sys

import numpy as np
import pytest

from mynah_tts_b200 import synth
from oracle import oracle as O

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
from make_golden_local import TINY_LANES  # noqa: E402

QT = {"f32": O.F32, "int8": O.INT8, "int4": O.INT4}
GOLDEN_LOCAL = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "golden_local.npz")
needs_ref = pytest.mark.skipif(not O.have_ref("strict"), reason="oracle/_ref not built here")


@pytest.fixture(scope="module")
def gl():
    return np.load(GOLDEN_LOCAL)


@pytest.fixture(scope="module")
def tiny_local_model():
    return synth.make_model(synth.TINY_LOCAL, seed=3)


def test_local_tensors_do_not_disturb_the_decoder(tiny_local_model, tiny_model):
    for name, value in tiny_model.tensors.items():
        assert np.array_equal(tiny_local_model.tensors[name], value), name


def test_xorshift_known_values(port):
    # src/graph.c:1606-1610: x ^= x << 13; x ^= x >> 7; x ^= x << 17 on 64 bits, and the
    # all-zero state is replaced by the golden-ratio constant
    def step(x):
        x ^= (x << 13) & 0xFFFFFFFFFFFFFFFF
        x ^= x >> 7
        x ^= (x << 17) & 0xFFFFFFFFFFFFFFFF
        return x or 0x9E3779B97F4A7C15
    for seed in (1, 0x1234, 0x9E3779B97F4A7C15, 2 ** 63 + 5):
        assert port.lib.orc_xorshift64(seed) == step(seed)
    assert port.lib.orc_xorshift64(0) == 0x9E3779B97F4A7C15


@pytest.mark.parametrize("name", ["f32", "int8", "int4"])
def test_port_local_step_and_frame_match_reference_fixtures(name, gl, tiny_local_model):
    shape = synth.TINY_LOCAL
    pm = O.PortModel(tiny_local_model, QT[name])
    pl = O.PortLocal(pm, top_count=shape.vocab)
    rows = gl["tiny_rows"]
    for b, (temp, topk, seed, allow) in enumerate(TINY_LANES):
        pl.length = 0
        assert np.array_equal(pl.step(rows[b]), gl[f"tiny_{name}_step"][b])
        codes, values, saw, eos_frame, rng = pl.frame(rows[b], temp, topk, seed, bool(allow))
        assert np.array_equal(codes, gl[f"tiny_{name}_frame_codes"][b])
        assert saw == bool(gl[f"tiny_{name}_frame_saw_eos"][b])
        assert eos_frame == gl[f"tiny_{name}_frame_eos_frame"][b]
        assert rng == int(gl[f"tiny_{name}_frame_rng"][b])
        assert pl.length == shape.tables
        # stored codes collapse specials to 0; the fed-back values keep them
        assert np.array_equal(codes, np.where(values < shape.codebook_size, values, 0))
        if not allow:
            assert not (values == shape.eos_id).any()
    pl.close(); pm.close()


def port_generate(pm, shape, memories, start, frames, lanes, min_frames, capacity):
    streams = [pm.new_stream(m, capacity) for m in memories]
    top = max(min(k, shape.vocab) for _, k, _, _ in lanes)
    locals_ = [O.PortLocal(pm, top) for _ in memories]
    codes = np.array(start, np.uint32).copy()
    rng = [seed for _, _, seed, _ in lanes]
    all_codes = np.zeros((frames, len(memories), shape.tables), np.uint32)
    hidden = np.zeros((frames, len(memories), shape.width), np.float32)
    saw = np.zeros((frames, len(memories)), np.int32)
    for f in range(frames):
        for b, st in enumerate(streams):
            out = st.step(pm.embed_frame(codes[b]))
            hidden[f, b] = out
            temp, topk, _, _ = lanes[b]
            c, _, s, _, rng[b] = locals_[b].frame(out, temp, topk, rng[b], f >= min_frames)
            codes[b] = c
            all_codes[f, b] = c
            saw[f, b] = s
    for st in streams:
        st.close()
    for l in locals_:
        l.close()
    return all_codes, hidden, saw, np.array(rng, np.uint64)


@pytest.mark.parametrize("name", ["f32", "int8", "int4"])
def test_port_generation_loop_matches_reference_fixture(name, gl, tiny_local_model):
    shape = synth.TINY_LOCAL
    pm = O.PortModel(tiny_local_model, QT[name])
    memories = [synth.make_memory(shape, seed=300 + b) for b in range(4)]
    start = np.stack([synth.make_codes(shape, seed=400 + b, frames=1)[0] for b in range(4)])
    codes, hidden, saw, rng = port_generate(pm, shape, memories, start, 24, TINY_LANES[:4], 4, 32)
    assert np.array_equal(codes, gl[f"tiny_{name}_gen_codes"])
    assert np.array_equal(hidden[[0, 1, 23]], gl[f"tiny_{name}_gen_hidden"])
    assert np.array_equal(saw, gl[f"tiny_{name}_gen_saw_eos"])
    assert np.array_equal(rng, gl[f"tiny_{name}_gen_rng"])
    pm.close()


@needs_ref
def test_port_matches_compiled_reference_batched(tiny_local_model):
    """The reference steps requests together (projections batched, attention per
    request); the port steps them one by one.  Same bits."""
    shape = synth.TINY_LOCAL
    rng = np.random.default_rng(9)
    rows = rng.normal(0, 1, size=(5, shape.width)).astype(np.float32)
    for name, qt in QT.items():
        rm = O.RefModel(tiny_local_model, qt, "strict")
        pm = O.PortModel(tiny_local_model, qt)
        rl = [rm.new_local(16) for _ in range(5)]
        pl = O.PortLocal(pm, 16)
        codes, saw, eos, rngs = rm.local_frame(rl, rows, [0.9] * 5, [16] * 5, [3, 4, 5, 6, 7], [1] * 5)
        for b in range(5):
            c, _, s, e, r = pl.frame(rows[b], 0.9, 16, 3 + b, True)
            assert np.array_equal(c, codes[b]) and s == bool(saw[b]) and e == eos[b] and r == rngs[b]
        for l in rl:
            l.close()
        pl.close(); pm.close(); rm.close()
