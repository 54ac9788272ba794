"""GPU parity of the whole decoder step through the C ABI: per-layer hidden
states, KV layout, batch invariance, greedy token streams against fixtures
generated from the reference, and round-trip properties at full size.

Tolerances (relative to the largest magnitude of the reference row):
  strict mode        f32/f16 2e-5, int8/int4 2e-5 (bit-equal except where libm's
                     expf/tanhf are not correctly rounded)
  fast mode          f32/f16 1e-3, int8 1e-2, int4 2e-2   (int8/int4: one
                     activation-rounding flip moves a row by ~1/127 of a product)
"""
import numpy as np
import pytest

from conftest import rel_err
from mynah_tts_b200 import synth
from mynah_tts_b200.backend import Backend, Decoder, MynahB200Error
from oracle import oracle as O

pytestmark = pytest.mark.gpu
QT = {"f32": O.F32, "int8": O.INT8, "int4": O.INT4, "f16": O.F16}
FAST_TOL = {"f32": 1e-3, "f16": 1e-3, "int8": 1e-2, "int4": 2e-2}
STRICT_TOL = 2e-5


@pytest.mark.parametrize("name", ["f32", "int8", "int4", "f16"])
@pytest.mark.parametrize("strict", [True, False])
def test_tiny_decoder_per_layer_and_kv(name, strict, tiny_model, tiny_memory):
    shape = synth.TINY
    tol = STRICT_TOL if strict else FAST_TOL[name]
    pm = O.PortModel(tiny_model, QT[name])
    ps = pm.new_stream(tiny_memory, 64)
    be = Backend(name, strict=strict)
    assert be.libm_exact == strict
    exact = strict and name in ("int8", "int4")
    dec = Decoder(be, tiny_model, capacity=64, slots=3)
    dec.slot_load(1, ps.cross_k, ps.cross_v)
    forced = synth.make_codes(shape, seed=7, frames=10)
    for f in range(10):
        row = pm.embed_frame(forced[f])
        want = ps.step(row)
        got = dec.step_batch([1], row[None, :])[0]
        assert rel_err(got, want) < tol, (name, strict, f)
        if exact:
            assert np.array_equal(got, want), (name, f)
    k, v = dec.slot_read_kv(1)
    if exact:
        # integer products + reference-order glue + the host's libm: the cache is the
        # reference's, bit for bit
        assert np.array_equal(k[:, :10], ps.self_k[:, :10]) and np.array_equal(v[:, :10], ps.self_v[:, :10])
    assert rel_err(k[:, :10], ps.self_k[:, :10]) < tol and rel_err(v[:, :10], ps.self_v[:, :10]) < tol
    assert not k[:, 10:].any() and not v[:, 10:].any()          # nothing written past the length
    assert dec.slot_length(1) == 10 and dec.slot_length(0) == 0
    # per-layer hidden states of one more step at position 10
    row = pm.embed_frame(forced[0])
    for n in range(1, shape.layers + 1):
        ps.length = 10
        ps.set_layers(n)
        dec.slot_set_length(1, 10)
        dec.set_layers(n)
        got, want = dec.step_batch([1], row[None, :])[0], ps.step(row)
        assert rel_err(got, want) < tol
        if exact:
            assert np.array_equal(got, want), (name, n)
    dec.close(); be.close(); ps.close(); pm.close()


def test_tiny_decoder_against_reference_fixtures(golden, tiny_model, tiny_memory):
    """Strict int8/f32 against hidden states and tokens the reference produced."""
    shape = synth.TINY
    forced = synth.make_codes(shape, seed=7, frames=10)
    for name in ("int8", "f32", "int4"):
        be = Backend(name, strict=True)
        dec = Decoder(be, tiny_model, capacity=64, slots=1)
        dec.slot_load(0, golden["tiny_cross_k"], golden["tiny_cross_v"])
        for f in range(10):
            tokens, hidden = dec.frame_batch([0], forced[f:f + 1], [1], want_hidden=True)
            assert rel_err(hidden[0], golden[f"tiny_{name}_forced_hidden"][f]) < STRICT_TOL
            if name != "f32":
                assert np.array_equal(hidden[0], golden[f"tiny_{name}_forced_hidden"][f])
            assert np.array_equal(tokens[0], golden[f"tiny_{name}_forced_tokens"][f])
        dec.close(); be.close()


@pytest.mark.parametrize("strict", [True, False])
def test_stream_result_does_not_depend_on_batch(strict, tiny_model, tiny_memory):
    """Stream s alone == stream s inside a batch of 2, 16, 17 and 64, bit for bit
    (the reference asserts the same of its batched products, src/qmat.c:1107-1179)."""
    shape = synth.TINY
    pm = O.PortModel(tiny_model, O.INT8)
    ps = pm.new_stream(tiny_memory, 8)
    ck, cv = ps.cross_k.copy(), ps.cross_v.copy()
    rng = np.random.default_rng(4)
    rows = rng.normal(0, 0.05, size=(64, 3, shape.width)).astype(np.float32)
    for name in ("int8", "f32", "int4"):
        be = Backend(name, strict=strict)
        dec = Decoder(be, tiny_model, capacity=40, slots=64)
        for s in range(64):
            dec.slot_load(s, ck, cv)
        solo = [dec.step_batch([5], rows[5, t][None, :])[0].copy() for t in range(3)]
        for batch in (2, 16, 17, 64):
            for s in range(64):
                dec.slot_set_length(s, 0)
            # slot 5 rides in lane batch-1, with staggered positions around it
            lanes = [s for s in range(64) if s != 5][:batch - 1] + [5]
            for lane, s in enumerate(lanes[:-1]):
                dec.slot_set_length(s, lane % 7)
            for t in range(3):
                out = dec.step_batch(lanes, np.stack([rows[s, t] for s in lanes]))
                assert np.array_equal(out[-1], solo[t]), (name, strict, batch, t)
        dec.close(); be.close()
    ps.close(); pm.close()


@pytest.mark.parametrize("strict", [False, True])
@pytest.mark.parametrize("shape_name,name", [("tiny", "int8"), ("full", "int8"), ("tiny", "int4"), ("full", "int4")])
def test_cross_block_launch_matches_separate_launches(shape_name, name, strict, tiny_model, tiny_memory, monkeypatch):
    """The one-launch cross-attention block (norm, query product, attention, output
    product, norm; int8 or int4 weights) gives the bits of the five launches it replaces,
    the tensor-core product split along K over a cluster the bits of the unsplit one, and the
    strict self attention followed by a quantizing launch the bits of the attention that
    quantizes its rows in its own tail (MYNAH_B200_NO_SPLIT_QUANT), at 1, 2, 5, 16 and 64
    streams with different rows and staggered positions."""
    if shape_name == "tiny":
        shape, model, memory = synth.TINY, tiny_model, tiny_memory
    else:
        shape = synth.MAGPIE_357M
        model = synth.make_model(shape, seed=31)
        memory = synth.make_memory(shape, seed=131)
    pm = O.PortModel(model, QT[name])
    ps = pm.new_stream(memory, 4)
    ck, cv = ps.cross_k.copy(), ps.cross_v.copy()
    ps.close(); pm.close()
    rng = np.random.default_rng(12)
    rows = rng.normal(0, 0.05, size=(3, 64, shape.width)).astype(np.float32)
    outs, launches = {}, {}
    for mode in ("block", "separate", "unsplit", "tail"):
        monkeypatch.delenv("MYNAH_B200_NO_CROSS_BLOCK", raising=False)
        monkeypatch.delenv("MYNAH_B200_NO_KSPLIT", raising=False)
        monkeypatch.delenv("MYNAH_B200_NO_SPLIT_QUANT", raising=False)
        if mode == "tail":
            monkeypatch.setenv("MYNAH_B200_NO_SPLIT_QUANT", "1")
        if mode == "separate":
            monkeypatch.setenv("MYNAH_B200_NO_CROSS_BLOCK", "1")
        if mode == "unsplit":
            monkeypatch.setenv("MYNAH_B200_NO_KSPLIT", "1")
        be = Backend(name, strict=strict)
        dec = Decoder(be, model, capacity=16, slots=64)
        for s in range(64):
            # every slot its own text states: a rolled copy of the same cross K/V
            dec.slot_load(s, np.roll(ck, s, axis=1), np.roll(cv, s, axis=1))
        got = []
        launches0 = be.launch_count
        for batch in (1, 2, 5, 16, 64):
            for s in range(64):
                dec.slot_set_length(s, s % 5)
            lanes = list(range(64))[::-1][:batch]
            for t in range(3):
                got.append(dec.step_batch(lanes, rows[t, :batch]).copy())
        outs[mode] = got
        launches[mode] = be.launch_count - launches0
        dec.close(); be.close()
    for a, b, c, d in zip(outs["block"], outs["separate"], outs["unsplit"], outs["tail"]):
        assert np.array_equal(a, b)
        assert np.array_equal(a, c)
        assert np.array_equal(a, d)
    assert launches["block"] < launches["separate"]          # the block really replaced launches
    if strict:
        assert launches["tail"] < launches["block"]          # the quantizing launch really ran


def test_staggered_lengths_and_lane_masking(tiny_model, tiny_memory):
    """Streams at different positions in one step, and a batch that is not a
    power of two (lanes past the live count stay untouched)."""
    shape = synth.TINY
    pm = O.PortModel(tiny_model, O.INT8)
    be = Backend("int8", strict=True)
    dec = Decoder(be, tiny_model, capacity=32, slots=8)
    streams = [pm.new_stream(tiny_memory, 32) for _ in range(5)]
    rng = np.random.default_rng(8)
    for s, st in enumerate(streams):
        dec.slot_load(s, st.cross_k, st.cross_v)
    # advance stream s by s steps alone
    for s, st in enumerate(streams):
        for _ in range(s):
            row = rng.normal(0, 0.05, size=(shape.width,)).astype(np.float32)
            assert rel_err(dec.step_batch([s], row[None, :])[0], st.step(row)) < STRICT_TOL
    rows = rng.normal(0, 0.05, size=(5, shape.width)).astype(np.float32)
    out = dec.step_batch([4, 2, 0, 3, 1], rows)
    for lane, s in enumerate([4, 2, 0, 3, 1]):
        assert rel_err(out[lane], streams[s].step(rows[lane])) < STRICT_TOL
        assert dec.slot_length(s) == s + 1
    k, _ = dec.slot_read_kv(7)
    assert not k.any()                                  # an unused slot is never written
    for st in streams:
        st.close()
    dec.close(); be.close(); pm.close()


@pytest.mark.parametrize("name", ["int8", "f32"])
@pytest.mark.parametrize("strict", [True, False])
def test_requests_of_different_text_lengths_in_one_batch(name, strict, tiny_model):
    """Every request keeps its own text length (decoder_cache.memory_length,
    src/graph.c:2820,3223-3243): slots holding 24, 17, 9, 1 and 24 text states are stepped
    together and each lane must equal its own stream through the CPU checker -- bit for bit
    in strict mode with integer weights -- both when the cross K/V come from the host
    (slot_load, the request's own [layers][length][xw] arrays) and when they are made on the
    device (slot_prefill)."""
    shape = synth.TINY
    lengths = [24, 17, 9, 1, 24]
    pm = O.PortModel(tiny_model, QT[name])
    be = Backend(name, strict=strict)
    dec = Decoder(be, tiny_model, capacity=16, slots=8)
    tol = STRICT_TOL if strict else FAST_TOL[name]
    rng = np.random.default_rng(19)
    for how in ("load", "prefill"):
        streams = []
        for slot, n in enumerate(lengths):
            memory = synth.make_memory(shape, seed=60 + slot)[:n]
            st = pm.new_stream(memory, 16)
            streams.append(st)
            if how == "load":
                dec.slot_load(slot, st.cross_k, st.cross_v)
            else:
                dec.slot_prefill(slot, memory)
        for t in range(3):
            rows = rng.normal(0, 0.05, size=(len(lengths), shape.width)).astype(np.float32)
            lanes = [3, 0, 4, 2, 1]
            out = dec.step_batch(lanes, rows[lanes])
            for lane, slot in enumerate(lanes):
                want = streams[slot].step(rows[slot])
                assert rel_err(out[lane], want) < tol, (how, t, slot)
                if strict and name == "int8":
                    assert np.array_equal(out[lane], want), (how, t, slot)
        for st in streams:
            st.close()
    with pytest.raises(MynahB200Error, match="memory"):
        dec.slot_prefill(0, np.zeros((shape.memory_length + 1, shape.width), np.float32))
    dec.close(); be.close(); pm.close()


def test_decoder_errors(tiny_model, tiny_memory):
    be = Backend("int8")
    dec = Decoder(be, tiny_model, capacity=4, slots=2)
    pm = O.PortModel(tiny_model, O.INT8)
    ps = pm.new_stream(tiny_memory, 4)
    dec.slot_load(0, ps.cross_k, ps.cross_v)
    row = np.zeros((1, synth.TINY.width), np.float32)
    with pytest.raises(MynahB200Error, match="slot"):
        dec.step_batch([2], row)
    with pytest.raises(MynahB200Error, match="once"):
        dec.step_batch([0, 0], np.concatenate([row, row]))
    with pytest.raises(MynahB200Error, match="max_batch"):       # src/graph.c:3133-3136
        dec.step_batch([0, 1, 0], np.concatenate([row, row, row]))
    for _ in range(4):
        dec.step_batch([0], row)
    with pytest.raises(MynahB200Error, match="capacity"):        # src/graph.c:3152-3155
        dec.step_batch([0], row)
    bad = np.full((1, synth.TINY.tables), synth.TINY.vocab + 3, np.uint32)
    dec.slot_set_length(0, 0)
    with pytest.raises(MynahB200Error, match="vocabulary"):      # src/graph.c:794-797
        dec.frame_batch([0], bad)
    assert dec.step_batch([], row[:0]) is not None               # empty batch is a no-op (src/graph.c:3132)
    dec.close(); be.close(); ps.close(); pm.close()


def test_bound_frame_call_matches_frame_batch(golden, tiny_model):
    """bind_frame_batch (arguments made once, one foreign call per frame on the caller's two
    host buffers) gives frame_batch's tokens, frame after frame, and refuses buffers of the
    wrong type or shape."""
    shape = synth.TINY
    start = np.concatenate([synth.make_codes(shape, seed=9 + g, frames=1) for g in range(3)])
    be = Backend("int8", strict=True)
    dec = Decoder(be, tiny_model, capacity=40, slots=6)
    for s in range(6):
        dec.slot_load(s, golden["tiny_cross_k"], golden["tiny_cross_v"])
    codes = np.ascontiguousarray(start, np.uint32)
    want = []
    for f in range(12):
        tokens = dec.frame_batch([0, 1, 2], codes, [0, 0, 0])
        want.append(tokens.copy())
        codes = tokens.copy()
    buf_codes = np.ascontiguousarray(start, np.uint32).copy()
    buf_tokens = np.zeros_like(buf_codes)
    step = dec.bind_frame_batch([3, 4, 5], buf_codes, [0, 0, 0], buf_tokens)
    for f in range(12):
        assert step() is buf_tokens
        assert np.array_equal(buf_tokens, want[f]), f
        buf_codes[:] = buf_tokens
    with pytest.raises(ValueError):
        dec.bind_frame_batch([3, 4, 5], buf_codes.astype(np.int64), [0, 0, 0], buf_tokens)
    with pytest.raises(ValueError):
        dec.bind_frame_batch([3, 4], buf_codes, [0, 0], buf_tokens)
    dec.close(); be.close()


@pytest.mark.parametrize("name", ["f32", "int8", "int4"])
def test_tiny_greedy_tokens_match_reference(name, golden, tiny_model, tiny_memory):
    """Free-running greedy decode (EOS allowed from frame 4) through both entry
    points -- the per-frame host-buffer call and the device-resident loop --
    against the reference's token stream."""
    shape = synth.TINY
    want = golden[f"tiny_{name}_greedy_tokens"]
    start = synth.make_codes(shape, seed=9, frames=1)
    be = Backend(name, strict=True)
    dec = Decoder(be, tiny_model, capacity=80, slots=2)
    dec.slot_load(0, golden["tiny_cross_k"], golden["tiny_cross_v"])
    dec.slot_load(1, golden["tiny_cross_k"], golden["tiny_cross_v"])
    codes = start.copy()
    got = []
    for f in range(64):
        tokens = dec.frame_batch([0], codes, [int(f >= 4)])
        got.append(tokens[0].copy())
        if (tokens[0] == shape.eos_id).any():
            break
        codes = np.where(tokens < shape.codebook_size, tokens, 0).astype(np.uint32)
    assert np.array_equal(np.stack(got), want)
    tokens, eos, ms, _ = dec.greedy([1], start, 64, min_frames=4)
    n = len(want)
    assert np.array_equal(tokens[:n, 0], want)
    assert eos[0] == (n - 1 if (want[-1] == shape.eos_id).any() else -1)
    dec.close(); be.close()


def _full_setup(seed, name, strict, capacity, slots=1):
    shape = synth.MAGPIE_357M
    model = synth.make_model(shape, seed=seed)
    memory = synth.make_memory(shape, seed=seed + 100)
    start = synth.make_codes(shape, seed=seed + 200, frames=1)
    pm = O.PortModel(model, QT[name])
    ps = pm.new_stream(memory, 4)            # only for the cross K/V precompute
    be = Backend(name, strict=strict)
    dec = Decoder(be, model, capacity=capacity, slots=max(slots, 2))
    for s in range(max(slots, 2)):
        dec.slot_load(s, ps.cross_k, ps.cross_v)
    ps.close(); pm.close()
    return shape, model, start, be, dec


def first_divergence(got, want):
    bad = np.nonzero((got != want).any(axis=-1))[0]
    return int(bad[0]) if len(bad) else -1


@pytest.mark.parametrize("name,seed", [("int8", 21), ("int8", 22), ("int8", 23), ("f32", 21), ("int4", 21)])
def test_full_greedy_512_frames_match_reference(name, seed, golden, record_property):
    """The Magpie-357M shape, 512 greedy frames from empty KV, strict mode: the
    token stream must equal the reference's.  Every seed of the fixture file is
    listed here; none is left out."""
    shape, model, start, be, dec = _full_setup(seed, name, True, 520)
    want = golden[f"full_{name}_s{seed}_tokens"].astype(np.uint32)
    tokens, eos, ms, _ = dec.greedy([0], start, 512, min_frames=10 ** 6)
    div = first_divergence(tokens[:, 0], want)
    record_property("first_divergence", div)
    k, v = dec.slot_read_kv(0)
    dec.close(); be.close()
    if name != "f32":
        import zlib
        kv_crc = np.uint32(zlib.crc32(np.ascontiguousarray(k[:, :512]).tobytes())) ^ \
            np.uint32(zlib.crc32(np.ascontiguousarray(v[:, :512]).tobytes()))
        record_property("kv_crc_equal", bool(kv_crc == golden[f"full_{name}_s{seed}_kv_crc"]))
    margin = golden[f"full_{name}_s{seed}_margin"]
    assert div == -1, (f"{name} seed {seed}: token streams part at frame {div}; the reference's "
                       f"top-2 margin there is {margin[div]:.2e}")
    if name != "f32":
        # the whole KV cache after 512 frames is the reference's, bit for bit
        assert kv_crc == golden[f"full_{name}_s{seed}_kv_crc"]


@pytest.mark.parametrize("name", ["int8", "f32", "int4"])
def test_full_fast_mode_single_steps_and_picks(name, golden, record_property):
    """Fast (production) mode on the Magpie-357M shape, teacher-forced with the
    reference's tokens.

    (a) Single steps from the reference's exact state: the strict decoder (which
    the tests above pin to the reference bit for bit) carries the KV cache; at
    frames 0, 1, 63, 64, 255, 256, 511 its cache is copied into the fast
    decoder, which then runs that one frame.  The hidden row must be within the
    mode's tolerance of the reference's.  For the quantized modes the tolerance
    is set by activation-rounding flips: a last-bit difference in a LayerNorm
    sum can move one int8 activation by one step, and twelve random-init layers
    amplify that to about 1e-2 of the row.
    (b) Greedy picks of the fast decoder running all 512 frames on its own
    cache, teacher-forced: a pick may differ from the reference's only where the
    reference's top-2 margin is within what the measured deviation of that
    frame's hidden row can move two logits by -- 2 * |h_fast - h_strict| * (largest
    head-row norm), plus one activation-rounding step of the head product for the
    quantized formats.  While the fast decoder's cache has not drifted (no
    rounding flip yet) that bound is ~1e-4 or the rounding step, far below the
    typical margin, so the check is a real one: the number of frames it covered
    is asserted and recorded, with the first frame at which the picks part.
    (c) The free-running fast decode (its own picks fed back): first frame at
    which its tokens part from the reference's, recorded per seed."""
    seed = 21
    shape, model, start, be, dec = _full_setup(seed, name, False, 520, slots=3)
    _, _, _, sbe, sdec = _full_setup(seed, name, True, 520)
    want_tokens = golden[f"full_{name}_s{seed}_tokens"].astype(np.uint32)
    want_hidden = golden[f"full_{name}_s{seed}_hidden"]
    margin = golden[f"full_{name}_s{seed}_margin"]
    keep = (0, 1, 63, 64, 255, 256, 511)
    tol = {"f32": 1e-3, "int8": 2e-2, "int4": 2e-2}[name]
    head_norm = max(float(np.linalg.norm(model.tensors[f"local_transformer_out_projections.{t}.weight"], axis=1).max())
                    for t in range(shape.tables))
    head_wmax = max(float(np.abs(model.tensors[f"local_transformer_out_projections.{t}.weight"]).max())
                    for t in range(shape.tables))
    codes = start.copy()
    single, drift, disagree_wide, checked, first_part = [], 0.0, 0, 0, -1
    for f in range(512):
        if f in keep:
            k, v = sdec.slot_read_kv(0)
            dec.slot_load(1, golden_cross(sdec, be, model, seed)[0], golden_cross(sdec, be, model, seed)[1],
                          k, v, length=f)
            _, h1 = dec.frame_batch([1], codes, [0], want_hidden=True)
            single.append(rel_err(h1[0], want_hidden[keep.index(f)]))
        _, shidden = sdec.frame_batch([0], codes, [0], want_hidden=True)
        tokens, hidden = dec.frame_batch([0], codes, [0], want_hidden=True)
        if f in keep:
            drift = max(drift, rel_err(hidden[0], want_hidden[keep.index(f)]))
        # what the deviation of this frame's hidden row can move the gap between two logits by
        dh = float(np.linalg.norm(hidden[0].astype(np.float64) - shidden[0].astype(np.float64)))
        step = 0.0 if name == "f32" else float(np.abs(shidden[0]).max()) / 127.0 * head_wmax
        eps = 2.0 * dh * head_norm + 2.0 * step + 1e-6
        same = np.array_equal(tokens[0], want_tokens[f])
        if not same and first_part < 0:
            first_part = f
        if margin[f] > eps:
            checked += 1
            if not same:
                disagree_wide += 1
        codes = np.where(want_tokens[f] < shape.codebook_size, want_tokens[f], 0).astype(np.uint32)[None, :]
    # (c) free-running: the fast decoder feeds back its own picks
    free, _, _, _ = dec.greedy([2], start, 512, min_frames=10 ** 6)
    free_div = first_divergence(free[:, 0], want_tokens)
    dec.close(); be.close(); sdec.close(); sbe.close()
    record_property("single_step_rel_err", [float(x) for x in single])
    record_property("drift_rel_err", drift)
    record_property("teacher_forced_frames_checked", checked)
    record_property("teacher_forced_first_parting_frame", first_part)
    record_property("free_running_first_divergence_frame", free_div)
    print(f"{name}: single-step errors {single}, drift over 512 frames {drift:.3e}; teacher-forced picks checked on "
          f"{checked} of 512 frames, first parting frame {first_part}; free-running first divergence {free_div}")
    assert max(single) < tol, single
    assert drift < 5e-2
    assert checked > 0, checked            # the margin test must have covered real frames
    assert disagree_wide == 0


_cross_cache = {}


def golden_cross(sdec, be, model, seed):
    """Cross K/V of the request (CPU precompute of decoder_cache_init, cached)."""
    if seed not in _cross_cache:
        shape = synth.MAGPIE_357M
        pm = O.PortModel(model, O.F32)
        ps = pm.new_stream(synth.make_memory(shape, seed=seed + 100), 4)
        _cross_cache[seed] = (ps.cross_k.copy(), ps.cross_v.copy())
        ps.close(); pm.close()
    return _cross_cache[seed]


@pytest.mark.parametrize("name", ["int8", "int4"])
def test_full_size_properties_64_streams(name, golden):
    """At the benchmark's size (64 streams, products on the tensor cores): every lane
    that starts from the same codes and memory yields the same tokens as lane 0 and as
    the single-stream run (SIMT products), and a lane's tokens do not change when the
    others stop early."""
    seed = 21
    shape, model, start, be, dec = _full_setup(seed, name, False, 140, slots=64)
    slots = list(range(64))
    codes = np.repeat(start, 64, axis=0)
    tokens, eos, ms, _ = dec.greedy(slots, codes, 128, min_frames=10 ** 6)
    for b in range(1, 64):
        assert np.array_equal(tokens[:, b], tokens[:, 0])
    for s in slots:
        dec.slot_set_length(s, 0)
    solo, _, _, _ = dec.greedy([0], start, 128, min_frames=10 ** 6)     # one lane: the SIMT kernel
    assert np.array_equal(solo[:, 0], tokens[:, 0])
    dec.slot_set_length(0, 0)
    frames = [128 if b % 3 == 0 else 16 + b for b in range(64)]
    tokens2, _, _, _ = dec.greedy(slots, codes, frames, min_frames=10 ** 6)
    for b in range(64):
        assert np.array_equal(tokens2[:frames[b], b], tokens[:frames[b], 0])
        assert not tokens2[frames[b]:, b].any()
        assert dec.slot_length(b) == frames[b]
    dec.close(); be.close()


def _oracle_lanes(model, shape, qtype, cross, positions, codes, frames, capacity):
    """Hidden rows and picks of `len(positions)` independent streams, lane b starting at
    position positions[b] over zeroed cache rows with cross K/V cross[b], through the CPU
    checker: the reference's own strict build stepping 16 lanes at a time on all host cores
    where it is present (it equals the C restatement bit for bit), else the restatement."""
    lanes = len(positions)
    hidden = np.empty((frames, lanes, shape.width), np.float32)
    tokens = np.empty((frames, lanes, shape.tables), np.uint32)
    memory = synth.make_memory(shape, seed=1)
    if O.have_ref("strict"):
        import os
        rm = O.RefModel(model, qtype, "strict", threads=os.cpu_count() or 1)
        decs = [rm.new_decoder(memory, capacity) for _ in range(lanes)]
        for b, d in enumerate(decs):
            d.cross_k[:] = cross[b][0]
            d.cross_v[:] = cross[b][1]
            d.length = positions[b]
        cur = codes.copy()
        for f in range(frames):
            rows = np.stack([rm.embed_frame(cur[b]) for b in range(lanes)])
            for g in range(0, lanes, 16):
                hidden[f, g:g + 16] = rm.step_batch(decs[g:g + 16], rows[g:g + 16])
            for b in range(lanes):
                tokens[f, b] = rm.heads_argmax(hidden[f, b], False)[0]
            cur = np.where(tokens[f] < shape.codebook_size, tokens[f], 0).astype(np.uint32)
        for d in decs:
            d.close()
        rm.close()
        return hidden, tokens
    pm = O.PortModel(model, qtype)
    for b in range(lanes):
        ps = pm.new_stream(memory, capacity)
        ps.cross_k[:] = cross[b][0]
        ps.cross_v[:] = cross[b][1]
        ps.length = positions[b]
        cur = codes[b].copy()
        for f in range(frames):
            tok, hid, _ = ps.greedy_frame(cur.copy(), allow_eos=False)
            hidden[f, b], tokens[f, b] = hid, tok
            cur = np.where(tok < shape.codebook_size, tok, 0).astype(np.uint32)
        ps.close()
    pm.close()
    return hidden, tokens


@pytest.mark.parametrize("name", ["int8", "int4"])
def test_full_size_distinct_lanes_match_oracle(name, monkeypatch):
    """The Magpie-357M shape at 64 lanes that all differ -- their own start codes, their own
    text states (rolled cross K/V) and staggered positions up to 77 (three cache chunks) --
    for three greedy frames against the CPU checker lane by lane: in strict mode every hidden
    row and pick must be the checker's bit for bit, on the tensor-core products (K = 768 and
    the K = 3072 ring with its cluster split, the six-stage logit-head product, the int4
    tile) and again with MYNAH_B200_NO_TC=1 (the SIMT products); fast mode is held to rounding
    on the typical lane and to its drift bound on every lane, and its tensor-core and SIMT
    runs to each other bit for bit."""
    shape = synth.MAGPIE_357M
    qtype = QT[name]
    model = synth.make_model(shape, seed=51)
    lanes, frames, capacity = 64, 3, 96
    pm = O.PortModel(model, O.F32)
    ps = pm.new_stream(synth.make_memory(shape, seed=151), 4)
    ck, cv = ps.cross_k.copy(), ps.cross_v.copy()
    ps.close(); pm.close()
    cross = [(np.roll(ck, b, axis=1), np.roll(cv, b, axis=1)) for b in range(lanes)]
    positions = [(11 * b) % 78 for b in range(lanes)]
    codes = np.stack([synth.make_codes(shape, seed=300 + b, frames=1)[0] for b in range(lanes)])
    want_hidden, want_tokens = _oracle_lanes(model, shape, qtype, cross, positions, codes, frames, capacity)
    got = {}
    for strict in (True, False):
        for no_tc in (False, True):
            monkeypatch.delenv("MYNAH_B200_NO_TC", raising=False)
            if no_tc:
                monkeypatch.setenv("MYNAH_B200_NO_TC", "1")
            be = Backend(name, strict=strict)
            dec = Decoder(be, model, capacity=capacity, slots=lanes)
            for b in range(lanes):
                dec.slot_load(b, cross[b][0], cross[b][1])
                dec.slot_set_length(b, positions[b])
            # lanes in reverse slot order: lane index and slot index differ
            order = list(range(lanes))[::-1]
            cur = codes[order].copy()
            hid, tok = [], []
            for f in range(frames):
                t, h = dec.frame_batch(order, cur, [0] * lanes, want_hidden=True)
                hid.append(h.copy()); tok.append(t.copy())
                cur = np.where(t < shape.codebook_size, t, 0).astype(np.uint32)
            dec.close(); be.close()
            inv = np.argsort(order)
            got[(strict, no_tc)] = (np.stack(hid)[:, inv], np.stack(tok)[:, inv])
    for no_tc in (False, True):
        h, t = got[(True, no_tc)]
        for b in range(lanes):
            assert np.array_equal(h[:, b], want_hidden[:, b]), (name, "strict", no_tc, b)
        assert np.array_equal(t, want_tokens), (name, "strict", no_tc)
    hf, tf = got[(False, False)]
    # frame 0 starts from the checker's exact state (later frames follow the lane's own picks):
    # a lane is within rounding unless one of its ~75k int8 activations rounded the other way,
    # which twelve random-init layers amplify to the order of 1e-2 of the row
    per_lane = np.array([rel_err(hf[0, b], want_hidden[0, b]) for b in range(lanes)])
    assert np.median(per_lane) < 1e-4 and per_lane.max() < 5e-2, per_lane
    assert np.array_equal(hf, got[(False, True)][0]) and np.array_equal(tf, got[(False, True)][1])


@pytest.mark.parametrize("shape_name,lanes", [("tiny", 16), ("tiny", 64), ("full", 17)])
def test_f16_weights_on_the_tensor_cores_match_oracle(shape_name, lanes, tiny_model, monkeypatch):
    """f16 weights at 16 or more lanes run on tcgen05 tiles (kind::f16, activations split into
    two f16 halves): lanes that all differ, staggered positions, two frames, every lane
    against the CPU restatement of the reference's f16 product (f32 activations, f16 weights,
    src/qmat.c:319-377) within its 1e-3 bound, and against the same decoder on the SIMT
    products (MYNAH_B200_NO_TC=1) to f32 rounding of the sums."""
    if shape_name == "tiny":
        shape, model = synth.TINY, tiny_model
    else:
        shape, model = synth.MAGPIE_357M, synth.make_model(synth.MAGPIE_357M, seed=61)
    capacity, frames = 48, 2
    pm = O.PortModel(model, O.F16)
    streams, cross = [], []
    positions = [(5 * b) % 37 for b in range(lanes)]
    for b in range(lanes):
        st = pm.new_stream(synth.make_memory(shape, seed=70 + b % 3), capacity)
        st.length = positions[b]
        streams.append(st)
        cross.append((st.cross_k.copy(), st.cross_v.copy()))
    rng = np.random.default_rng(23)
    rows = rng.normal(0, 0.05, size=(frames, lanes, shape.width)).astype(np.float32)
    want = np.stack([np.stack([streams[b].step(rows[f, b]) for b in range(lanes)]) for f in range(frames)])
    got = {}
    for no_tc in (False, True):
        monkeypatch.delenv("MYNAH_B200_NO_TC", raising=False)
        if no_tc:
            monkeypatch.setenv("MYNAH_B200_NO_TC", "1")
        be = Backend("f16", strict=False)
        dec = Decoder(be, model, capacity=capacity, slots=lanes)
        for b in range(lanes):
            dec.slot_load(b, cross[b][0], cross[b][1])
            dec.slot_set_length(b, positions[b])
        launches0 = be.launch_count
        got[no_tc] = np.stack([dec.step_batch(list(range(lanes)), rows[f]).copy() for f in range(frames)])
        got[(no_tc, "launches")] = be.launch_count - launches0
        dec.close(); be.close()
    for st in streams:
        st.close()
    pm.close()
    for f in range(frames):
        for b in range(lanes):
            assert rel_err(got[False][f, b], want[f, b]) < 1e-3, (f, b)
            assert rel_err(got[False][f, b], got[True][f, b]) < 2e-5, (f, b)
    # the tensor-core run really took the other path: a split launch rides with every product
    assert got[(False, "launches")] > got[(True, "launches")]


@pytest.mark.parametrize("shape_name,name,count,strict", [
    ("tiny", "int8", 20, True), ("tiny", "int8", 9, True), ("tiny", "f32", 20, True), ("tiny", "int4", 17, True),
    ("tiny", "int8", 16, True), ("tiny", "int8", 20, False), ("tiny", "f16", 20, False), ("full", "int8", 24, True),
    # fast mode at full size: more than 16 rows run on the tensor cores over split f16 planes
    ("full", "int8", 40, False), ("full", "f32", 19, False)])
def test_multi_row_prefill_matches_decoder_run(shape_name, name, count, strict, tiny_model, tiny_memory):
    """decoder_run with count > 1 (src/graph.c:3506-3641): a few rows stepped one by one, then
    `count` rows pushed at once, then a step on top, against the CPU restatement (itself equal
    to the reference's decoder_run bit for bit, tests/test_oracle.py).  More than 16 rows of a
    quantized model take the f32 weights, as in the reference.  Strict mode: hidden rows and
    the appended KV rows bit for bit for the integer and f32-weight paths."""
    if shape_name == "tiny":
        shape, model, memory = synth.TINY, tiny_model, tiny_memory
    else:
        shape = synth.MAGPIE_357M
        model = synth.make_model(shape, seed=71)
        memory = synth.make_memory(shape, seed=171)
    capacity = 64
    rng = np.random.default_rng(37)
    # the full-size fast cases isolate the many-row products (f32 weights on the tensor cores):
    # no quantized single steps in front, whose rounding flips would ride into the cache
    tc_case = shape_name == "full" and not strict
    first = rng.normal(0, 0.05, size=(0 if tc_case else 3, shape.width)).astype(np.float32)
    rows = rng.normal(0, 0.05, size=(count, shape.width)).astype(np.float32)
    after = rng.normal(0, 0.05, size=(shape.width,)).astype(np.float32)
    pm = O.PortModel(model, QT[name])
    ps = pm.new_stream(memory, capacity)
    be = Backend(name, strict=strict)
    dec = Decoder(be, model, capacity=capacity, slots=2, max_batch=max(count, 2), keep_f32_weights=True)
    dec.slot_load(1, ps.cross_k, ps.cross_v)
    # strict: exact wherever every sum is an integer or a reference-order chain (f32 products
    # of more than 16 rows are sequential sums in strict mode)
    exact = strict and (name in ("int8", "int4") or (name == "f32"))
    tol = STRICT_TOL if strict else FAST_TOL[name]
    for r in first:
        want, got = ps.step(r), dec.step_batch([1], r[None, :])[0]
        assert rel_err(got, want) < tol
    want, got = ps.prefill(rows), dec.prefill(1, rows)
    if tc_case:
        tol = 1e-4          # f32 weights as split f16 planes: measured 9e-6
    assert rel_err(got, want) < tol, (name, count, strict)
    if exact:
        assert np.array_equal(got, want), (name, count)
    assert dec.slot_length(1) == len(first) + count
    k, v = dec.slot_read_kv(1)
    n = len(first) + count
    assert rel_err(k[:, :n], ps.self_k[:, :n]) < tol and rel_err(v[:, :n], ps.self_v[:, :n]) < tol
    if tc_case:
        tol = 2e-2 if name != "f32" else 1e-3          # the single step on top is quantized again
    if exact:
        assert np.array_equal(k[:, :n], ps.self_k[:, :n]) and np.array_equal(v[:, :n], ps.self_v[:, :n])
    assert not k[:, n:].any()
    want, got = ps.step(after), dec.step_batch([1], after[None, :])[0]
    assert rel_err(got, want) < tol
    if exact:
        assert np.array_equal(got, want)
    with pytest.raises(MynahB200Error, match="capacity"):
        dec.prefill(1, np.zeros((capacity, shape.width), np.float32))
    dec.close(); be.close(); ps.close(); pm.close()


def test_prefill_of_a_quantized_model_needs_its_f32_weights(tiny_model, tiny_memory):
    be = Backend("int8", strict=True)
    dec = Decoder(be, tiny_model, capacity=48, slots=1, max_batch=20)
    with pytest.raises(MynahB200Error, match="f32 weights"):
        dec.prefill(0, np.zeros((20, synth.TINY.width), np.float32))
    dec.close(); be.close()


@pytest.mark.parametrize("strict", [True, False])
def test_slot_prefill_makes_the_reference_cross_kv(strict, tiny_model, tiny_memory, golden):
    """Cross K/V made on the device from the text memory (decoder_cache_init,
    src/graph.c:3002-3027: LayerNorm then the f32 kv_net product, whatever the
    weight format of the step) against the fixture taken from the reference, and a
    greedy decode from the prefilled slot against the reference's token stream."""
    shape = synth.TINY
    be = Backend("int8", strict=strict)
    dec = Decoder(be, tiny_model, capacity=80, slots=2)
    dec.slot_prefill(1, tiny_memory)
    k, v = dec.slot_read_cross(1)
    if strict:
        assert np.array_equal(k, golden["tiny_cross_k"]) and np.array_equal(v, golden["tiny_cross_v"])
        want = golden["tiny_int8_greedy_tokens"]
        start = synth.make_codes(shape, seed=9, frames=1)
        tokens, _, _, _ = dec.greedy([1], start, 64, min_frames=4)
        assert np.array_equal(tokens[:len(want), 0], want)
    else:
        assert rel_err(k, golden["tiny_cross_k"]) < 1e-5 and rel_err(v, golden["tiny_cross_v"]) < 1e-5
    with pytest.raises(MynahB200Error):
        dec.slot_prefill(0, np.concatenate([tiny_memory, tiny_memory[:1]]))   # more rows than the slots hold
    dec.close(); be.close()


@pytest.mark.parametrize("strict", [True, False])
def test_f32_heads_and_pick_in_one_launch(strict, tiny_model, tiny_memory, golden, monkeypatch):
    """f32 weights: the logit heads and the constrained first-on-ties pick run as one launch
    (the reference's fused f32 greedy path, src/qmat.c:453-536).  Strict: the tokens of the
    two-launch form (MYNAH_B200_NO_FUSE) at 1, 3 and 6 lanes with EOS allowed on some lanes;
    fast: both forms keep one sequential sum per logit, so they agree there too."""
    shape = synth.TINY
    rng = np.random.default_rng(3)
    got, launches = {}, {}
    for mode in ("fused", "separate"):
        monkeypatch.delenv("MYNAH_B200_NO_FUSE", raising=False)
        if mode == "separate":
            monkeypatch.setenv("MYNAH_B200_NO_FUSE", "1")
        be = Backend("f32", strict=strict)
        dec = Decoder(be, tiny_model, capacity=40, slots=6)
        for s in range(6):
            dec.slot_load(s, np.roll(golden["tiny_cross_k"], s, axis=1), np.roll(golden["tiny_cross_v"], s, axis=1))
        out = []
        l0 = be.launch_count
        for lanes in ([0], [3, 1, 4], [5, 4, 3, 2, 1, 0]):
            codes = rng.integers(0, shape.codebook_size, size=(len(lanes), shape.tables)).astype(np.uint32) \
                if mode == "fused" else None
            if mode == "fused":
                got.setdefault("codes", []).append(codes)
            codes = got["codes"][len(out) // 4]
            for f in range(4):
                tokens = dec.frame_batch(lanes, codes, [int((f + i) % 2) for i in range(len(lanes))])
                out.append(tokens.copy())
                codes = np.where(tokens < shape.codebook_size, tokens, 0).astype(np.uint32)
        got[mode] = out
        launches[mode] = be.launch_count - l0
        dec.close(); be.close()
    for a, b in zip(got["fused"], got["separate"]):
        if strict:
            assert np.array_equal(a, b)
        else:
            assert (a == b).mean() > 0.9          # the fast two-launch form sums its logits as a tree
    assert launches["fused"] < launches["separate"]


@pytest.mark.parametrize("lanes", [128, 256])
def test_many_streams_match_their_solo_runs(lanes):
    """128 and 256 streams stepped together (the attention launcher splits the heads of a
    stream over three or four CTAs there, several waves deep): strict mode, long staggered
    positions, every sampled lane's tokens equal the same stream stepped alone."""
    shape = synth.MAGPIE_357M
    model = synth.make_model(shape, seed=81)
    rng = np.random.default_rng(82)
    ck = rng.normal(0, 1, size=(shape.layers, shape.memory_length, shape.xattn_width)).astype(np.float32)
    be = Backend("int8", strict=True)
    dec = Decoder(be, model, capacity=300, slots=lanes)
    for s in range(lanes):
        dec.slot_load(s, np.roll(ck, s, axis=1), np.roll(ck, s + 1, axis=1))
    start = rng.integers(0, shape.codebook_size, size=(lanes, shape.tables)).astype(np.uint32)
    frames = 5
    for s in range(lanes):
        dec.slot_set_length(s, 200 + (s * 7) % 90)          # cached rows are zeros: positions matter, not contents
    together, _, _, _ = dec.greedy(list(range(lanes)), start, frames, min_frames=10 ** 6)
    for s in (0, 1, lanes // 2 + 3, lanes - 1):
        dec.slot_set_length(s, 200 + (s * 7) % 90)
        # the rows appended by the joint run lie beyond the reset length and are overwritten
        solo, _, _, _ = dec.greedy([s], start[s:s + 1], frames, min_frames=10 ** 6)
        assert np.array_equal(solo[:, 0], together[:, s]), s
    dec.close(); be.close()
