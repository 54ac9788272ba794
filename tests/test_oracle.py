"""CPU tests of the parity checker itself (no GPU): the C restatement in
oracle/mynah_oracle.c against (1) the known answers the reference's own
self-tests hold for this path, (2) fixtures generated from the reference's
sources (tests/golden/make_golden.py) and (3) the compiled reference, bit for
bit, wherever oracle/_ref exists."""
import zlib

import numpy as np
import pytest

from conftest import rel_err
from mynah_tts_b200 import synth
from oracle import oracle as O

QT = {"f32": O.F32, "int8": O.INT8, "int4": O.INT4}
needs_ref = pytest.mark.skipif(not O.have_ref("strict"), reason="oracle/_ref not built here")


def crc(a):
    return np.uint32(zlib.crc32(np.ascontiguousarray(a).tobytes()))


# ---- known answers of the reference's self-tests ---------------------------------
def test_kernels_known_answers(port):
    # src/kernels.c:440-509
    a = np.array([1, 2, 3], np.float32)
    b = np.array([4, -2, 0.5], np.float32)
    assert abs(port.lib.orc_dot_f32(O._fp(a), O._fp(b), 3) - 1.5) < 1e-6
    ln = port.layernorm(np.array([[1, 2, 3, 4]], np.float32), np.ones(4, np.float32), eps=1e-6)
    assert abs(ln[0, 0] + 1.34164) < 1e-4 and abs(ln[0, 3] - 1.34164) < 1e-4
    g = port.gelu(np.array([-1, 0, 1], np.float32))
    assert abs(g[1]) < 1e-6 and abs(g[2] - 0.8411920) < 1e-5
    probs = np.empty(3, np.float32)
    logits = np.array([1, 2, 3], np.float32)
    assert port.lib.orc_softmax(O._fp(logits), O._fp(probs), 3) == 0
    assert abs(probs.sum() - 1) < 1e-6 and probs.argmax() == 2
    assert port.lib.orc_softmax(O._fp(logits), O._fp(probs), 0) != 0   # empty softmax is refused


def test_backend_matmul_known_answer(port):
    # src/backend.c:290-310: 2x3x4 product with bias
    x = np.array([[1, 2, 3], [-1, 0.5, 2]], np.float32)
    w = np.array([[1, 0, 0], [0, 1, 0], [0, 0, 1], [1, 1, 1]], np.float32)
    bias = np.array([0.5, -0.5, 1, 2], np.float32)
    y = port.qmat_linear(O.F32, w, x, bias)
    assert np.allclose(y.ravel(), [1.5, 1.5, 4, 8, -0.5, 0, 3, 3.5], atol=1e-5)


def _selftest_data(n, k, wf, wc):
    i = np.arange(n, dtype=np.float32)[:, None]
    j = np.arange(k, dtype=np.float32)[None, :]
    return i, j


def test_qmat_selftest_bounds(port):
    # src/qmat.c:904-965: deterministic sin/cos data, int8 within 0.05 and int4
    # within 0.20 of the exact f32 product (relative, floor 1e-3).
    n, k = 48, 768
    idx = (np.arange(n)[:, None] * 7 + np.arange(k)[None, :]).astype(np.float32)
    w = (np.sin(np.float32(0.017) * idx) *
         (0.5 + 0.5 * np.cos(np.float32(0.003) * np.arange(k, dtype=np.float32)))[None, :]).astype(np.float32)
    x = (np.cos(np.float32(0.011) * np.arange(k, dtype=np.float32)) - np.float32(0.3)).astype(np.float32)
    ref = (w.astype(np.float64) @ x.astype(np.float64))
    for qt, limit in ((O.INT8, 0.05), (O.INT4, 0.20)):
        got = port.qmat_linear(qt, w, x[None, :])[0]
        rel = np.abs(got - ref) / np.maximum(np.abs(ref), 1e-3)
        assert rel.max() <= limit


def test_qmat_f16_bound(port):
    # src/qmat.c:1064-1104: f16 weights within 1e-3 of the f64 product
    n, k = 64, 512
    i = np.arange(n * k, dtype=np.float32)
    w = (np.sin(np.float32(0.017) * i) * (0.5 + 0.5 * np.cos(np.float32(0.003) * i))).astype(np.float32).reshape(n, k)
    x = (np.cos(np.float32(0.011) * np.arange(k, dtype=np.float32)) - np.float32(0.3)).astype(np.float32)
    bias = (np.arange(n, dtype=np.float32) * 0.125 - 0.25).astype(np.float32)
    got = port.qmat_linear(O.F16, w, x[None, :], bias)[0]
    ref = w.astype(np.float64) @ x.astype(np.float64) + bias
    assert (np.abs(got - ref) / np.maximum(np.abs(ref), 1e-3)).max() <= 1e-3


def test_f16_conversion_is_ieee_rne(port):
    rng = np.random.default_rng(0)
    vals = np.concatenate([rng.normal(0, 1, 4000), rng.normal(0, 1e-6, 500), rng.normal(0, 3e4, 500),
                           [0.0, -0.0, 65504.0, 65520.0, 1e-8, 6e-8]]).astype(np.float32)
    got = port.quantize_weight_f16(vals.reshape(1, -1))[0]
    want = vals.astype(np.float16).view(np.uint16)
    assert np.array_equal(got, want)


def test_batched_rows_equal_single_rows(port):
    # src/qmat.c:1107-1179: a row's result must not depend on its batch
    n, k, b = 96, 256, 5
    i = np.arange(n * k, dtype=np.float32)
    w = (np.sin(np.float32(0.017) * i) * (0.5 + 0.5 * np.cos(np.float32(0.0011) * i))).astype(np.float32).reshape(n, k)
    x = (np.cos(np.float32(0.019) * np.arange(b * k, dtype=np.float32)) - np.float32(0.25)).astype(np.float32).reshape(b, k)
    for qt in (O.INT8, O.INT4, O.F16, O.F32):
        together = port.qmat_linear(qt, w, x)
        for r in range(b):
            assert np.array_equal(together[r], port.qmat_linear(qt, w, x[r:r + 1])[0])


def test_attention_closed_form(port):
    # gpu/metal/backend_metal_ops.m:1049-1079
    k = np.zeros(4, np.float32)
    v = np.zeros(4, np.float32)
    out = port.self_attention(np.array([1, 0, 1, 0, 2, 3], np.float32), k, v, 0, 2, 1, 1, 2, 1.0)
    assert np.allclose(out, [2, 3], atol=1e-6)
    out = port.self_attention(np.array([1, 0, 0, 1, 4, 5], np.float32), k, v, 1, 2, 2, 1, 2, 1.0)
    e = np.exp(1.0)
    assert np.allclose(out, [(2 * e + 4) / (e + 1), (3 * e + 5) / (e + 1)], atol=1e-5)
    out = port.cross_attention(np.array([1, 2], np.float32), k, v, 1, 2, 1, 2, 1.0)
    assert np.allclose(out, [2, 3], atol=1e-6)


def test_argmax_rule(port):
    # first index wins ties; non-codes masked; EOS only when allowed (src/backend.c:825-847)
    logits = np.zeros(16, np.float32)
    logits[[3, 7]] = 2.0
    logits[12] = 9.0   # not a code
    logits[13] = 5.0   # eos
    assert port.argmax_constrained(logits, 10, 13, False) == 3
    assert port.argmax_constrained(logits, 10, 13, True) == 13
    assert port.argmax_constrained(np.full(16, -np.inf, np.float32), 10, 13, True) == 0


def test_edge_cases(port):
    # all-zero row: scale 1, zeros (src/qmat.c:48); all-zero activation: sx 0 (src/qmat.c:100-103)
    w = np.zeros((2, 32), np.float32)
    w[1, 5] = -3.0
    q, s = port.quantize_weight_int8(w)
    assert s[0] == 1.0 and not q[0].any() and q[1, 5] == -127
    q4, s4 = port.quantize_weight_int4(w)
    assert s4[0, 0] == 1.0 and (q4[0] == 0x88).all()
    assert q4[1, 2] == (8 | ((-7 + 8) << 4))   # index 5 is the high nibble of byte 2
    qa, sx = port.quantize_act_int8(np.zeros(32, np.float32))
    assert sx == 0.0 and not qa.any()
    # int4 refuses k not a multiple of 32 and falls back to the exact product (src/qmat.c:630)
    rng = np.random.default_rng(1)
    w = rng.normal(size=(8, 48)).astype(np.float32)
    x = rng.normal(size=(1, 48)).astype(np.float32)
    assert np.array_equal(port.qmat_linear(O.INT4, w, x), port.qmat_linear(O.F32, w, x))


# ---- fixtures generated from the reference ----------------------------------------
def test_linear_case_matches_reference_fixtures(port, golden):
    x, w, gain, bias = synth.make_linear_case(seed=1)
    nrm = port.layernorm(x, gain)
    assert np.array_equal(nrm[0], golden["linear_ln"])
    q8, s8 = port.quantize_weight_int8(w)
    q4, s4 = port.quantize_weight_int4(w)
    assert np.array_equal(np.array([crc(q8), crc(s8), crc(q4), crc(s4)], np.uint32), golden["linear_pack_crc"])
    qa, sx = port.quantize_act_int8(nrm[0])
    assert np.array_equal(qa, golden["linear_act_q"]) and sx == golden["linear_act_sx"]
    for name, qt in QT.items():
        assert np.array_equal(port.qmat_linear(qt, w, nrm, bias)[0], golden[f"linear_y_{name}"]), name


@pytest.mark.parametrize("name", ["f32", "int8", "int4"])
def test_tiny_decoder_matches_reference_fixtures(name, golden, tiny_model, tiny_memory):
    shape = synth.TINY
    pm = O.PortModel(tiny_model, QT[name])
    ps = pm.new_stream(tiny_memory, 64)
    if name == "f32":
        assert np.array_equal(ps.cross_k, golden["tiny_cross_k"])
        assert np.array_equal(ps.cross_v, golden["tiny_cross_v"])
    forced = synth.make_codes(shape, seed=7, frames=10)
    for f in range(10):
        hidden = ps.step(pm.embed_frame(forced[f]))
        tokens, _ = pm.heads_argmax(hidden, True)
        assert np.array_equal(hidden, golden[f"tiny_{name}_forced_hidden"][f]), (name, f)
        assert np.array_equal(tokens, golden[f"tiny_{name}_forced_tokens"][f])
    assert crc(ps.self_k[:, :10]) ^ crc(ps.self_v[:, :10]) == golden[f"tiny_{name}_forced_kv_crc"]
    row = pm.embed_frame(forced[0])
    for n in range(1, shape.layers + 1):
        ps.length = 10
        ps.set_layers(n)
        assert np.array_equal(ps.step(row), golden[f"tiny_{name}_layers"][n - 1])
    ps.set_layers(shape.layers)
    ps.length = 0
    start = synth.make_codes(shape, seed=9, frames=1)[0]
    tokens = ps.greedy_decode(start, 64, 4)
    assert np.array_equal(tokens, golden[f"tiny_{name}_greedy_tokens"])
    ps.close()
    pm.close()


def test_full_shape_first_frames_match_reference_fixtures(golden):
    """The 357M-parameter shape: the first two greedy frames of the int8 fixture
    (the CPU needs ~0.2 s per frame; the GPU tests cover all 512)."""
    shape = synth.MAGPIE_357M
    model = synth.make_model(shape, seed=21)
    pm = O.PortModel(model, O.INT8)
    ps = pm.new_stream(synth.make_memory(shape, seed=121), 8)
    codes = synth.make_codes(shape, seed=221, frames=1)[0].copy()
    want_tokens = golden["full_int8_s21_tokens"]
    want_hidden = golden["full_int8_s21_hidden"]
    for f in range(2):
        tokens, hidden, _ = ps.greedy_frame(codes, False)
        assert np.array_equal(tokens, want_tokens[f])
        assert np.array_equal(hidden, want_hidden[f])   # kept frames start 0, 1
    ps.close()
    pm.close()


# ---- the compiled reference itself ---------------------------------------------------
@needs_ref
def test_reference_self_tests_pass():
    rc, msg = O.Ref.get("strict").self_tests()
    assert rc == 0, msg
    rc, msg = O.Ref.get("fast").self_tests()
    assert rc == 0, msg


@needs_ref
@pytest.mark.parametrize("name", ["f32", "int8", "int4"])
def test_port_equals_compiled_reference(name, tiny_model, tiny_memory):
    shape = synth.TINY
    pm = O.PortModel(tiny_model, QT[name])
    rm = O.RefModel(tiny_model, QT[name], "strict")
    ps = pm.new_stream(tiny_memory, 48)
    rd = rm.new_decoder(tiny_memory, 48)
    assert np.array_equal(ps.cross_k, rd.cross_k) and np.array_equal(ps.cross_v, rd.cross_v)
    codes = synth.make_codes(shape, seed=17, frames=12)
    for f in range(12):
        row = pm.embed_frame(codes[f])
        hp, hr = ps.step(row), rd.step(row)
        assert np.array_equal(hp, hr)
        tp, lp = pm.heads_argmax(hp, True)
        tr, lr = rm.heads_argmax(hr, True)
        assert np.array_equal(tp, tr) and np.array_equal(lp, lr)
    assert np.array_equal(ps.self_k, rd.self_k) and np.array_equal(ps.self_v, rd.self_v)
    # the reference's batched step equals its single-slot step bit for bit
    rd2 = [rm.new_decoder(tiny_memory, 48) for _ in range(3)]
    rows = np.stack([pm.embed_frame(codes[f]) for f in range(3)])
    together = rm.step_batch(rd2, rows)
    for b in range(3):
        solo = rm.new_decoder(tiny_memory, 48)
        assert np.array_equal(solo.step(rows[b]), together[b])
        solo.close()
    for d in rd2:
        d.close()
    ps.close(); rd.close(); pm.close(); rm.close()


@needs_ref
def test_fast_reference_build_is_close_to_strict(tiny_model, tiny_memory):
    """The timed baseline (reference flags, -O3 -ffast-math -mavx2) and the parity
    oracle (strict flags) are the same code: they must agree to rounding."""
    shape = synth.TINY
    fast = O.RefModel(tiny_model, O.F32, "fast")
    strict = O.RefModel(tiny_model, O.F32, "strict")
    df, ds = fast.new_decoder(tiny_memory, 16), strict.new_decoder(tiny_memory, 16)
    pm = O.PortModel(tiny_model, O.F32)
    row = pm.embed_frame(synth.make_codes(shape, seed=2, frames=1)[0])
    assert rel_err(df.step(row), ds.step(row)) < 1e-5
    df.close(); ds.close(); fast.close(); strict.close(); pm.close()


@pytest.mark.parametrize("qtype,count", [(O.INT8, 20), (O.INT8, 9), (O.F32, 20), (O.INT4, 17)])
def test_port_prefill_equals_reference_decoder_run(qtype, count, tiny_model, tiny_memory):
    """The restated multi-row prefill (decoder_run with count > 1, src/graph.c:3506-3641)
    against the reference's own, bit for bit: hidden row of the last new row, the KV rows it
    appended, and a decode step on top; more than 16 rows take the f32 weights in both."""
    if not O.have_ref("strict"):
        pytest.skip("compiled reference absent")
    from mynah_tts_b200 import synth
    shape = synth.TINY
    rng = np.random.default_rng(31)
    first = rng.normal(0, 0.05, size=(3, shape.width)).astype(np.float32)
    rows = rng.normal(0, 0.05, size=(count, shape.width)).astype(np.float32)
    after = rng.normal(0, 0.05, size=(shape.width,)).astype(np.float32)
    rm = O.RefModel(tiny_model, qtype, "strict")
    rd = rm.new_decoder(tiny_memory, 40)
    pm = O.PortModel(tiny_model, qtype)
    ps = pm.new_stream(tiny_memory, 40)
    for r in first:                                   # a few cached rows first
        assert np.array_equal(ps.step(r), rd.step(r))
    want, got = rd.run(rows), ps.prefill(rows)
    assert np.array_equal(got, want)
    assert rd.length == ps.length == 3 + count
    assert np.array_equal(ps.self_k[:, :3 + count], rd.self_k[:, :3 + count])
    assert np.array_equal(ps.self_v[:, :3 + count], rd.self_v[:, :3 + count])
    assert np.array_equal(ps.step(after), rd.step(after))
    rd.close(); rm.close(); ps.close(); pm.close()


def test_port_text_encoder_equals_reference(tiny_model):
    """The restated text encoder (encode_text, src/graph.c:709-748: embedding rows, six-tensor
    layers with causal self attention and the kernel-3 causal convolution feed-forward, output
    norm) against the reference's own, bit for bit."""
    if not O.have_ref("strict"):
        pytest.skip("compiled reference absent")
    import copy
    from mynah_tts_b200 import synth
    model = copy.copy(tiny_model)
    model = type(tiny_model)(shape=tiny_model.shape, seed=tiny_model.seed, tensors=dict(tiny_model.tensors))
    enc = synth.TINY_ENCODER
    tensors = synth.add_encoder(model, enc, seed=91)
    rm = O.RefModel(model, O.INT8, "strict")          # the cache format must not matter: linear() is f32
    rng = np.random.default_rng(5)
    for count in (1, 2, 19, 40):
        ids = rng.integers(0, enc.vocab, size=count).astype(np.int32)
        want = rm.encode_text(enc, ids)
        got = O.Port.get().encode_text(tensors, enc, ids)
        assert np.array_equal(got, want), count
    rm.close()
