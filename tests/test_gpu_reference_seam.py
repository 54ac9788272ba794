"""The reference's own decoder_run driving this library through the backend seam.

oracle/_ref/libmynah_ref_b200.so is the reference's src/graph.c and src/backend.c (its CUDA
branch, -DMYNAH_ENABLE_CUDA) linked against libmynah_b200.so, plus the seven assignments
that wire the resident-attention ops (oracle/harness_ref_cuda.c).  decoder_run(count = 1)
then takes its resident path (src/graph.c:3363-3491): h2d, batch_begin, layer_norm_inplace,
matmul_d2d, self_attention_dev, residual_inplace, cross_attention_dev, gelu_inplace, sync,
d2h -- every one of them served by this library, with MYNAH_QUANT quantizing behind the
seam.  The same rows go through the reference's CPU build (decoder_run ->
decoder_step_batch); in strict mode hidden rows and KV must agree bit for bit for the
integer formats.
"""
import os

import numpy as np
import pytest

from conftest import rel_err
from mynah_tts_b200 import synth
from oracle import oracle as O

pytestmark = pytest.mark.gpu
NAMES = {O.F32: "f32", O.INT8: "int8", O.INT4: "int4"}


def _open_pair(model, qtype, strict, monkeypatch):
    monkeypatch.setenv("MYNAH_QUANT", NAMES[qtype])
    monkeypatch.setenv("MYNAH_B200_STRICT", "1" if strict else "0")
    monkeypatch.delenv("MYNAH_GPU_RESIDENT", raising=False)
    gpu = O.RefModel(model, qtype, "b200")
    cpu = O.RefModel(model, qtype, "strict")
    return gpu, cpu


@pytest.mark.skipif(not (O.have_ref("b200") and O.have_ref("strict")), reason="compiled reference absent")
@pytest.mark.parametrize("shape_name,qtype,strict", [("tiny", O.INT8, True), ("tiny", O.INT4, True),
                                                     ("tiny", O.F32, True), ("tiny", O.INT8, False),
                                                     ("full", O.INT8, True)])
def test_reference_decoder_run_resident_path(shape_name, qtype, strict, tiny_model, tiny_memory, monkeypatch):
    if shape_name == "tiny":
        shape, model, memory, frames = synth.TINY, tiny_model, tiny_memory, 16
    else:
        shape = synth.MAGPIE_357M
        model = synth.make_model(shape, seed=41)
        memory = synth.make_memory(shape, seed=141)
        frames = 8
    gpu, cpu = _open_pair(model, qtype, strict, monkeypatch)
    assert gpu.backend_name == "cuda" and gpu.resident          # the resident step is open ...
    assert cpu.backend_name != "cuda" and not cpu.resident      # ... and only there
    dg, dc = gpu.new_decoder(memory, frames + 4), cpu.new_decoder(memory, frames + 4)
    exact = strict and qtype in (O.INT8, O.INT4)
    tol = 2e-5 if strict else {O.INT8: 1e-2, O.INT4: 2e-2, O.F32: 1e-3}[qtype]
    # decoder_cache_init ran its kv_net products through the seam's host matmul (f32 whatever
    # MYNAH_QUANT says, src/graph.c:3002-3027)
    assert rel_err(dg.cross_k, dc.cross_k) < 1e-5 and rel_err(dg.cross_v, dc.cross_v) < 1e-5
    if strict:
        assert np.array_equal(dg.cross_k, dc.cross_k) and np.array_equal(dg.cross_v, dc.cross_v)
    codes = synth.make_codes(shape, seed=17, frames=frames)
    for f in range(frames):
        row = cpu.embed_frame(codes[f])
        want = dc.run(row)
        got = dg.run(row)
        assert rel_err(got, want) < tol, (shape_name, f)
        if exact:
            assert np.array_equal(got, want), (shape_name, NAMES[qtype], f)
    assert dg.length == frames and dc.length == frames
    # the resident path keeps K/V on the device: the host arrays of the GPU-backed cache were
    # never written, the device copy holds what the CPU build appended
    assert not dg.self_k[:, :frames].any()
    dg.download_kv()
    assert rel_err(dg.self_k[:, :frames], dc.self_k[:, :frames]) < tol
    assert rel_err(dg.self_v[:, :frames], dc.self_v[:, :frames]) < tol
    if exact:
        assert np.array_equal(dg.self_k[:, :frames], dc.self_k[:, :frames])
        assert np.array_equal(dg.self_v[:, :frames], dc.self_v[:, :frames])
    dg.close(); dc.close(); gpu.close(); cpu.close()


@pytest.mark.skipif(not (O.have_ref("b200") and O.have_ref("strict")), reason="compiled reference absent")
def test_reference_decode_codec_cpu_path_with_seam_ops(monkeypatch):
    """MYNAH_METAL_CPU_CODEC=1 keeps the reference on its CPU codec loop (src/graph.c:2517-2518),
    which still hands every convolution to the backend as HOST buffers (conv1d_causal,
    src/graph.c:2033-2046) and every Snake through upload / snake_dev / download (half_snake,
    src/graph.c:2262-2280).  Strict mode: one sequential sum per output and the host libm's
    sinf, so the samples are the CPU build's bit for bit."""
    import sys
    import os as _os
    sys.path.insert(0, _os.path.join(_os.path.dirname(_os.path.abspath(__file__)), "golden"))
    import make_golden_frontend as G
    monkeypatch.setenv("MYNAH_METAL_CPU_CODEC", "1")
    shape = synth.CodecShape()
    model = G.bare_model(lambda m: synth.add_codec(m, shape, seed=61))
    gpu, cpu = _open_pair(model, O.F32, True, monkeypatch)
    codes = synth.make_codec_codes(shape, 64, 2)
    got, want = gpu.decode_codec(codes), cpu.decode_codec(codes)
    assert np.array_equal(got, want)
    gpu.close(); cpu.close()


@pytest.mark.skipif(not (O.have_ref("b200") and O.have_ref("strict")), reason="compiled reference absent")
@pytest.mark.parametrize("strict", [True, False])
def test_reference_decode_codec_resident_path(strict, monkeypatch):
    """With the resident ops wired, the reference's decode_codec takes decode_codec_resident
    (src/graph.c:2511-2638): dev_alloc, h2d, conv1d on DEVICE buffers, snake_dev,
    conv_transpose_dev, copy_dev, residual_inplace, scale_dev, clip_dev, d2h -- all served by
    this library.  Against the reference's CPU build on the same codes: the resident form
    scales the branch sum by 1/3 where the CPU form divides by 3, so the samples agree to
    rounding, not bit for bit."""
    import sys
    import os as _os
    sys.path.insert(0, _os.path.join(_os.path.dirname(_os.path.abspath(__file__)), "golden"))
    import make_golden_frontend as G
    shape = synth.CodecShape()
    model = G.bare_model(lambda m: synth.add_codec(m, shape, seed=61))
    gpu, cpu = _open_pair(model, O.F32, strict, monkeypatch)
    assert gpu.backend_name == "cuda" and gpu.resident
    for frames in (1, 3):
        codes = synth.make_codec_codes(shape, 62 + frames, frames)
        want = cpu.decode_codec(codes)
        got = gpu.decode_codec(codes)
        assert got.shape == want.shape == (frames * 1024,)
        assert np.abs(got - want).max() < (2e-6 if strict else 1e-4), frames
    gpu.close(); cpu.close()


@pytest.mark.skipif(not (O.have_ref("b200") and O.have_ref("strict")), reason="compiled reference absent")
@pytest.mark.parametrize("qtype", [O.INT8, O.F32])
def test_reference_local_frame_device_path(qtype, monkeypatch):
    """One request's stacked frame through the reference's own local transformer: with the
    resident ops wired its local_step_device runs (src/graph.c:1101-1159, 1403-1520: copy_dev,
    residual_inplace, layer_norm_inplace, matmul_d2d, self_attention_dev, gelu_inplace, the
    head's matmul_d2d with bias, argmax_dev or d2h of the logits) through this library.
    Strict mode, greedy and sampling: the codes, EOS reports and RNG state of its CPU build."""
    shape = synth.TINY_LOCAL
    model = synth.make_model(shape, seed=3)
    gpu, cpu = _open_pair(model, qtype, True, monkeypatch)
    assert gpu.resident
    rng = np.random.default_rng(43)
    for temp, topk, seed, allow in ((0.0, 0, 1, 1), (0.7, 8, 0x1234, 1), (1.3, 5, 99, 0)):
        rows = rng.normal(0.0, 1.0, size=(1, shape.width)).astype(np.float32)
        lg, lc = gpu.new_local(shape.vocab), cpu.new_local(shape.vocab)
        got = gpu.local_frame([lg], rows, [temp], [topk], [seed], [allow])
        want = cpu.local_frame([lc], rows, [temp], [topk], [seed], [allow])
        assert np.array_equal(got[0], want[0]), (temp, topk)          # codes
        assert np.array_equal(got[1], want[1]) and np.array_equal(got[2], want[2])
        assert got[3] == want[3]                                       # xorshift state
        lg.close(); lc.close()
    gpu.close(); cpu.close()


@pytest.mark.skipif(not (O.have_ref("b200") and O.have_ref("strict")), reason="compiled reference absent")
def test_reference_encode_text_and_prefill_through_host_matmul(tiny_model, tiny_memory, monkeypatch):
    """The reference's many-row paths keep their host loops and hand only the products to the
    backend: encode_text (linear -> matmul with host buffers, graph_sgemm for the attention,
    src/graph.c:259-265, 446-452) and decoder_run with count > 1 (src/graph.c:3506-3641).
    Strict mode: the seam's f32 matmul and sgemm keep one sequential sum per output, so both
    equal the CPU build bit for bit."""
    enc = synth.TINY_ENCODER
    model = type(tiny_model)(shape=tiny_model.shape, seed=tiny_model.seed, tensors=dict(tiny_model.tensors))
    synth.add_encoder(model, enc, seed=91)
    gpu, cpu = _open_pair(model, O.F32, True, monkeypatch)
    ids = np.random.default_rng(8).integers(0, enc.vocab, size=21).astype(np.int32)
    assert np.array_equal(gpu.encode_text(enc, ids), cpu.encode_text(enc, ids))
    rows = np.random.default_rng(9).normal(0, 0.05, size=(20, tiny_model.shape.width)).astype(np.float32)
    dg, dc = gpu.new_decoder(tiny_memory, 32), cpu.new_decoder(tiny_memory, 32)
    got, want = dg.run(rows), dc.run(rows)
    assert np.array_equal(got, want)
    assert dg.length == dc.length == 20
    dg.close(); dc.close(); gpu.close(); cpu.close()
