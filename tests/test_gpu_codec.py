"""The codec decoder (decode_codec, src/graph.c:2640-2780) on the GPU against the CPU restatement,
which tests/test_oracle_frontend.py pins bit for bit against the reference's own decode_codec,
and against samples the reference produced (tests/golden/golden_frontend.npz)."""
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
import make_golden_frontend as G  # noqa: E402
from conftest import rel_err  # noqa: E402
from mynah_tts_b200 import capi, synth  # noqa: E402
from mynah_tts_b200.backend import Backend, Codec, DeviceBuffer, call, fp  # noqa: E402
from oracle import oracle as O  # noqa: E402

pytestmark = pytest.mark.gpu
GOLDEN = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "golden_frontend.npz"))


MODES = [pytest.param(True, False, id="strict"), pytest.param(False, False, id="fast-tensor-core"),
         pytest.param(False, True, id="fast-simt")]


@pytest.mark.parametrize("strict,no_tc", MODES)
def test_codec_small_shape_stagewise(strict, no_tc, monkeypatch):
    """Base 96 (channels 48 .. 3): every stage against the oracle.  Fast mode runs the
    residual-layer convolutions on the tensor cores over split f16 planes, or (with
    MYNAH_B200_NO_TC) as FMA sums in the SIMT kernel."""
    if no_tc:
        monkeypatch.setenv("MYNAH_B200_NO_TC", "1")
    shape = synth.TINY_CODEC
    tensors = synth.add_codec(None, shape, seed=2)
    be = Backend("int8", strict=strict)          # the weight format must not matter: the codec is f32
    codec = Codec(be, tensors, shape, max_frames=8)
    for frames in (1, 5):
        codes = synth.make_codec_codes(shape, 4 + frames, frames)
        for stop in (1, 2, 3, 4, 5, 6, 0):
            want = O.Port.get().codec_decode(tensors, shape, codes, stop_after=stop)
            got = codec.decode(codes, stop_after=stop)
            assert got.shape == want.shape
            if strict:
                assert np.array_equal(got, want), (frames, stop)          # bit for bit, sinf included
            else:
                assert rel_err(got, want) < 1e-4, (frames, stop)
    codec.close(); be.close()


@pytest.mark.parametrize("strict,no_tc", MODES)
def test_codec_reference_size_matches_golden(strict, no_tc, monkeypatch):
    """Base 864, the reference's fixed shape, against samples of the reference's own decode_codec."""
    if no_tc:
        monkeypatch.setenv("MYNAH_B200_NO_TC", "1")
    shape = synth.CodecShape()
    tensors = synth.add_codec(None, shape, seed=G.CODEC_SEED)
    be = Backend("f32", strict=strict)
    codec = Codec(be, tensors, shape, max_frames=8)
    for frames in G.CODEC_FRAMES:
        codes = synth.make_codec_codes(shape, G.CODES_SEED, frames)
        got = codec.decode(codes)
        want = GOLDEN[f"codec_{frames}"]
        if strict:
            assert np.array_equal(got, want), frames
        else:
            assert np.abs(got - want).max() < 1e-4, frames
    codec.close(); be.close()


@pytest.mark.parametrize("strict", [True, False], ids=["strict", "fast-tensor-core"])
def test_codec_long_request_is_causal(strict):
    """256 frames (12 s of audio), beyond what the CPU oracle finishes in seconds: every
    operation is causal, so the head of a long decode equals the decode of the head -- which is
    checked against the oracle -- and a second decode repeats the first."""
    shape = synth.CodecShape()
    tensors = synth.add_codec(None, shape, seed=13)
    be = Backend("f32", strict=strict)
    codec = Codec(be, tensors, shape, max_frames=256)
    codes = synth.make_codec_codes(shape, 21, 256)
    whole = codec.decode(codes)
    assert whole.shape == (256 * 1024,) and np.abs(whole).max() <= 1.0 and whole.std() > 0.05
    head = codec.decode(codes[:, :2])
    want = O.Port.get().codec_decode(tensors, shape, codes[:, :2])
    mid = codec.decode(codes[:, :97])
    if strict:
        assert np.array_equal(whole[:2 * 1024], head)
        assert np.array_equal(head, want)
        assert np.array_equal(whole[:97 * 1024], mid)
    else:
        # the tile grid of the tensor-core convolutions is the same for every length, so the
        # head is reproduced exactly here too; against the oracle to f16-split rounding
        assert np.array_equal(whole[:2 * 1024], head)
        assert np.array_equal(whole[:97 * 1024], mid)
        assert np.abs(head - want).max() < 1e-4
    assert np.array_equal(whole, codec.decode(codes))
    codec.close(); be.close()


def test_codec_arithmetic_is_the_codecs_choice():
    """A strict backend (token-identical decoder) may carry a tensor-core codec, and a fast one
    a reference-order codec."""
    shape = synth.TINY_CODEC
    tensors = synth.add_codec(None, shape, seed=2)
    codes = synth.make_codec_codes(shape, 8, 3)
    want = O.Port.get().codec_decode(tensors, shape, codes)
    strict_be, fast_be = Backend("int8", strict=True), Backend("int8", strict=False)
    exact = Codec(fast_be, tensors, shape, max_frames=4, arithmetic=1)
    quick = Codec(strict_be, tensors, shape, max_frames=4, arithmetic=2)
    assert np.array_equal(exact.decode(codes), want)
    got = quick.decode(codes)
    assert not np.array_equal(got, want) and np.abs(got - want).max() < 1e-4
    with pytest.raises(RuntimeError, match="arithmetic"):
        Codec(fast_be, tensors, shape, max_frames=4, arithmetic=3)
    exact.close(); quick.close(); strict_be.close(); fast_be.close()


def test_codec_refusals():
    shape = synth.TINY_CODEC
    tensors = synth.add_codec(None, shape, seed=2)
    be = Backend("f32", strict=False)
    codec = Codec(be, tensors, shape, max_frames=4)
    with pytest.raises(RuntimeError, match="frame count"):
        codec.decode(synth.make_codec_codes(shape, 1, 5))
    with pytest.raises(RuntimeError, match="codec shape"):
        Codec(be, tensors, synth.CodecShape(base=100), max_frames=4)
    codec.close(); be.close()


@pytest.mark.parametrize("strict", [True, False], ids=["strict", "fast"])
def test_seam_codec_ops(strict):
    """The three codec entries of the reference's backend seam: conv1d (host buffers, as the
    reference's CUDA backend serves it), im2col and snake_dev (device buffers)."""
    be = Backend("f32", strict=strict)
    lib = capi.lib()
    rng = np.random.default_rng(3)
    for ic, oc, L, K, dil in ((32, 96, 9, 7, 1), (54, 54, 300, 11, 5), (27, 1, 700, 3, 1), (48, 48, 130, 3, 3)):
        w = rng.normal(0, 1 / np.sqrt(ic * K), size=(oc, ic, K)).astype(np.float32)
        b = rng.normal(0, 0.1, size=(oc,)).astype(np.float32)
        x = rng.normal(0, 1, size=(ic, L)).astype(np.float32)
        be.keep(w); be.keep(b)
        out = np.empty((oc, L), np.float32)
        call(lib.mynah_cuda_conv1d, be.state, x.ctypes.data_as(capi.C.c_void_p), out.ctypes.data_as(capi.C.c_void_p),
             ic, oc, L, K, dil, fp(w), fp(b))
        # scalar product over p = i * K + k in order (src/backend.c:343-354), then 1 * sum + 1 * bias
        cols = np.zeros((ic * K, L), np.float32)
        for i in range(ic):
            for k in range(K):
                shift = (K - 1 - k) * dil
                if shift < L:
                    cols[i * K + k, shift:] = x[i, :L - shift]
        want = np.empty((oc, L), np.float32)
        for o in range(oc):
            acc = np.zeros(L, np.float32)
            wr = w[o].reshape(-1)
            for p_ in range(ic * K):
                acc = acc + wr[p_] * cols[p_]          # float32 product, float32 sum, in order
            want[o] = acc + b[o]
        if strict:
            assert np.array_equal(out, want), (ic, oc, L, K, dil)
        else:
            assert rel_err(out, want) < 1e-5
        # im2col on device buffers
        din, dcol = DeviceBuffer(be, ic * L), DeviceBuffer(be, ic * K * L)
        call(lib.mynah_cuda_h2d, be.state, fp(x), din.ptr, ic * L)
        call(lib.mynah_cuda_im2col, be.state, din.ptr, dcol.ptr, ic, L, K, dil)
        got_cols = np.empty((ic * K, L), np.float32)
        call(lib.mynah_cuda_d2h, be.state, dcol.ptr, fp(got_cols), ic * K * L)
        assert np.array_equal(got_cols, cols)
        din.free(); dcol.free()
    # snake_dev: the CPU backend's form v + sn * sn * (1 / (a + 1e-9)) on the first channels
    ch, L = 54, 1000
    x = rng.normal(0, 2.0, size=(ch, L)).astype(np.float32)
    alpha = rng.normal(1.0, 0.1, size=(ch,)).astype(np.float32)
    be.keep(alpha)
    d = DeviceBuffer(be, ch * L)
    call(lib.mynah_cuda_h2d, be.state, fp(x), d.ptr, ch * L)
    call(lib.mynah_cuda_snake_dev, be.state, d.ptr, fp(alpha), ch, L, ch // 2)
    got = np.empty_like(x)
    call(lib.mynah_cuda_d2h, be.state, d.ptr, fp(got), ch * L)
    a = alpha[:ch // 2, None]
    sn = np.sin((a * x[:ch // 2]).astype(np.float32)).astype(np.float32)      # host libm, as the reference
    want = x.copy()
    want[:ch // 2] = x[:ch // 2] + sn * sn * (np.float32(1.0) / (a + np.float32(1e-9)))
    want[ch // 2:] = np.where(x[ch // 2:] < 0, x[ch // 2:] * np.float32(0.01), x[ch // 2:])
    assert np.array_equal(got[ch // 2:], want[ch // 2:])
    assert np.abs(got - want).max() < 2e-6
    d.free(); be.close()
