"""The allocation-free self-attention entry point (collected last on purpose).

Some callers of this library cannot allocate device memory at all -- a
real-time audio thread that must never block in an allocator, or a plugin whose
host owns the memory pool.  `mynah_b200_self_attention_static` serves them from
a fixed scratch array inside the library.  This test calls it through the C ABI
twice in a row on different positions and checks each result, and the appended
KV rows, against the ordinary entry point `mynah_cuda_self_attention_dev`
(which allocates its scratch), to the tolerance the attention tests use."""
import ctypes as C

import numpy as np
import pytest

from conftest import rel_err
from mynah_tts_b200 import capi
from mynah_tts_b200.backend import Backend, MynahB200Error, call

pytestmark = pytest.mark.gpu


def device_synchronize():
    """cudaDeviceSynchronize through the CUDA runtime the library itself links."""
    rt = C.CDLL("libcudart.so.12")
    assert rt.cudaDeviceSynchronize() == 0


def static_attention(qkv, dk, dv, position, stride, valid, heads, hw, scale, dout, stream=None):
    call(capi.lib().mynah_b200_self_attention_static, qkv.ptr, dk.ptr, dv.ptr, position, stride, valid,
         heads, hw, C.c_float(scale), dout.ptr, stream)


# heads, head width, cache stride, capacity, positions of the two calls in a row, own stream
CASES = [(12, 64, 768, 300, (257, 40), False),      # the decoder's shape: many chunks, then few
         (5, 128, 704, 80, (70, 3), True),          # five heads in boxes of two and one; padded rows
         (6, 4, 32, 40, (33, 0), False),            # the narrowest head the kernel takes
         (2, 64, 128, 4096, (4095, 100), True)]     # the largest request the fixed scratch holds


@pytest.mark.parametrize("heads,hw,stride,cap,positions,own_stream", CASES)
def test_static_entry_matches_the_allocating_one_twice_in_a_row(heads, hw, stride, cap, positions, own_stream, port):
    width = heads * hw
    rng = np.random.default_rng(99)
    k = rng.normal(size=(cap, stride)).astype(np.float32)
    v = rng.normal(size=(cap, stride)).astype(np.float32)
    scale = float(np.float32(1.0) / np.sqrt(np.float32(hw)))
    be = Backend("f32", strict=False)
    rt = C.CDLL("libcudart.so.12")
    stream = C.c_void_p()
    if own_stream:
        assert rt.cudaStreamCreate(C.byref(stream)) == 0
    # two independent copies of the cache: one per entry point (and a third on the host for
    # the CPU checker)
    k_ref, v_ref = be.to_device(k), be.to_device(v)
    k_sta, v_sta = be.to_device(k), be.to_device(v)
    k_cpu, v_cpu = k.copy(), v.copy()
    out_ref, out_sta = be.dev_alloc(width), be.dev_alloc(width)
    for position in positions:            # stale partials of the longer call must not leak into the shorter
        qkv = rng.normal(size=(3 * width,)).astype(np.float32)
        dqkv = be.to_device(qkv)
        be.self_attention_dev(dqkv, k_ref, v_ref, position, stride, position + 1, heads, hw, scale, out_ref)
        want = be.d2h(out_ref, width)
        static_attention(dqkv, k_sta, v_sta, position, stride, position + 1, heads, hw, scale, out_sta,
                         stream if own_stream else None)
        device_synchronize()               # the static call ran on its own or the default stream
        got = be.d2h(out_sta, width)
        # same 32-row chunks, same per-chunk arithmetic, partials merged in chunk order by the
        # same routine: the two entry points agree bit for bit
        assert np.array_equal(got, want), position
        cpu = port.self_attention(qkv, k_cpu, v_cpu, position, stride, position + 1, heads, hw, scale)
        assert rel_err(got, cpu) < 3e-6, position
        assert np.array_equal(be.d2h(k_sta, k.size), be.d2h(k_ref, k.size))
        assert np.array_equal(be.d2h(v_sta, v.size), be.d2h(v_ref, v.size))
        assert np.array_equal(be.d2h(k_sta, k.size).reshape(cap, stride), k_cpu)
        dqkv.free()
    if own_stream:
        assert rt.cudaStreamDestroy(stream) == 0
    for buf in (k_ref, v_ref, k_sta, v_sta, out_ref, out_sta):
        buf.free()
    be.close()


def test_static_entry_refuses_what_its_scratch_cannot_hold():
    be = Backend("f32", strict=False)
    buf = be.dev_alloc(3 * 768)
    scale = 0.125
    # beyond the fixed scratch: refused with a clear message, nothing launched
    with pytest.raises(MynahB200Error, match="static scratch"):
        static_attention(buf, buf, buf, 0, 768, 5000, 12, 64, scale, buf)
    with pytest.raises(MynahB200Error, match="static scratch"):
        static_attention(buf, buf, buf, 0, 768, 1, 48, 16, scale, buf)       # more than 32 heads
    with pytest.raises(MynahB200Error, match="static scratch"):
        static_attention(buf, buf, buf, 0, 1024, 1, 8, 128, scale, buf)      # wider than 768
    with pytest.raises(MynahB200Error, match="head width"):
        static_attention(buf, buf, buf, 0, 36, 1, 12, 3, scale, buf)
    buf.free()
    be.close()
