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


def static_attention(qkv, dk, dv, position, stride, valid, heads, hw, scale, dout):
    call(capi.lib().mynah_b200_self_attention_static, qkv.ptr, dk.ptr, dv.ptr, position, stride, valid,
         heads, hw, C.c_float(scale), dout.ptr, None)


def test_static_entry_matches_the_allocating_one_twice_in_a_row():
    heads, hw = 12, 64
    width = heads * hw
    cap = 300
    rng = np.random.default_rng(99)
    k = rng.normal(size=(cap, width)).astype(np.float32)
    v = rng.normal(size=(cap, width)).astype(np.float32)
    scale = float(np.float32(1.0) / np.sqrt(np.float32(hw)))
    be = Backend("f32", strict=False)
    # two independent copies of the cache: one per entry point
    k_ref, v_ref = be.to_device(k), be.to_device(v)
    k_sta, v_sta = be.to_device(k), be.to_device(v)
    out_ref, out_sta = be.dev_alloc(width), be.dev_alloc(width)
    for position in (257, 40):            # many chunks, then few: stale partials must not leak
        qkv = rng.normal(size=(3 * width,)).astype(np.float32)
        dqkv = be.to_device(qkv)
        be.self_attention_dev(dqkv, k_ref, v_ref, position, width, position + 1, heads, hw, scale, out_ref)
        want = be.d2h(out_ref, width)
        static_attention(dqkv, k_sta, v_sta, position, width, position + 1, heads, hw, scale, out_sta)
        device_synchronize()               # the static call ran on the default stream
        got = be.d2h(out_sta, width)
        assert rel_err(got, want) < 3e-6, position
        assert np.array_equal(be.d2h(k_sta, k.size), be.d2h(k_ref, k.size))
        assert np.array_equal(be.d2h(v_sta, v.size), be.d2h(v_ref, v.size))
        dqkv.free()
    # beyond the fixed scratch: refused with a clear message, nothing launched
    with pytest.raises(MynahB200Error, match="static scratch"):
        static_attention(k_sta, k_sta, v_sta, 0, width, 5000, heads, hw, scale, out_sta)
    with pytest.raises(MynahB200Error, match="head width"):
        static_attention(k_sta, k_sta, v_sta, 0, 36, 1, 12, 3, scale, out_sta)
    for buf in (k_ref, v_ref, k_sta, v_sta, out_ref, out_sta):
        buf.free()
    be.close()
