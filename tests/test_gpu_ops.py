"""GPU parity of the single ops, through the C ABI, against the CPU oracle:
weight packing and activation quantization bit for bit, the quantized products
per format, LayerNorm, GELU, attention, argmax, and the reference's known
answers.  Tolerances: strict mode is compared bit for bit wherever the
arithmetic is integer or uses only +,-,*,/,sqrt; fast mode to 2e-6 relative
(f32 reduction order only); transcendental paths to 1e-6."""
import numpy as np
import pytest

from conftest import rel_err
from mynah_tts_b200 import synth
from mynah_tts_b200.backend import F16, F32, INT4, INT8, Backend, MynahB200Error
from oracle import oracle as O

pytestmark = pytest.mark.gpu
QT = {"f32": F32, "int8": INT8, "int4": INT4, "f16": F16}


@pytest.fixture(scope="module")
def backends():
    made = {}

    def get(quant, strict):
        key = (quant, strict)
        if key not in made:
            made[key] = Backend(quant, strict=strict)
        return made[key]
    yield get
    for b in made.values():
        b.close()


def test_backend_self_test_known_answers():
    # gpu/cuda/backend_cuda.cu:514-529 of the reference: matmul {1.5,1.5,4,8,-0.5,0,3,3.5},
    # sgemm {1,2,3,6,-1,0.5,2,1.5}
    be = Backend(from_env=True)
    be.self_test()
    x = np.array([[1, 2, 3], [-1, 0.5, 2]], np.float32)
    w = np.array([[1, 0, 0], [0, 1, 0], [0, 0, 1], [1, 1, 1]], np.float32)
    y = be.matmul(x, w, np.array([0.5, -0.5, 1, 2], np.float32))
    assert np.allclose(y.ravel(), [1.5, 1.5, 4, 8, -0.5, 0, 3, 3.5], atol=1e-5)
    c = np.zeros((2, 4), np.float32)
    be.sgemm(0, 1, 2, 4, 3, 1.0, x, 3, w, 3, 0.0, c, 4)
    assert np.allclose(c.ravel(), [1, 2, 3, 6, -1, 0.5, 2, 1.5], atol=1e-5)
    assert be.launch_count > 0
    be.close()


@pytest.mark.parametrize("shape", [(3072, 768), (200, 256), (7, 32), (96, 3072), (5, 8192)])
def test_weight_packing_is_bit_exact(shape, backends, port):
    rng = np.random.default_rng(shape[0])
    w = rng.normal(0, 0.02, size=shape).astype(np.float32)
    w[1] = 0.0                      # an all-zero row / group: scale 1 (src/qmat.c:48,75)
    w[2, ::3] *= 40.0               # outliers
    be = backends("f32", False)
    q, s = be.pack_weight(INT8, w)
    rq, rs = port.quantize_weight_int8(w)
    assert np.array_equal(q, rq) and np.array_equal(s, rs)
    q, s = be.pack_weight(INT4, w)
    rq, rs = port.quantize_weight_int4(w)
    assert np.array_equal(q, rq) and np.array_equal(s, rs)
    q, _ = be.pack_weight(F16, w)
    assert np.array_equal(q, port.quantize_weight_f16(w))


def test_int4_packing_refuses_ragged_k(backends):
    with pytest.raises(MynahB200Error):
        backends("f32", False).pack_weight(INT4, np.ones((4, 48), np.float32))


@pytest.mark.parametrize("k", [768, 128, 3072, 33, 8192])
def test_activation_quantization_is_bit_exact(k, backends, port):
    rng = np.random.default_rng(k)
    x = rng.normal(size=(6, k)).astype(np.float32)
    x[1] = 0.0                       # all-zero vector: zeros, scale 0 (src/qmat.c:100-103)
    x[2] *= 1e-20
    x[3, 0] = 1e20
    q, sx = backends("f32", False).quantize_act(x)
    for r in range(6):
        rq, rsx = port.quantize_act_int8(x[r])
        assert np.array_equal(q[r], rq) and sx[r] == rsx


def test_linear_case_against_reference_fixture(backends, golden):
    """The single-op configuration: x [1,768], W [3072,768], LayerNorm + bias."""
    x, w, gain, bias = synth.make_linear_case(seed=1)
    for name in ("int8", "int4", "f32"):
        y = backends(name, True).qmat_linear(w, x, bias, gain)[0]
        want = golden[f"linear_y_{name}"]
        if name == "f32":
            assert rel_err(y, want) < 2e-6
        else:
            assert np.array_equal(y, want), name      # exact integer sums, ordered f32 tail
        y = backends(name, False).qmat_linear(w, x, bias, gain)[0]
        assert rel_err(y, want) < (2e-2 if name == "int4" else 5e-3)


@pytest.mark.parametrize("name", ["int8", "int4", "f16", "f32"])
@pytest.mark.parametrize("n,k,count", [(3072, 768, 1), (768, 3072, 3), (200, 256, 5), (128, 768, 16),
                                       (48, 32, 2), (2304, 768, 17), (10, 8192, 1), (9, 24, 2)])
def test_products_match_oracle(name, n, k, count, backends, port):
    """out = x W^T + b for every format and for shapes that exercise every lane
    split (rows not a multiple of the warp tile, k = one group, k beyond the
    quantized limit's neighbours, 17 rows = past the quantized row limit)."""
    rng = np.random.default_rng(n * 31 + k)
    w = rng.normal(0, 0.02, size=(n, k)).astype(np.float32)
    x = rng.normal(size=(count, k)).astype(np.float32)
    bias = rng.normal(0, 0.01, size=(n,)).astype(np.float32)
    qt = QT[name] if count <= 16 else F32           # src/qmat.c:773-774
    want = port.qmat_linear(qt, w, x, bias)
    got = backends(name, False).qmat_linear(w, x, bias)
    exact = qt in (INT8, INT4) and not (qt == INT4 and k % 32)
    if exact:
        assert np.array_equal(got, want)
    else:
        assert rel_err(got, want) < 3e-6
    assert np.array_equal(got, backends(name, False).qmat_linear(w, x, bias))   # deterministic


def test_rows_do_not_depend_on_their_batch(backends):
    """src/qmat.c:1107-1179 asserts this with memcmp; same here, every format."""
    rng = np.random.default_rng(5)
    w = rng.normal(0, 0.02, size=(96, 256)).astype(np.float32)
    x = rng.normal(size=(5, 256)).astype(np.float32)
    for name in QT:
        be = backends(name, False)
        together = be.qmat_linear(w, x)
        for r in range(5):
            assert np.array_equal(together[r], be.qmat_linear(w, x[r:r + 1])[0]), name


@pytest.mark.parametrize("width", [768, 192, 4, 3072, 50])
def test_layernorm(width, backends, port):
    rng = np.random.default_rng(width)
    x = (rng.normal(size=(3, width)) * 3 + 0.5).astype(np.float32)
    gain = rng.normal(1, 0.01, size=(width,)).astype(np.float32)
    want = port.layernorm(x, gain)
    for strict in (True, False):
        be = backends("f32", strict)
        din, dout = be.to_device(x), be.dev_alloc(x.size)
        be.layer_norm_inplace(din, dout, gain, 3, width)
        got = be.d2h(dout, x.size).reshape(x.shape)
        if strict:
            assert np.array_equal(got, want)       # sequential sums, IEEE sqrt and divide
        else:
            assert rel_err(got, want) < 2e-6
        din.free(); dout.free()


def test_gelu_residual_scale_clip_copy(backends, port):
    rng = np.random.default_rng(3)
    x = np.concatenate([rng.normal(size=(200000,)) * 2, rng.normal(size=(50000,)) * 1e-3,
                        [0.0, -0.0, 12.0, -12.0, 1e-30]]).astype(np.float32)
    want = port.gelu(x)
    for strict in (True, False):
        be = backends("f32", strict)
        d = be.to_device(x)
        be.gelu_inplace(d, x.size)
        got = be.d2h(d, x.size)
        assert np.abs(got - want).max() <= 1e-6 * max(1.0, np.abs(want).max())
        if strict:
            # strict mode carries the host libm's tanhf: the same bits as the CPU
            assert be.libm_exact
            assert np.array_equal(got, want)
        d.free()
    be = backends("f32", True)
    a, b = be.to_device(x), be.to_device(want)
    be.residual_inplace(a, b, x.size)
    assert np.array_equal(be.d2h(a, x.size), x + want)
    be.scale_dev(a, x.size, 0.25)
    assert np.array_equal(be.d2h(a, x.size), (x + want) * np.float32(0.25))
    be.h2d(np.array([-2, np.nan, 0.5, np.inf], np.float32), a)
    be.clip_dev(a, 4)                                   # src/backend.c:815-820
    assert np.array_equal(be.d2h(a, 4), np.array([-1, 0, 0.5, 0], np.float32))
    be.copy_dev(b, a, 4)
    assert np.array_equal(be.d2h(b, 4), be.d2h(a, 4))
    a.free(); b.free()


def test_attention_closed_form(backends):
    # gpu/metal/backend_metal_ops.m:1049-1079 of the reference
    e = np.exp(1.0)
    for strict in (True, False):
        be = backends("f32", strict)
        dqkv = be.to_device(np.array([1, 0, 1, 0, 2, 3], np.float32))
        dk, dv, dout = be.dev_alloc(4), be.dev_alloc(4), be.dev_alloc(2)
        be.self_attention_dev(dqkv, dk, dv, 0, 2, 1, 1, 2, 1.0, dout)
        assert np.allclose(be.d2h(dout, 2), [2, 3], atol=1e-6)
        be.h2d(np.array([1, 0, 0, 1, 4, 5], np.float32), dqkv)
        be.self_attention_dev(dqkv, dk, dv, 1, 2, 2, 1, 2, 1.0, dout)
        assert np.allclose(be.d2h(dout, 2), [(2 * e + 4) / (e + 1), (3 * e + 5) / (e + 1)], atol=1e-5)
        dq = be.to_device(np.array([1, 2], np.float32))
        be.cross_attention_dev(dq, dk, dv, 1, 2, 1, 2, 1.0, dout)
        assert np.allclose(be.d2h(dout, 2), [2, 3], atol=1e-6)


@pytest.mark.parametrize("heads,hw,position", [(12, 64, 0), (12, 64, 31), (12, 64, 32), (12, 64, 256),
                                               (12, 64, 1023), (1, 128, 100), (12, 16, 70), (3, 20, 9)])
def test_self_attention_matches_oracle(heads, hw, position, backends, port):
    """Random KV; the new row is appended at `position` and lands at
    [position][h*hw + d] bit for bit."""
    width = heads * hw
    cap = position + 2
    rng = np.random.default_rng(position * 7 + hw)
    k = rng.normal(size=(cap, width)).astype(np.float32)
    v = rng.normal(size=(cap, width)).astype(np.float32)
    qkv = rng.normal(size=(3 * width,)).astype(np.float32)
    scale = float(np.float32(1.0) / np.sqrt(np.float32(hw)))
    rk, rv = k.copy(), v.copy()
    want = port.self_attention(qkv, rk, rv, position, width, position + 1, heads, hw, scale)
    for strict in (True, False):
        be = backends("f32", strict)
        dqkv, dk, dv, dout = be.to_device(qkv), be.to_device(k), be.to_device(v), be.dev_alloc(width)
        be.self_attention_dev(dqkv, dk, dv, position, width, position + 1, heads, hw, scale, dout)
        got = be.d2h(dout, width)
        assert np.array_equal(be.d2h(dk, k.size).reshape(k.shape), rk)       # KV append, bit exact
        assert np.array_equal(be.d2h(dv, v.size).reshape(v.shape), rv)
        assert rel_err(got, want) < (2e-7 if strict else 3e-6)
        if strict:
            assert np.array_equal(got, want)     # reference order + the host's expf
        for buf in (dqkv, dk, dv, dout):
            buf.free()


def test_cross_attention_matches_oracle(backends, port):
    rng = np.random.default_rng(11)
    for valid, xw in ((128, 128), (24, 32), (5, 768)):
        k = rng.normal(size=(valid, xw)).astype(np.float32)
        v = rng.normal(size=(valid, xw)).astype(np.float32)
        q = rng.normal(size=(xw,)).astype(np.float32)
        scale = float(np.float32(1.0) / np.sqrt(np.float32(xw)))
        want = port.cross_attention(q, k, v, valid, xw, 1, xw, scale)
        for strict in (True, False):
            be = backends("f32", strict)
            dq, dk, dv, dout = be.to_device(q), be.to_device(k), be.to_device(v), be.dev_alloc(xw)
            be.cross_attention_dev(dq, dk, dv, valid, xw, 1, xw, scale, dout)
            got = be.d2h(dout, xw)
            assert rel_err(got, want) < (2e-7 if strict else 3e-6)
            if strict:
                assert np.array_equal(got, want)


def test_argmax_first_on_ties(backends, port):
    be = backends("f32", False)
    rng = np.random.default_rng(2)
    for trial in range(6):
        logits = rng.normal(size=(2048,)).astype(np.float32)
        if trial % 2:
            logits[rng.integers(0, 2016, 5)] = logits.max() + 1.0      # five-way tie
        logits[2017] = logits.max() + (2.0 if trial < 3 else -2.0)     # EOS sometimes best
        logits[2040] = 99.0                                            # never a candidate
        d = be.to_device(logits)
        for allow in (0, 1):
            assert be.argmax_dev(d, 2048, 2016, 2017, allow) == port.argmax_constrained(logits, 2016, 2017, allow)
        d.free()
    d = be.to_device(np.full(64, -np.inf, np.float32))
    assert be.argmax_dev(d, 64, 56, 57, 1) == 0


def test_invalid_requests_return_errors(backends):
    be = backends("f32", False)
    with pytest.raises(MynahB200Error):
        be.qmat_linear(np.ones((4, 8), np.float32), np.ones((0, 8), np.float32))   # zero rows
    d = be.dev_alloc(8)
    with pytest.raises(MynahB200Error):
        be.self_attention_dev(d, d, d, 0, 1, 1, 1, 2, 1.0, d)    # cache_stride < heads*head_width
    d.free()
