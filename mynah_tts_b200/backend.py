"""Host-side mirror of the reference's backend and decoder interfaces over the
C ABI: method names and argument meaning follow mynah-tts's src/backend.h
(`matmul_d2d`, `layer_norm_inplace`, `self_attention_dev`, ...) and
src/graph.c's decoder step (`step_batch`), so parity tests read like the
reference's own.  Every call goes through libmynah_b200.so; nothing here
computes.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import capi
from .capi import F16, F32, INT4, INT8, QUANT, MynahB200Error, call, fp  # noqa: F401


class DeviceBuffer:
    """n floats on the device, owned through dev_alloc/dev_free (src/backend.h:181-186)."""

    def __init__(self, backend: "Backend", n: int):
        self.backend = backend
        self.n = n
        ptr = C.c_void_p()
        call(capi.lib().mynah_cuda_dev_alloc, backend.state, n, C.byref(ptr))
        self.ptr = ptr

    def at(self, offset: int) -> C.c_void_p:
        return C.c_void_p(self.ptr.value + 4 * offset)

    def free(self):
        if self.ptr:
            capi.lib().mynah_cuda_dev_free(self.backend.state, self.ptr)
            self.ptr = None


class Backend:
    def __init__(self, quant="f32", strict: bool = False, device: int = 0, from_env: bool = False):
        self.lib = capi.lib()
        self.state = C.c_void_p()
        self._keep = []   # host arrays whose addresses key the device caches
        if from_env:
            self.matmul_fn, self.sgemm_fn = capi.MATMUL_FN(), capi.SGEMM_FN()
            self.close_fn, self.self_test_fn = capi.CLOSE_FN(), capi.SELF_TEST_FN()
            call(self.lib.mynah_backend_cuda_open, C.byref(self.state), C.byref(self.matmul_fn),
                 C.byref(self.sgemm_fn), C.byref(self.close_fn), C.byref(self.self_test_fn))
        else:
            q = QUANT[quant] if isinstance(quant, str) else int(quant)
            call(self.lib.mynah_b200_open, C.byref(self.state), device, q, int(strict))
        self.quant = self.lib.mynah_b200_quant(self.state)
        self.strict = bool(self.lib.mynah_b200_strict(self.state))
        self.libm_exact = bool(self.lib.mynah_b200_libm_exact(self.state))

    def close(self):
        if self.state:
            self.lib.mynah_b200_close(self.state)
            self.state = None

    def keep(self, a: np.ndarray | None):
        """Pin a host array's lifetime to the backend (host pointers are cache keys)."""
        if a is not None:
            self._keep.append(a)
        return a

    def set_stream(self, cuda_stream: int):
        call(self.lib.mynah_b200_set_stream, self.state, C.c_void_p(cuda_stream))

    def timer_start(self):
        call(self.lib.mynah_b200_timer_start, self.state)

    def timer_stop(self) -> float:
        ms = C.c_float(0.0)
        call(self.lib.mynah_b200_timer_stop, self.state, C.byref(ms))
        return float(ms.value)

    @property
    def launch_count(self) -> int:
        return int(self.lib.mynah_b200_launch_count(self.state))

    # ---- memory ----------------------------------------------------------
    def dev_alloc(self, n: int) -> DeviceBuffer:
        return DeviceBuffer(self, n)

    def h2d(self, host: np.ndarray, dev, n: int | None = None):
        host = np.ascontiguousarray(host, np.float32)
        call(self.lib.mynah_cuda_h2d, self.state, fp(host), _p(dev), host.size if n is None else n)

    def d2h(self, dev, n: int) -> np.ndarray:
        out = np.empty((n,), np.float32)
        call(self.lib.mynah_cuda_d2h, self.state, _p(dev), fp(out), n)
        return out

    def to_device(self, host: np.ndarray) -> DeviceBuffer:
        buf = self.dev_alloc(host.size)
        self.h2d(host, buf)
        return buf

    def sync(self):
        call(self.lib.mynah_cuda_sync, self.state)

    # ---- seam ops on device rows -------------------------------------------
    def matmul(self, x: np.ndarray, weight: np.ndarray, bias=None) -> np.ndarray:
        """Host-buffer product through the function pointer mynah_backend_cuda_open returns."""
        rows, iw = x.shape
        ow = weight.shape[0]
        out = np.empty((rows, ow), np.float32)
        self.keep(weight), self.keep(bias)
        call(self.lib.mynah_cuda_matmul_graph, self.state, fp(x), fp(out), rows, iw, ow, fp(weight),
             None if bias is None else fp(bias))
        return out

    def matmul_d2d(self, din, dout, rows, iw, ow, weight: np.ndarray, bias=None):
        self.keep(weight), self.keep(bias)
        call(self.lib.mynah_cuda_matmul_d2d, self.state, _p(din), _p(dout), rows, iw, ow, fp(weight),
             None if bias is None else fp(bias))

    def layer_norm_inplace(self, din, dout, gain: np.ndarray, rows, width):
        self.keep(gain)
        call(self.lib.mynah_cuda_layer_norm_inplace, self.state, _p(din), _p(dout), fp(gain), rows, width)

    def gelu_inplace(self, dev, n):
        call(self.lib.mynah_cuda_gelu_inplace, self.state, _p(dev), n)

    def residual_inplace(self, dout, din, n):
        call(self.lib.mynah_cuda_residual_inplace, self.state, _p(dout), _p(din), n)

    def self_attention_dev(self, dqkv, dk, dv, position, cache_stride, valid, heads, head_width,
                           scale, dout):
        call(self.lib.mynah_cuda_self_attention_dev, self.state, _p(dqkv), _p(dk), _p(dv), position,
             cache_stride, valid, heads, head_width, C.c_float(scale), _p(dout))

    def cross_attention_dev(self, dq, dk, dv, valid, cache_stride, heads, head_width, scale, dout):
        call(self.lib.mynah_cuda_cross_attention_dev, self.state, _p(dq), _p(dk), _p(dv), valid,
             cache_stride, heads, head_width, C.c_float(scale), _p(dout))

    def argmax_dev(self, dlogits, vocab, codebook_size, eos_id, allow_eos) -> int:
        out = C.c_uint(0)
        call(self.lib.mynah_cuda_argmax_dev, self.state, _p(dlogits), vocab, codebook_size, eos_id,
             int(allow_eos), C.byref(out))
        return int(out.value)

    def copy_dev(self, dst, src, n):
        call(self.lib.mynah_cuda_copy_dev, self.state, _p(dst), _p(src), n)

    def scale_dev(self, dev, n, scale):
        call(self.lib.mynah_cuda_scale_dev, self.state, _p(dev), n, C.c_float(scale))

    def clip_dev(self, dev, n):
        call(self.lib.mynah_cuda_clip_dev, self.state, _p(dev), n)

    def sgemm(self, trans_a, trans_b, m, n, k, alpha, a, lda, b, ldb, beta, c, ldc):
        call(self.sgemm_fn, self.state, trans_a, trans_b, m, n, k, C.c_float(alpha), fp(a), lda, fp(b),
             ldb, C.c_float(beta), fp(c), ldc)

    def self_test(self):
        call(self.self_test_fn, self.state)

    # ---- extensions ---------------------------------------------------------
    def pack_weight(self, quant: int, w: np.ndarray):
        n, k = w.shape
        if quant == INT8:
            q, s = np.empty((n, k), np.int8), np.empty((n,), np.float32)
        elif quant == INT4:
            q, s = np.empty((n, k // 2), np.uint8), np.empty((n, k // 32), np.float32)
        elif quant == F16:
            q, s = np.empty((n, k), np.uint16), np.empty((0,), np.float32)
        else:
            q, s = np.empty((n, k), np.float32), np.empty((0,), np.float32)
        call(self.lib.mynah_b200_pack_weight, self.state, quant, fp(w), n, k,
             q.ctypes.data_as(C.c_void_p), fp(s) if s.size else None)
        return q, s

    def quantize_act(self, x: np.ndarray):
        x2 = np.ascontiguousarray(x.reshape(-1, x.shape[-1]))
        q = np.empty(x2.shape, np.int8)
        sx = np.empty((x2.shape[0],), np.float32)
        call(self.lib.mynah_b200_quantize_act, self.state, fp(x2), x2.shape[0], x2.shape[1],
             q.ctypes.data_as(C.c_void_p), fp(sx))
        return q.reshape(x.shape), sx

    def qmat_linear(self, weight: np.ndarray, x: np.ndarray, bias=None, ln_gain=None,
                    out: np.ndarray | None = None) -> np.ndarray:
        x2 = x.reshape(-1, x.shape[-1])
        n, k = weight.shape[0], weight.shape[1]
        if out is None:
            out = np.empty((x2.shape[0], n), np.float32)
        self.keep(weight), self.keep(bias), self.keep(ln_gain)
        call(self.lib.mynah_b200_qmat_linear, self.state, fp(weight), fp(x2), fp(out), x2.shape[0], k,
             n, None if bias is None else fp(bias), None if ln_gain is None else fp(ln_gain))
        return out


def _p(dev):
    if isinstance(dev, DeviceBuffer):
        return dev.ptr
    return dev


class MatrixPool:
    """`groups` distinct matrices (row rotations of one seeded matrix) resident
    on the device, for streaming more weight bytes than L2 holds through the
    product kernel."""

    def __init__(self, backend: Backend, w: np.ndarray, groups: int, bias=None, gain=None):
        self.backend = backend
        self.n, self.k = w.shape
        self.groups = groups
        self.handle = C.c_void_p()
        call(capi.lib().mynah_b200_pool_create, backend.state, fp(w), self.n, self.k, groups,
             None if bias is None else fp(bias), None if gain is None else fp(gain),
             C.byref(self.handle))

    @property
    def bytes_per_pass(self) -> int:
        return int(capi.lib().mynah_b200_pool_bytes_per_pass(self.handle))

    def linear(self, dev_x, dev_out):
        call(capi.lib().mynah_b200_pool_linear, self.handle, _p(dev_x), _p(dev_out))

    def close(self):
        if self.handle:
            capi.lib().mynah_b200_pool_destroy(self.handle)
            self.handle = None


class TextEncoder:
    """encode_text over the reference-named tensors of synth.add_encoder (or a real pack)."""

    def __init__(self, backend: Backend, tensors: dict, shape):
        self.backend, self.shape = backend, shape
        self._keep = [np.ascontiguousarray(v, np.float32) for v in tensors.values()]
        t = {k: self._keep[i] for i, k in enumerate(tensors)}
        layers = (capi.EncoderLayerWeights * shape.layers)()
        for i in range(shape.layers):
            pre = f"encoder.layers.{i}."
            layers[i].norm_self = fp(t[pre + "norm_self.weight"])
            layers[i].norm_pos_ff = fp(t[pre + "norm_pos_ff.weight"])
            layers[i].qkv_w = fp(t[pre + "self_attention.qkv_net.weight"])
            layers[i].o_w = fp(t[pre + "self_attention.o_net.weight"])
            layers[i].ffn_proj_w = fp(t[pre + "pos_ff.proj.conv.weight"])
            layers[i].ffn_out_w = fp(t[pre + "pos_ff.o_net.conv.weight"])
        desc = capi.EncoderDesc()
        desc.layers, desc.width, desc.heads, desc.kernel = shape.layers, shape.width, shape.heads, shape.kernel
        desc.vocab, desc.max_length = shape.vocab, shape.max_length
        desc.layer = layers
        desc.embedding = fp(t["text_embedding.weight"])
        desc.position = fp(t["encoder.position_embeddings.weight"])
        desc.norm_out = fp(t["encoder.norm_out.weight"])
        self.handle = C.c_void_p()
        call(capi.lib().mynah_b200_encoder_create, backend.state, C.byref(desc), C.byref(self.handle))

    def encode(self, ids) -> np.ndarray:
        ids = np.ascontiguousarray(ids, np.int32)
        out = np.empty((len(ids), self.shape.width), np.float32)
        call(capi.lib().mynah_b200_encoder_encode, self.handle, ids.ctypes.data_as(capi.c_int_p), len(ids), fp(out))
        return out

    def close(self):
        if self.handle:
            capi.lib().mynah_b200_encoder_destroy(self.handle)
            self.handle = None


class Codec:
    """decode_codec over the reference-named tensors of synth.add_codec (or a real pack)."""

    def __init__(self, backend: Backend, tensors: dict, shape, max_frames: int, arithmetic: int = 0):
        """arithmetic: 0 the backend's mode, 1 reference order, 2 tensor cores."""
        self.backend, self.shape, self.max_frames = backend, shape, max_frames
        self._keep = []

        def p(name):
            a = np.ascontiguousarray(tensors[name], np.float32)
            self._keep.append(a)
            return fp(a)
        desc = capi.CodecDesc()
        desc.base, desc.max_frames, desc.arithmetic = shape.base, max_frames, arithmetic
        desc.pre_w, desc.pre_b = p("audio_decoder.pre_conv.conv.weight"), p("audio_decoder.pre_conv.conv.bias")
        for s in range(5):
            st = desc.stage[s]
            st.alpha = p(f"audio_decoder.activations.{s}.activation.snake_act.alpha")
            st.up_w = p(f"audio_decoder.up_sample_conv_layers.{s}.conv.weight")
            st.up_b = p(f"audio_decoder.up_sample_conv_layers.{s}.conv.bias")
            for b in range(3):
                for d in range(3):
                    pre = f"audio_decoder.res_layers.{s}.res_blocks.{b}.res_blocks.{d}."
                    blk = st.block[b][d]
                    blk.in_alpha = p(pre + "input_activation.activation.snake_act.alpha")
                    blk.in_w, blk.in_b = p(pre + "input_conv.conv.weight"), p(pre + "input_conv.conv.bias")
                    blk.skip_alpha = p(pre + "skip_activation.activation.snake_act.alpha")
                    blk.skip_w, blk.skip_b = p(pre + "skip_conv.conv.weight"), p(pre + "skip_conv.conv.bias")
        desc.post_alpha = p("audio_decoder.post_activation.activation.snake_act.alpha")
        desc.post_w, desc.post_b = p("audio_decoder.post_conv.conv.weight"), p("audio_decoder.post_conv.conv.bias")
        self.handle = C.c_void_p()
        call(capi.lib().mynah_b200_codec_create, backend.state, C.byref(desc), C.byref(self.handle))
        self._keep = []          # the weights were uploaded during the call

    def decode(self, codes, stop_after: int = 0) -> np.ndarray:
        """codes [8, frames] -> samples [frames * 1024]; stop_after as in
        mynah_b200_codec_decode_partial (1: first convolution, 2 + s: stage s)."""
        codes = np.ascontiguousarray(codes, np.uint32)
        frames = codes.shape[1]
        n = C.c_size_t()
        if stop_after == 0:
            out = np.empty((frames * int(capi.lib().mynah_b200_codec_samples_per_frame()),), np.float32)
            call(capi.lib().mynah_b200_codec_decode, self.handle, codes.ctypes.data_as(capi.c_uint_p), frames, fp(out),
                 C.byref(n))
        else:
            s = stop_after - 2
            dims = (self.shape.base, frames) if stop_after == 1 else \
                (self.shape.base >> (s + 1), frames * int(np.prod(self.shape.rates[:s + 1])))
            out = np.empty(dims, np.float32)
            call(capi.lib().mynah_b200_codec_decode_partial, self.handle, codes.ctypes.data_as(capi.c_uint_p), frames,
                 stop_after, fp(out), out.size, C.byref(n))
        assert n.value == out.size
        return out

    def time(self, codes, repeats: int = 5) -> float:
        """Device milliseconds of one decode."""
        codes = np.ascontiguousarray(codes, np.uint32)
        ms = C.c_float()
        call(capi.lib().mynah_b200_codec_time, self.handle, codes.ctypes.data_as(capi.c_uint_p), codes.shape[1], repeats,
             C.byref(ms))
        return float(ms.value)

    def close(self):
        if self.handle:
            capi.lib().mynah_b200_codec_destroy(self.handle)
            self.handle = None


class Decoder:
    """The whole-step decoder over a synth.SynthModel (or any object with the
    same accessors)."""

    def __init__(self, backend: Backend, model, capacity: int, slots: int, max_batch: int | None = None,
                 with_heads: bool = True, keep_f32_weights: bool = False):
        self.backend = backend
        self.model = model
        s = model.shape
        self.shape = s
        self.capacity = capacity
        self.slots = slots
        self.max_batch = max_batch or slots
        layers = (capi.LayerWeights * s.layers)()
        for i in range(s.layers):
            L = layers[i]
            L.norm_self = fp(model.layer(i, "norm_self.weight"))
            L.norm_xattn_query = fp(model.layer(i, "norm_xattn_query.weight"))
            L.norm_pos_ff = fp(model.layer(i, "norm_pos_ff.weight"))
            L.qkv_w = fp(model.layer(i, "self_attention.qkv_net.weight"))
            L.o_self_w = fp(model.layer(i, "self_attention.o_net.weight"))
            L.q_cross_w = fp(model.layer(i, "cross_attention.q_net.weight"))
            L.o_cross_w = fp(model.layer(i, "cross_attention.o_net.weight"))
            L.ffn_up_w = fp(model.layer(i, "pos_ff.proj.conv.weight"))
            L.ffn_down_w = fp(model.layer(i, "pos_ff.o_net.conv.weight"))
            L.norm_xattn_memory = fp(model.layer(i, "norm_xattn_memory.weight"))
            L.kv_cross_w = fp(model.layer(i, "cross_attention.kv_net.weight"))
        desc = capi.DecoderDesc()
        desc.layers, desc.width, desc.heads, desc.xattn_width = s.layers, s.width, s.heads, s.xattn_width
        desc.memory_length, desc.capacity, desc.slots = s.memory_length, capacity, slots
        desc.max_batch, desc.max_positions = self.max_batch, s.max_positions
        desc.layer = layers
        desc.position, desc.norm_out = fp(model.position), fp(model.norm_out)
        desc.keep_f32_weights = int(keep_f32_weights)
        if with_heads:
            tabs = (capi.c_float_p * s.tables)(*[fp(model.embedding(t)) for t in range(s.tables)])
            hw = (capi.c_float_p * s.tables)(*[fp(model.head_weight(t)) for t in range(s.tables)])
            hb = (capi.c_float_p * s.tables)(*[fp(model.head_bias(t)) for t in range(s.tables)])
            desc.tables, desc.vocab = s.tables, s.vocab
            desc.codebook_size, desc.eos_id = s.codebook_size, s.eos_id
            desc.embeddings, desc.head_w, desc.head_b = tabs, hw, hb
        self.handle = C.c_void_p()
        call(capi.lib().mynah_b200_decoder_create, backend.state, C.byref(desc), C.byref(self.handle))
        self.has_local = False
        if with_heads and getattr(s, "local_layers", 0):
            ll = (capi.LocalLayerWeights * s.local_layers)()
            for i in range(s.local_layers):
                ll[i].norm_self = fp(model.local_layer(i, "norm_self.weight"))
                ll[i].norm_pos_ff = fp(model.local_layer(i, "norm_pos_ff.weight"))
                ll[i].qkv_w = fp(model.local_layer(i, "self_attention.qkv_net.weight"))
                ll[i].o_w = fp(model.local_layer(i, "self_attention.o_net.weight"))
                ll[i].ffn_up_w = fp(model.local_layer(i, "pos_ff.proj.conv.weight"))
                ll[i].ffn_down_w = fp(model.local_layer(i, "pos_ff.o_net.conv.weight"))
            ld = capi.LocalDesc()
            ld.layers, ld.layer = s.local_layers, ll
            ld.position, ld.position_rows = fp(model.local_position), model.local_position.shape[0]
            ld.codebooks = s.tables // 2       # stacking factor 2, as the reference requires
            call(capi.lib().mynah_b200_decoder_local_attach, self.handle, C.byref(ld))
            self.has_local = True

    def close(self):
        if self.handle:
            capi.lib().mynah_b200_decoder_destroy(self.handle)
            self.handle = None

    @property
    def weight_bytes(self) -> int:
        return int(capi.lib().mynah_b200_decoder_weight_bytes(self.handle))

    def kv_bytes(self, length: int) -> int:
        return int(capi.lib().mynah_b200_decoder_kv_bytes(self.handle, length))

    def profile(self, enable: bool):
        call(capi.lib().mynah_b200_decoder_profile, self.handle, int(enable))

    def profile_read(self) -> dict:
        """{call site: (launches, total device ms)} since profiling was enabled."""
        n = capi.PROFILE_CLASSES
        launches = (C.c_ulonglong * n)()
        ms = (C.c_double * n)()
        call(capi.lib().mynah_b200_decoder_profile_read, self.handle, launches, ms, n)
        names = [capi.lib().mynah_b200_profile_class_name(i).decode() for i in range(n)]
        return {names[i]: (int(launches[i]), float(ms[i])) for i in range(n)}

    def slot_load(self, slot: int, cross_k, cross_v, self_k=None, self_v=None, length: int = 0):
        """cross_k / cross_v: [layers, memory_length, xattn_width] of THIS request (its own
        text length, at most the decoder's); self_k / self_v: [layers, capacity, width]."""
        ck = np.ascontiguousarray(cross_k, np.float32)
        cv = np.ascontiguousarray(cross_v, np.float32)
        assert ck.ndim == 3 and ck.shape == cv.shape
        sk = None if self_k is None else np.ascontiguousarray(self_k, np.float32)
        sv = None if self_v is None else np.ascontiguousarray(self_v, np.float32)
        call(capi.lib().mynah_b200_decoder_slot_load, self.handle, slot, fp(ck), fp(cv), ck.shape[1],
             None if sk is None else fp(sk), None if sv is None else fp(sv), length)

    def slot_prefill(self, slot: int, memory: np.ndarray):
        """Cross K/V of a request made on the device from its text-encoder memory."""
        mem = np.ascontiguousarray(memory, np.float32)
        call(capi.lib().mynah_b200_decoder_slot_prefill, self.handle, slot, fp(mem), mem.shape[0])

    def prefill(self, slot: int, rows: np.ndarray) -> np.ndarray:
        """decoder_run with count > 1: rows [count, width] of one request pushed through the
        stack together; returns the output-norm row of the last one."""
        rows = np.ascontiguousarray(rows, np.float32)
        out = np.empty((self.shape.width,), np.float32)
        call(capi.lib().mynah_b200_decoder_prefill, self.handle, slot, fp(rows), rows.shape[0], fp(out))
        return out

    def slot_read_cross(self, slot: int):
        s = self.shape
        k = np.empty((s.layers, s.memory_length, s.xattn_width), np.float32)
        v = np.empty_like(k)
        call(capi.lib().mynah_b200_decoder_slot_read_cross, self.handle, slot, fp(k), fp(v))
        return k, v

    def slot_length(self, slot: int) -> int:
        n = capi.sz(0)
        call(capi.lib().mynah_b200_decoder_slot_length, self.handle, slot, C.byref(n))
        return int(n.value)

    def slot_set_length(self, slot: int, length: int):
        call(capi.lib().mynah_b200_decoder_slot_set_length, self.handle, slot, length)

    def slot_read_kv(self, slot: int):
        s = self.shape
        k = np.empty((s.layers, self.capacity, s.width), np.float32)
        v = np.empty_like(k)
        call(capi.lib().mynah_b200_decoder_slot_read_kv, self.handle, slot, fp(k), fp(v))
        return k, v

    def set_layers(self, n: int):
        call(capi.lib().mynah_b200_decoder_set_layers, self.handle, n)

    def step_batch(self, slots, rows: np.ndarray, outs: np.ndarray | None = None) -> np.ndarray:
        rows = np.ascontiguousarray(rows, np.float32)
        batch = len(slots)
        if outs is None:
            outs = np.empty_like(rows)
        slot_arr = (C.c_uint * batch)(*slots)
        ins = (capi.c_float_p * batch)(*[fp(rows[b]) for b in range(batch)])
        out_ptrs = (capi.c_float_p * batch)(*[fp(outs[b]) for b in range(batch)])
        call(capi.lib().mynah_b200_decoder_step_batch, self.handle, slot_arr, ins, out_ptrs, batch)
        return outs

    def frame_batch(self, slots, codes: np.ndarray, allow_eos=None, want_hidden: bool = False,
                    tokens: np.ndarray | None = None):
        batch = len(slots)
        codes = np.ascontiguousarray(codes, np.uint32)
        if tokens is None:
            tokens = np.empty((batch, self.shape.tables), np.uint32)
        hidden = np.empty((batch, self.shape.width), np.float32) if want_hidden else None
        slot_arr = (C.c_uint * batch)(*slots)
        allow = None if allow_eos is None else (C.c_int * batch)(*[int(a) for a in allow_eos])
        call(capi.lib().mynah_b200_decoder_frame_batch, self.handle, slot_arr,
             codes.ctypes.data_as(capi.c_uint_p), allow, tokens.ctypes.data_as(capi.c_uint_p),
             None if hidden is None else fp(hidden), batch)
        return (tokens, hidden) if want_hidden else tokens

    def bind_frame_batch(self, slots, codes: np.ndarray, allow_eos, tokens: np.ndarray):
        """frame_batch for a loop that calls it every frame with the same buffers: the C
        arguments (slot ids, EOS rule, the addresses of `codes` and `tokens`) are made once and
        the returned function only makes the foreign call: it reads `codes` and fills `tokens`
        as they are at that moment.  `codes` and `tokens` must be C-contiguous uint32 arrays of
        [len(slots), tables] that outlive the returned function."""
        batch = len(slots)
        want = (batch, self.shape.tables)
        for name, arr in (("codes", codes), ("tokens", tokens)):
            if arr.dtype != np.uint32 or arr.shape != want or not arr.flags["C_CONTIGUOUS"]:
                raise ValueError(f"{name} must be a C-contiguous uint32 array of shape {want}")
        fn = capi.lib().mynah_b200_decoder_frame_batch
        slot_arr = (C.c_uint * batch)(*slots)
        allow = None if allow_eos is None else (C.c_int * batch)(*[int(a) for a in allow_eos])
        codes_p, tokens_p = codes.ctypes.data_as(capi.c_uint_p), tokens.ctypes.data_as(capi.c_uint_p)
        err = C.create_string_buffer(capi.ERR_CAP)
        handle, keep = self.handle, (codes, tokens)

        def step():
            if fn(handle, slot_arr, codes_p, allow, tokens_p, None, batch, err, capi.ERR_CAP) != 0:
                raise MynahB200Error(err.value.decode(errors="replace") or "frame_batch failed")
            return keep[1]
        return step

    @staticmethod
    def _samplers(batch, samplers):
        """samplers: None (greedy) or a list of (temperature, topk, rng_state[, allow_eos])."""
        arr = (capi.Sampler * batch)()
        for b in range(batch):
            t = (0.0, 0, 0, 1) if samplers is None else tuple(samplers[b])
            arr[b].temperature, arr[b].topk, arr[b].rng_state = float(t[0]), int(t[1]), int(t[2])
            arr[b].allow_eos = int(t[3]) if len(t) > 3 else 1
        return arr

    def local_frame(self, decoder_last: np.ndarray, samplers=None):
        """One stacked frame of the local transformer for len(decoder_last) requests ->
        codes, values [batch, tables], saw_eos, eos_frame [batch], new rng states."""
        rows = np.ascontiguousarray(decoder_last, np.float32)
        batch = rows.shape[0]
        arr = self._samplers(batch, samplers)
        codes = np.zeros((batch, self.shape.tables), np.uint32)
        values = np.zeros_like(codes)
        saw = (C.c_int * batch)()
        eos = (C.c_long * batch)()
        call(capi.lib().mynah_b200_decoder_local_frame, self.handle, fp(rows), batch, arr,
             codes.ctypes.data_as(capi.c_uint_p), values.ctypes.data_as(capi.c_uint_p), saw, eos)
        return (codes, values, np.array(list(saw)), np.array(list(eos)),
                [int(arr[b].rng_state) for b in range(batch)])

    def generate(self, slots, codes: np.ndarray, frames, min_frames: int = 0, samplers=None):
        """greedy() with the local transformer and its sampler in place of the logit
        heads.  Returns (tokens [max_frames, batch, tables], eos_frame, device ms, last
        stored codes, new rng states)."""
        batch = len(slots)
        frames = [frames] * batch if isinstance(frames, int) else list(frames)
        codes = np.ascontiguousarray(codes, np.uint32).copy()
        tokens = np.zeros((max(frames), batch, self.shape.tables), np.uint32)
        eos = (C.c_long * batch)()
        ms = C.c_float(0.0)
        arr = self._samplers(batch, samplers)
        call(capi.lib().mynah_b200_decoder_generate, self.handle, (C.c_uint * batch)(*slots), batch,
             codes.ctypes.data_as(capi.c_uint_p), (capi.sz * batch)(*frames), min_frames, arr,
             tokens.ctypes.data_as(capi.c_uint_p), eos, C.byref(ms))
        return (tokens, np.array(list(eos)), float(ms.value), codes,
                [int(arr[b].rng_state) for b in range(batch)])

    def frame_batch_local(self, slots, codes: np.ndarray, samplers=None):
        """One sampled frame for the given slots -> codes, values, saw_eos, eos_frame, rng."""
        batch = len(slots)
        codes = np.ascontiguousarray(codes, np.uint32)
        arr = self._samplers(batch, samplers)
        out = np.zeros((batch, self.shape.tables), np.uint32)
        values = np.zeros_like(out)
        saw = (C.c_int * batch)()
        eos = (C.c_long * batch)()
        call(capi.lib().mynah_b200_decoder_frame_batch_local, self.handle, (C.c_uint * batch)(*slots),
             codes.ctypes.data_as(capi.c_uint_p), arr, out.ctypes.data_as(capi.c_uint_p),
             values.ctypes.data_as(capi.c_uint_p), saw, eos, batch)
        return (out, values, np.array(list(saw)), np.array(list(eos)),
                [int(arr[b].rng_state) for b in range(batch)])

    def serve(self, requests):
        """Continuous batching.  requests: list of dicts with memory, start_codes,
        max_frames, min_frames, sampler (temperature, topk, rng).  Returns a list of
        (codes [frames_done, tables], eos_frame, admitted_at, rng) and the step count."""
        n = len(requests)
        arr = (capi.Request * n)()
        keep = []
        for i, r in enumerate(requests):
            mem = np.ascontiguousarray(r["memory"], np.float32)
            start = np.ascontiguousarray(r["start_codes"], np.uint32)
            out = np.zeros((r["max_frames"], self.shape.tables), np.uint32)
            keep.append((mem, start, out))
            arr[i].memory, arr[i].start_codes = fp(mem), start.ctypes.data_as(capi.c_uint_p)
            arr[i].memory_length = mem.shape[0]
            arr[i].max_frames, arr[i].min_frames = r["max_frames"], r.get("min_frames", 0)
            t = r.get("sampler", (0.0, 0, 0))
            arr[i].sampler.temperature, arr[i].sampler.topk, arr[i].sampler.rng_state = float(t[0]), int(t[1]), int(t[2])
            arr[i].codes = out.ctypes.data_as(capi.c_uint_p)
        steps = capi.sz(0)
        call(capi.lib().mynah_b200_decoder_serve, self.handle, arr, n, C.byref(steps))
        results = [(keep[i][2][:arr[i].frames_done].copy(), int(arr[i].eos_frame), int(arr[i].admitted_at),
                    int(arr[i].sampler.rng_state)) for i in range(n)]
        return results, int(steps.value)

    def greedy(self, slots, codes: np.ndarray, frames, min_frames: int = 0):
        """codes [batch, tables]; frames: int or per-lane list.  Returns
        (tokens [max_frames, batch, tables], eos_frame [batch], device ms)."""
        batch = len(slots)
        frames = [frames] * batch if isinstance(frames, int) else list(frames)
        codes = np.ascontiguousarray(codes, np.uint32).copy()
        tokens = np.zeros((max(frames), batch, self.shape.tables), np.uint32)
        eos = (C.c_long * batch)()
        ms = C.c_float(0.0)
        call(capi.lib().mynah_b200_decoder_greedy, self.handle, (C.c_uint * batch)(*slots), batch,
             codes.ctypes.data_as(capi.c_uint_p), (capi.sz * batch)(*frames), min_frames,
             tokens.ctypes.data_as(capi.c_uint_p), eos, C.byref(ms))
        return tokens, np.array(list(eos)), float(ms.value), codes
