"""ctypes front end of the parity checkers.  TEST INFRASTRUCTURE ONLY.

Two libraries sit behind this module:

* ``liboracle_port.so`` -- the C restatement in ``mynah_oracle.c`` (class
  ``Port`` / ``PortModel`` / ``PortStream``); built by ``make -C oracle port``.
* ``_ref/libmynah_ref_{strict,fast}.so`` -- the reference's own sources compiled
  around the harness (class ``Ref`` / ``RefModel`` / ``RefDecoder``); present
  only where ``make -C oracle ref`` could see a reference checkout.

Only tests, the smoke check and the benchmark's CPU-baseline leg import this.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
PORT_SO = os.path.join(HERE, "liboracle_port.so")
# "b200": the reference's graph.c + backend.c (CUDA branch) linked against libmynah_b200.so,
# i.e. the reference's own decoder_run driving the library under test (needs a GPU to open)
REF_SO = {kind: os.path.join(HERE, "_ref", f"libmynah_ref_{kind}.so") for kind in ("strict", "fast", "b200")}

F32, INT8, INT4, F16 = 0, 1, 2, 3
QTYPES = {"f32": F32, "int8": INT8, "int4": INT4, "f16": F16}

c_float_p = C.POINTER(C.c_float)
c_uint_p = C.POINTER(C.c_uint)


def build_port() -> str:
    subprocess.run(["make", "-C", HERE, "port"], check=True, capture_output=True)
    return PORT_SO


def have_ref(kind: str = "strict") -> bool:
    return os.path.exists(REF_SO[kind])


def _fp(a: np.ndarray):
    assert a.dtype == np.float32 and a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(c_float_p)


def _ptr_array(arrays):
    arr = (c_float_p * len(arrays))()
    for i, a in enumerate(arrays):
        arr[i] = _fp(a)
    return arr


class CodecBlock(C.Structure):
    _fields_ = [(n, C.POINTER(C.c_float)) for n in ("in_alpha", "in_w", "in_b", "skip_alpha", "skip_w", "skip_b")]


class CodecStage(C.Structure):
    _fields_ = [("alpha", C.POINTER(C.c_float)), ("up_w", C.POINTER(C.c_float)), ("up_b", C.POINTER(C.c_float)),
                ("block", (CodecBlock * 3) * 3)]


class CodecDesc(C.Structure):
    """orc_codec of mynah_oracle.c."""
    _fields_ = [("base", C.c_size_t), ("pre_w", C.POINTER(C.c_float)), ("pre_b", C.POINTER(C.c_float)),
                ("stage", CodecStage * 5), ("post_alpha", C.POINTER(C.c_float)),
                ("post_w", C.POINTER(C.c_float)), ("post_b", C.POINTER(C.c_float))]


def fill_codec_desc(desc, tensors: dict, keep: list):
    """Points a codec descriptor (this module's CodecDesc or any structure with the same field
    names) at the reference-named tensors of synth.add_codec."""
    def p(name):
        a = np.ascontiguousarray(tensors[name], np.float32)
        keep.append(a)
        return a.ctypes.data_as(C.POINTER(C.c_float))
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


class Port:
    """Typed access to liboracle_port.so."""

    _instance = None

    def __init__(self):
        if not os.path.exists(PORT_SO) or os.path.getmtime(PORT_SO) < os.path.getmtime(
                os.path.join(HERE, "mynah_oracle.c")):
            build_port()
        self.lib = lib = C.CDLL(PORT_SO)
        sz = C.c_size_t
        lib.orc_f32_to_f16.restype = C.c_uint16
        lib.orc_f32_to_f16.argtypes = [C.c_float]
        lib.orc_f16_to_f32.restype = C.c_float
        lib.orc_f16_to_f32.argtypes = [C.c_uint16]
        lib.orc_quantize_act_int8.restype = C.c_float
        lib.orc_quantize_act_int8.argtypes = [C.c_void_p, c_float_p, sz]
        lib.orc_dot_q8.restype = C.c_float
        lib.orc_dot_q4.restype = C.c_float
        lib.orc_dot_f16.restype = C.c_float
        lib.orc_dot_f32.restype = C.c_float
        lib.orc_dot_f32.argtypes = [c_float_p, c_float_p, sz]
        lib.orc_layernorm.argtypes = [c_float_p, c_float_p, c_float_p, c_float_p, sz, sz, C.c_float]
        lib.orc_qmat_linear.argtypes = [C.c_int, c_float_p, c_float_p, c_float_p, sz, sz, sz,
                                        c_float_p, c_float_p]
        lib.orc_argmax_constrained.restype = C.c_uint
        lib.orc_argmax_constrained.argtypes = [c_float_p, sz, sz, sz, C.c_int]
        lib.orc_self_attention.argtypes = [c_float_p, c_float_p, c_float_p, sz, sz, sz, sz, sz,
                                           C.c_float, c_float_p, c_float_p]
        lib.orc_cross_attention.argtypes = [c_float_p, c_float_p, c_float_p, sz, sz, sz, sz,
                                            C.c_float, c_float_p, c_float_p]
        lib.orc_model_new.restype = C.c_void_p
        lib.orc_model_free.argtypes = [C.c_void_p]
        lib.orc_stream_new.restype = C.c_void_p
        lib.orc_stream_new.argtypes = [C.c_void_p, c_float_p, sz, sz]
        lib.orc_stream_free.argtypes = [C.c_void_p]
        for name in ("self_k", "self_v", "cross_k", "cross_v"):
            fn = getattr(lib, f"orc_stream_{name}")
            fn.restype = c_float_p
            fn.argtypes = [C.c_void_p]
        lib.orc_stream_length.restype = sz
        lib.orc_stream_length.argtypes = [C.c_void_p]
        lib.orc_stream_set_length.argtypes = [C.c_void_p, sz]
        lib.orc_stream_set_layers.argtypes = [C.c_void_p, sz]
        lib.orc_decoder_step.argtypes = [C.c_void_p, c_float_p, c_float_p]
        lib.orc_decoder_prefill.argtypes = [C.c_void_p, c_float_p, C.c_size_t, c_float_p]
        fpp = C.POINTER(c_float_p)
        lib.orc_encode_text.argtypes = [C.POINTER(C.c_int), C.c_size_t, C.c_size_t, C.c_size_t, C.c_size_t, C.c_size_t,
                                        C.c_size_t, c_float_p, c_float_p, c_float_p, fpp, fpp, fpp, fpp, fpp, fpp,
                                        c_float_p]
        lib.orc_codec_decode.restype = C.c_long
        lib.orc_codec_decode.argtypes = [C.POINTER(CodecDesc), c_uint_p, C.c_size_t, C.c_int, c_float_p]
        lib.orc_embed_frame.argtypes = [C.c_void_p, c_uint_p, c_float_p]
        lib.orc_heads_argmax.argtypes = [C.c_void_p, c_float_p, C.c_int, c_uint_p, c_float_p]
        lib.orc_greedy_frame.argtypes = [C.c_void_p, c_uint_p, C.c_int, c_uint_p, c_float_p]
        lib.orc_greedy_decode.restype = C.c_long
        lib.orc_greedy_decode.argtypes = [C.c_void_p, c_uint_p, sz, sz, c_uint_p]
        lib.orc_local_new.restype = C.c_void_p
        lib.orc_local_free.argtypes = [C.c_void_p]
        lib.orc_local_length.restype = sz
        lib.orc_local_length.argtypes = [C.c_void_p]
        lib.orc_local_set_length.argtypes = [C.c_void_p, sz]
        lib.orc_local_k.restype = c_float_p
        lib.orc_local_k.argtypes = [C.c_void_p]
        lib.orc_local_v.restype = c_float_p
        lib.orc_local_v.argtypes = [C.c_void_p]
        lib.orc_local_step.argtypes = [C.c_void_p, c_float_p, c_float_p]
        lib.orc_local_frame.argtypes = [C.c_void_p, c_float_p, C.c_float, C.c_uint,
                                        C.POINTER(C.c_uint64), C.c_int, sz, c_uint_p, c_uint_p,
                                        C.POINTER(C.c_long)]
        lib.orc_xorshift64.restype = C.c_uint64
        lib.orc_xorshift64.argtypes = [C.c_uint64]

    @classmethod
    def get(cls) -> "Port":
        if cls._instance is None:
            cls._instance = cls()
        return cls._instance

    # ---- single ops -----------------------------------------------------
    def quantize_weight_int8(self, w: np.ndarray):
        n, k = w.shape
        q = np.empty((n, k), np.int8)
        s = np.empty((n,), np.float32)
        self.lib.orc_quantize_weight_int8(_fp(w), C.c_size_t(n), C.c_size_t(k),
                                          q.ctypes.data_as(C.c_void_p), _fp(s))
        return q, s

    def quantize_weight_int4(self, w: np.ndarray):
        n, k = w.shape
        q = np.empty((n, k // 2), np.uint8)
        s = np.empty((n, k // 32), np.float32)
        self.lib.orc_quantize_weight_int4(_fp(w), C.c_size_t(n), C.c_size_t(k),
                                          q.ctypes.data_as(C.c_void_p), _fp(s))
        return q, s

    def quantize_weight_f16(self, w: np.ndarray):
        h = np.empty(w.shape, np.uint16)
        self.lib.orc_quantize_weight_f16(_fp(w), C.c_size_t(w.size), h.ctypes.data_as(C.c_void_p))
        return h

    def quantize_act_int8(self, x: np.ndarray):
        q = np.empty(x.shape, np.int8)
        sx = self.lib.orc_quantize_act_int8(q.ctypes.data_as(C.c_void_p), _fp(x), x.size)
        return q, np.float32(sx)

    def layernorm(self, x: np.ndarray, gain: np.ndarray, eps: float = 1e-5) -> np.ndarray:
        x2 = np.ascontiguousarray(x.reshape(-1, x.shape[-1]))
        y = np.empty_like(x2)
        self.lib.orc_layernorm(_fp(x2), _fp(gain), None, _fp(y), x2.shape[0], x2.shape[1], eps)
        return y.reshape(x.shape)

    def gelu(self, x: np.ndarray) -> np.ndarray:
        y = np.ascontiguousarray(x.copy())
        self.lib.orc_gelu_scalar(_fp(y), C.c_size_t(y.size))
        return y

    def qmat_linear(self, qtype: int, w: np.ndarray, x: np.ndarray, bias=None, ln_gain=None):
        x2 = np.ascontiguousarray(x.reshape(-1, x.shape[-1]))
        n, k = w.shape[0], w.shape[1]
        out = np.empty((x2.shape[0], n), np.float32)
        rc = self.lib.orc_qmat_linear(qtype, _fp(w), _fp(x2), _fp(out), x2.shape[0], k, n,
                                      None if bias is None else _fp(bias),
                                      None if ln_gain is None else _fp(ln_gain))
        assert rc == 0
        return out

    def encode_text(self, tensors: dict, shape, ids) -> np.ndarray:
        """The text encoder over the reference-named tensors of synth.add_encoder:
        ids [count] -> states [count, width]."""
        ids = np.ascontiguousarray(ids, np.int32)
        L = shape.layers

        def arr(fmt):
            keep = [np.ascontiguousarray(tensors[fmt.format(l)], np.float32) for l in range(L)]
            return keep, (c_float_p * L)(*[_fp(a) for a in keep])
        keeps = []
        ptrs = []
        for fmt in ("encoder.layers.{}.norm_self.weight", "encoder.layers.{}.self_attention.qkv_net.weight",
                    "encoder.layers.{}.self_attention.o_net.weight", "encoder.layers.{}.norm_pos_ff.weight",
                    "encoder.layers.{}.pos_ff.proj.conv.weight", "encoder.layers.{}.pos_ff.o_net.conv.weight"):
            k, p = arr(fmt)
            keeps.append(k); ptrs.append(p)
        out = np.empty((len(ids), shape.width), np.float32)
        rc = self.lib.orc_encode_text(ids.ctypes.data_as(C.POINTER(C.c_int)), len(ids), L, shape.width, shape.heads,
                                      shape.kernel, shape.vocab, _fp(tensors["text_embedding.weight"]),
                                      _fp(tensors["encoder.position_embeddings.weight"]),
                                      _fp(tensors["encoder.norm_out.weight"]), *ptrs, _fp(out))
        assert rc == 0
        return out

    def codec_decode(self, tensors: dict, shape, codes, stop_after: int = 0) -> np.ndarray:
        """The codec decoder over the reference-named tensors of synth.add_codec: codes
        [8, frames] -> samples [frames * 1024]; stop_after = 1: the first convolution's output
        [base, frames]; 2 + s: stage s's output [channels, length]."""
        codes = np.ascontiguousarray(codes, np.uint32)
        frames = codes.shape[1]
        desc, keep = CodecDesc(), []
        desc.base = shape.base
        fill_codec_desc(desc, tensors, keep)
        if stop_after == 0:
            dims = (frames * shape.samples_per_frame,)
        elif stop_after == 1:
            dims = (shape.base, frames)
        else:
            s = stop_after - 2
            dims = (shape.base >> (s + 1), frames * int(np.prod(shape.rates[:s + 1])))
        out = np.empty(dims, np.float32)
        n = self.lib.orc_codec_decode(C.byref(desc), codes.ctypes.data_as(c_uint_p), frames, stop_after, _fp(out))
        assert n == out.size, n
        return out

    def argmax_constrained(self, logits, codebook_size, eos_id, allow_eos) -> int:
        return int(self.lib.orc_argmax_constrained(_fp(logits), logits.size, codebook_size, eos_id,
                                                   int(allow_eos)))

    def self_attention(self, qkv, k_cache, v_cache, position, stride, valid, heads, hw, scale):
        out = np.empty((heads * hw,), np.float32)
        scores = np.empty((max(valid, 1),), np.float32)
        self.lib.orc_self_attention(_fp(qkv), _fp(k_cache), _fp(v_cache), position, stride, valid,
                                    heads, hw, scale, _fp(out), _fp(scores))
        return out

    def cross_attention(self, q, k_cache, v_cache, valid, stride, heads, hw, scale):
        out = np.empty((heads * hw,), np.float32)
        scores = np.empty((max(valid, 1),), np.float32)
        self.lib.orc_cross_attention(_fp(q), _fp(k_cache), _fp(v_cache), valid, stride, heads, hw,
                                     scale, _fp(out), _fp(scores))
        return out


class PortModel:
    """orc_model over a mynah_tts_b200.synth.SynthModel (weights are borrowed:
    the SynthModel must outlive this object)."""

    def __init__(self, synth, qtype: int):
        self.port = Port.get()
        self.synth = synth
        self.qtype = qtype
        s = synth.shape
        L = range(s.layers)

        def col(suffix):
            return [synth.layer(i, suffix) for i in L]

        self._keep = [
            _ptr_array(col("norm_self.weight")), _ptr_array(col("norm_xattn_query.weight")),
            _ptr_array(col("norm_xattn_memory.weight")), _ptr_array(col("norm_pos_ff.weight")),
            _ptr_array(col("self_attention.qkv_net.weight")),
            _ptr_array(col("self_attention.o_net.weight")),
            _ptr_array(col("cross_attention.q_net.weight")),
            _ptr_array(col("cross_attention.kv_net.weight")),
            _ptr_array(col("cross_attention.o_net.weight")),
            _ptr_array(col("pos_ff.proj.conv.weight")), _ptr_array(col("pos_ff.o_net.conv.weight")),
            _ptr_array([synth.embedding(t) for t in range(s.tables)]),
            _ptr_array([synth.head_weight(t) for t in range(s.tables)]),
            _ptr_array([synth.head_bias(t) for t in range(s.tables)]),
        ]
        k = self._keep
        sz = C.c_size_t
        self.handle = C.c_void_p(self.port.lib.orc_model_new(
            sz(s.layers), sz(s.width), sz(s.heads), sz(s.xattn_width), C.c_int(qtype),
            _fp(synth.position), _fp(synth.norm_out),
            k[0], k[1], k[2], k[3], k[4], k[5], k[6], k[7], k[8], k[9], k[10],
            sz(s.tables), sz(s.vocab), sz(s.codebook_size), sz(s.eos_id), k[11], k[12], k[13]))
        assert self.handle.value

    def close(self):
        if self.handle:
            self.port.lib.orc_model_free(self.handle)
            self.handle = None

    def new_stream(self, memory: np.ndarray, capacity: int) -> "PortStream":
        return PortStream(self, memory, capacity)

    def embed_frame(self, codes: np.ndarray) -> np.ndarray:
        row = np.empty((self.synth.shape.width,), np.float32)
        codes = np.ascontiguousarray(codes, np.uint32)
        assert self.port.lib.orc_embed_frame(self.handle, codes.ctypes.data_as(c_uint_p), _fp(row)) == 0
        return row

    def heads_argmax(self, hidden: np.ndarray, allow_eos: bool):
        s = self.synth.shape
        tokens = np.empty((s.tables,), np.uint32)
        logits = np.empty((s.tables, s.vocab), np.float32)
        self.port.lib.orc_heads_argmax(self.handle, _fp(hidden), int(allow_eos),
                                       tokens.ctypes.data_as(c_uint_p), _fp(logits))
        return tokens, logits


class PortLocal:
    """orc_local: one request's local-transformer state over a PortModel whose
    SynthModel has local_layers > 0."""

    def __init__(self, model: PortModel, top_count: int = 0):
        self.model = model
        synth = model.synth
        s = synth.shape
        assert s.local_layers > 0
        L = range(s.local_layers)

        def col(suffix):
            return _ptr_array([synth.local_layer(i, suffix) for i in L])
        self._keep = [col("norm_self.weight"), col("self_attention.qkv_net.weight"),
                      col("self_attention.o_net.weight"), col("norm_pos_ff.weight"),
                      col("pos_ff.proj.conv.weight"), col("pos_ff.o_net.conv.weight")]
        k = self._keep
        self.handle = C.c_void_p(model.port.lib.orc_local_new(
            model.handle, C.c_size_t(s.local_layers), _fp(synth.local_position),
            k[0], k[1], k[2], k[3], k[4], k[5], C.c_size_t(top_count)))
        assert self.handle.value

    def close(self):
        if self.handle:
            self.model.port.lib.orc_local_free(self.handle)
            self.handle = None

    @property
    def length(self) -> int:
        return self.model.port.lib.orc_local_length(self.handle)

    @length.setter
    def length(self, n: int):
        self.model.port.lib.orc_local_set_length(self.handle, n)

    def kv(self):
        s = self.model.synth.shape
        shape = (s.local_layers, s.local_positions, s.width)
        lib = self.model.port.lib
        n = int(np.prod(shape))
        return (np.ctypeslib.as_array(lib.orc_local_k(self.handle), shape=(n,)).reshape(shape),
                np.ctypeslib.as_array(lib.orc_local_v(self.handle), shape=(n,)).reshape(shape))

    def step(self, row: np.ndarray) -> np.ndarray:
        row = np.ascontiguousarray(row, np.float32)
        out = np.empty_like(row)
        assert self.model.port.lib.orc_local_step(self.handle, _fp(row), _fp(out)) == 0
        return out

    def frame(self, decoder_last: np.ndarray, temperature: float = 0.0, topk: int = 0,
              rng_state: int = 0, allow_eos: bool = True, codebooks: int | None = None):
        """-> codes [tables], values [tables], saw_eos, eos_frame, new rng state."""
        s = self.model.synth.shape
        codes = np.zeros((s.tables,), np.uint32)
        values = np.zeros((s.tables,), np.uint32)
        rng = C.c_uint64(rng_state)
        eos_frame = C.c_long(-1)
        row = np.ascontiguousarray(decoder_last, np.float32)
        rc = self.model.port.lib.orc_local_frame(
            self.handle, _fp(row), C.c_float(temperature), C.c_uint(topk), C.byref(rng),
            int(allow_eos), C.c_size_t(codebooks if codebooks else s.tables // 2),
            codes.ctypes.data_as(c_uint_p), values.ctypes.data_as(c_uint_p), C.byref(eos_frame))
        assert rc >= 0
        return codes, values, bool(rc), int(eos_frame.value), int(rng.value)


class PortStream:
    def __init__(self, model: PortModel, memory: np.ndarray, capacity: int):
        self.model = model
        self.lib = model.port.lib
        self.capacity = capacity
        self.memory_length = memory.shape[0]
        self.handle = C.c_void_p(self.lib.orc_stream_new(model.handle, _fp(memory),
                                                         memory.shape[0], capacity))
        assert self.handle.value

    def close(self):
        if self.handle:
            self.lib.orc_stream_free(self.handle)
            self.handle = None

    def _view(self, name, shape):
        ptr = getattr(self.lib, f"orc_stream_{name}")(self.handle)
        return np.ctypeslib.as_array(ptr, shape=shape)

    @property
    def self_k(self):
        s = self.model.synth.shape
        return self._view("self_k", (s.layers, self.capacity, s.width))

    @property
    def self_v(self):
        s = self.model.synth.shape
        return self._view("self_v", (s.layers, self.capacity, s.width))

    @property
    def cross_k(self):
        s = self.model.synth.shape
        return self._view("cross_k", (s.layers, self.memory_length, s.xattn_width))

    @property
    def cross_v(self):
        s = self.model.synth.shape
        return self._view("cross_v", (s.layers, self.memory_length, s.xattn_width))

    @property
    def length(self) -> int:
        return int(self.lib.orc_stream_length(self.handle))

    @length.setter
    def length(self, n: int):
        self.lib.orc_stream_set_length(self.handle, n)

    def set_layers(self, n: int):
        self.lib.orc_stream_set_layers(self.handle, n)

    def step(self, row: np.ndarray) -> np.ndarray:
        out = np.empty_like(row)
        assert self.lib.orc_decoder_step(self.handle, _fp(row), _fp(out)) == 0
        return out

    def prefill(self, rows: np.ndarray) -> np.ndarray:
        """decoder_run with count > 1 (src/graph.c:3506-3641): rows [count, width] at once."""
        rows = np.ascontiguousarray(rows, np.float32)
        out = np.empty((rows.shape[1],), np.float32)
        assert self.lib.orc_decoder_prefill(self.handle, _fp(rows), rows.shape[0], _fp(out)) == 0
        return out

    def greedy_frame(self, codes: np.ndarray, allow_eos: bool):
        s = self.model.synth.shape
        tokens = np.empty((s.tables,), np.uint32)
        hidden = np.empty((s.width,), np.float32)
        eos = self.lib.orc_greedy_frame(self.handle, codes.ctypes.data_as(c_uint_p), int(allow_eos),
                                        tokens.ctypes.data_as(c_uint_p), _fp(hidden))
        assert eos >= 0
        return tokens, hidden, bool(eos)

    def greedy_decode(self, codes: np.ndarray, frames: int, min_frames: int):
        s = self.model.synth.shape
        codes = np.ascontiguousarray(codes, np.uint32).copy()
        tokens = np.zeros((frames, s.tables), np.uint32)
        n = self.lib.orc_greedy_decode(self.handle, codes.ctypes.data_as(c_uint_p), frames,
                                       min_frames, tokens.ctypes.data_as(c_uint_p))
        assert n >= 0
        return tokens[:n]


# --------------------------------------------------------------------- Ref
class Ref:
    """Typed access to one of the compiled-reference libraries."""

    _instances: dict = {}

    def __init__(self, kind: str):
        self.kind = kind
        self.lib = lib = C.CDLL(REF_SO[kind])
        sz = C.c_size_t
        lib.ref_model_open.restype = C.c_void_p
        lib.ref_model_open.argtypes = [C.c_char_p, C.c_uint, C.c_uint, C.c_uint, C.c_uint, C.c_uint,
                                       C.c_uint, C.c_uint, C.c_int, C.c_char_p, sz]
        lib.ref_model_close.argtypes = [C.c_void_p]
        lib.ref_decoder_new.restype = C.c_void_p
        lib.ref_decoder_new.argtypes = [C.c_void_p, c_float_p, sz, sz, C.c_char_p, sz]
        lib.ref_decoder_free.argtypes = [C.c_void_p]
        lib.ref_decoder_length.restype = sz
        lib.ref_decoder_length.argtypes = [C.c_void_p]
        lib.ref_decoder_set_length.argtypes = [C.c_void_p, sz]
        lib.ref_decoder_set_layers.argtypes = [C.c_void_p, sz]
        for name in ("self_k", "self_v", "cross_k", "cross_v"):
            fn = getattr(lib, f"ref_decoder_{name}")
            fn.restype = c_float_p
            fn.argtypes = [C.c_void_p]
        lib.ref_decoder_step_batch.argtypes = [C.c_void_p, C.POINTER(C.c_void_p), c_float_p,
                                               c_float_p, sz, C.c_char_p, sz]
        lib.ref_decoder_run.argtypes = [C.c_void_p, C.c_void_p, c_float_p, sz, c_float_p,
                                        C.c_char_p, sz]
        lib.ref_encode_text.argtypes = [C.c_void_p, C.c_uint, C.c_uint, C.POINTER(C.c_int), sz, c_float_p, C.c_char_p, sz]
        lib.ref_decode_codec.restype = C.c_long
        lib.ref_decode_codec.argtypes = [C.c_void_p, c_uint_p, sz, c_float_p, C.c_char_p, sz]
        lib.ref_model_resident.argtypes = [C.c_void_p]
        lib.ref_model_backend_name.restype = C.c_char_p
        lib.ref_model_backend_name.argtypes = [C.c_void_p]
        lib.ref_decoder_download_kv.argtypes = [C.c_void_p, C.c_void_p, C.c_char_p, sz]
        lib.ref_heads_argmax.argtypes = [C.c_void_p, c_float_p, sz, C.c_int, c_uint_p, c_float_p,
                                         C.c_char_p, sz]
        lib.ref_greedy_decode.argtypes = [C.c_void_p, C.POINTER(C.c_void_p), sz, c_uint_p, sz, sz,
                                          c_uint_p, C.POINTER(C.c_long), C.c_char_p, sz]
        lib.ref_embed_audio_frame.argtypes = [C.c_void_p, c_uint_p, sz, sz, c_float_p, C.c_char_p, sz]
        lib.ref_model_set_local_layers.argtypes = [C.c_void_p, C.c_uint]
        lib.ref_local_new.restype = C.c_void_p
        lib.ref_local_new.argtypes = [C.c_void_p, sz, C.c_char_p, sz]
        lib.ref_local_free.argtypes = [C.c_void_p]
        lib.ref_local_length.restype = sz
        lib.ref_local_length.argtypes = [C.c_void_p]
        lib.ref_local_set_length.argtypes = [C.c_void_p, sz]
        lib.ref_local_k.restype = c_float_p
        lib.ref_local_k.argtypes = [C.c_void_p]
        lib.ref_local_v.restype = c_float_p
        lib.ref_local_v.argtypes = [C.c_void_p]
        lib.ref_local_step_batch.argtypes = [C.c_void_p, C.POINTER(C.c_void_p), c_float_p, c_float_p,
                                             sz, C.c_char_p, sz]
        lib.ref_local_frame.argtypes = [C.c_void_p, C.POINTER(C.c_void_p), sz, c_float_p, c_float_p,
                                        c_uint_p, C.POINTER(C.c_uint64), C.POINTER(C.c_int), c_uint_p,
                                        C.POINTER(C.c_int), C.POINTER(C.c_long), C.c_char_p, sz]
        lib.ref_quantize_act_int8.restype = C.c_float
        lib.ref_quantize_act_int8.argtypes = [C.c_void_p, c_float_p, sz]
        lib.ref_qmat_linear.argtypes = [C.c_int, c_float_p, c_float_p, c_float_p, sz, sz, sz,
                                        c_float_p, C.c_char_p, sz]
        lib.ref_qmat_linear_batched.argtypes = lib.ref_qmat_linear.argtypes
        lib.ref_self_tests.argtypes = [C.c_char_p, sz]
        lib.mynah_layernorm_f32.argtypes = [c_float_p, c_float_p, c_float_p, c_float_p, sz, sz,
                                            C.c_float]
        lib.mynah_gelu_f32_scalar.argtypes = [c_float_p, sz]

    @classmethod
    def get(cls, kind: str = "strict") -> "Ref":
        if kind not in cls._instances:
            cls._instances[kind] = cls(kind)
        return cls._instances[kind]

    def self_tests(self):
        err = C.create_string_buffer(256)
        return self.lib.ref_self_tests(err, 256), err.value.decode()

    def quantize_weight_int8(self, w):
        n, k = w.shape
        q = np.empty((n, k), np.int8)
        s = np.empty((n,), np.float32)
        self.lib.ref_quantize_weight_int8(_fp(w), C.c_size_t(n), C.c_size_t(k),
                                          q.ctypes.data_as(C.c_void_p), _fp(s))
        return q, s

    def quantize_weight_int4(self, w):
        n, k = w.shape
        q = np.empty((n, k // 2), np.uint8)
        s = np.empty((n, k // 32), np.float32)
        self.lib.ref_quantize_weight_int4(_fp(w), C.c_size_t(n), C.c_size_t(k),
                                          q.ctypes.data_as(C.c_void_p), _fp(s))
        return q, s

    def quantize_act_int8(self, x):
        q = np.empty(x.shape, np.int8)
        sx = self.lib.ref_quantize_act_int8(q.ctypes.data_as(C.c_void_p), _fp(x), x.size)
        return q, np.float32(sx)

    def layernorm(self, x, gain, eps=1e-5):
        x2 = np.ascontiguousarray(x.reshape(-1, x.shape[-1]))
        y = np.empty_like(x2)
        self.lib.mynah_layernorm_f32(_fp(x2), _fp(gain), None, _fp(y), x2.shape[0], x2.shape[1], eps)
        return y.reshape(x.shape)

    def gelu(self, x):
        y = np.ascontiguousarray(x.copy())
        self.lib.mynah_gelu_f32_scalar(_fp(y), y.size)
        return y

    def qmat_linear(self, qtype, w, x, bias=None, batched=False):
        x2 = np.ascontiguousarray(x.reshape(-1, x.shape[-1]))
        n, k = w.shape[0], w.shape[1]
        out = np.empty((x2.shape[0], n), np.float32)
        err = C.create_string_buffer(256)
        fn = self.lib.ref_qmat_linear_batched if batched else self.lib.ref_qmat_linear
        rc = fn(qtype, _fp(w), _fp(x2), _fp(out), x2.shape[0], k, n,
                None if bias is None else _fp(bias), err, 256)
        assert rc == 0, err.value
        return out


class RefModel:
    """The reference's model struct over a synthetic safetensors file.

    `tables` stacked streams are presented to the reference as
    frame_stacking_factor 2 x codebook_count tables/2, the only stacking its
    embed_audio_frame accepts (src/graph.c:767-770)."""

    def __init__(self, synth, qtype: int, kind: str = "strict", threads: int | None = None):
        from mynah_tts_b200.synth import write_safetensors
        if threads is not None:
            os.environ["MYNAH_THREADS"] = str(threads)
        self.ref = Ref.get(kind)
        self.synth = synth
        s = synth.shape
        assert s.tables % 2 == 0
        self._dir = tempfile.TemporaryDirectory(prefix="mynah_ref_")
        path = os.path.join(self._dir.name, "tts.safetensors")
        write_safetensors(path, synth.tensors)
        err = C.create_string_buffer(512)
        self.handle = C.c_void_p(self.ref.lib.ref_model_open(
            path.encode(), s.width, s.layers, s.tables // 2, 2, s.codebook_size, s.vocab,
            s.eos_id, qtype, err, 512))
        assert self.handle.value, err.value
        if s.local_layers:
            self.ref.lib.ref_model_set_local_layers(self.handle, s.local_layers)

    def embed_frame(self, codes: np.ndarray) -> np.ndarray:
        """codes [tables] with table = fs * codebooks + codebook -> decoder input row
        (embed_audio_frame, src/graph.c:760-804)."""
        s = self.synth.shape
        codebooks = s.tables // 2
        flat = np.ascontiguousarray(codes, np.uint32).reshape(2, codebooks)   # [fs][codebook]
        laid = np.ascontiguousarray(flat.T)                                   # [codebook][fs]
        row = np.empty((s.width,), np.float32)
        err = C.create_string_buffer(256)
        rc = self.ref.lib.ref_embed_audio_frame(self.handle, laid.ctypes.data_as(c_uint_p), 2, 0,
                                                _fp(row), err, 256)
        assert rc == 0, err.value
        return row

    def decode_codec(self, codes) -> np.ndarray:
        """decode_codec (src/graph.c:2640-2780): codes [8, frames] -> samples [frames * 1024];
        the model's tensors must include synth.add_codec's at base 864."""
        codes = np.ascontiguousarray(codes, np.uint32)
        out = np.empty((codes.shape[1] * 1024,), np.float32)
        err = C.create_string_buffer(256)
        n = self.ref.lib.ref_decode_codec(self.handle, codes.ctypes.data_as(c_uint_p), codes.shape[1], _fp(out), err, 256)
        assert n == out.size, err.value
        return out

    def new_local(self, top_count: int = 0) -> "RefLocal":
        return RefLocal(self, top_count)

    def local_step_batch(self, locals_, rows: np.ndarray) -> np.ndarray:
        rows = np.ascontiguousarray(rows, np.float32)
        outs = np.empty_like(rows)
        arr = (C.c_void_p * len(locals_))(*[l.handle for l in locals_])
        err = C.create_string_buffer(256)
        rc = self.ref.lib.ref_local_step_batch(self.handle, arr, _fp(rows), _fp(outs), len(locals_), err, 256)
        assert rc == 0, err.value
        return outs

    def local_frame(self, locals_, decoder_last: np.ndarray, temperature, topk, rng_states, allow_eos):
        """One stacked frame for len(locals_) requests (<= 16) ->
        codes [batch, tables], saw_eos [batch], eos_frame [batch], new rng states."""
        s = self.synth.shape
        batch = len(locals_)
        rows = np.ascontiguousarray(decoder_last, np.float32)
        temp = np.ascontiguousarray(temperature, np.float32)
        tk = np.ascontiguousarray(topk, np.uint32)
        rng = (C.c_uint64 * batch)(*[int(x) for x in rng_states])
        allow = (C.c_int * batch)(*[int(bool(x)) for x in allow_eos])
        codes = np.zeros((batch, s.tables), np.uint32)
        saw = (C.c_int * batch)()
        eos = (C.c_long * batch)()
        arr = (C.c_void_p * batch)(*[l.handle for l in locals_])
        err = C.create_string_buffer(256)
        rc = self.ref.lib.ref_local_frame(self.handle, arr, batch, _fp(rows), _fp(temp),
                                          tk.ctypes.data_as(c_uint_p), rng, allow,
                                          codes.ctypes.data_as(c_uint_p), saw, eos, err, 256)
        assert rc == 0, err.value
        return codes, np.array(list(saw)), np.array(list(eos)), [int(x) for x in rng]

    def close(self):
        if self.handle:
            self.ref.lib.ref_model_close(self.handle)
            self.handle = None
            self._dir.cleanup()

    def new_decoder(self, memory: np.ndarray, capacity: int) -> "RefDecoder":
        return RefDecoder(self, memory, capacity)

    def encode_text(self, shape, ids) -> np.ndarray:
        """encode_text (src/graph.c:709-748) over the model file's "encoder" tensors."""
        ids = np.ascontiguousarray(ids, np.int32)
        out = np.empty((len(ids), shape.width), np.float32)
        err = C.create_string_buffer(256)
        rc = self.ref.lib.ref_encode_text(self.handle, shape.layers, shape.max_length,
                                          ids.ctypes.data_as(C.POINTER(C.c_int)), len(ids), _fp(out), err, 256)
        assert rc == 0, err.value
        return out

    @property
    def resident(self) -> bool:
        """True when decoder_run takes its resident device path (src/graph.c:3363-3368)."""
        return bool(self.ref.lib.ref_model_resident(self.handle))

    @property
    def backend_name(self) -> str:
        return self.ref.lib.ref_model_backend_name(self.handle).decode()

    def step_batch(self, decoders, rows: np.ndarray) -> np.ndarray:
        rows = np.ascontiguousarray(rows, np.float32)
        outs = np.empty_like(rows)
        arr = (C.c_void_p * len(decoders))(*[d.handle for d in decoders])
        err = C.create_string_buffer(256)
        rc = self.ref.lib.ref_decoder_step_batch(self.handle, arr, _fp(rows), _fp(outs),
                                                 len(decoders), err, 256)
        assert rc == 0, err.value
        return outs

    def heads_argmax(self, hidden, allow_eos):
        s = self.synth.shape
        tokens = np.empty((s.tables,), np.uint32)
        logits = np.empty((s.tables, s.vocab), np.float32)
        err = C.create_string_buffer(256)
        rc = self.ref.lib.ref_heads_argmax(self.handle, _fp(hidden), s.tables, int(allow_eos),
                                           tokens.ctypes.data_as(c_uint_p), _fp(logits), err, 256)
        assert rc == 0, err.value
        return tokens, logits

    def greedy_decode(self, decoders, codes: np.ndarray, frames: int, min_frames: int):
        """codes [batch, tables] -> tokens [frames, batch, tables], eos_frame [batch]."""
        s = self.synth.shape
        batch = len(decoders)
        codes = np.ascontiguousarray(codes, np.uint32).copy()
        tokens = np.zeros((frames, batch, s.tables), np.uint32)
        eos = (C.c_long * batch)()
        arr = (C.c_void_p * batch)(*[d.handle for d in decoders])
        err = C.create_string_buffer(256)
        rc = self.ref.lib.ref_greedy_decode(self.handle, arr, batch, codes.ctypes.data_as(c_uint_p),
                                            frames, min_frames, tokens.ctypes.data_as(c_uint_p),
                                            eos, err, 256)
        assert rc == 0, err.value
        return tokens, np.array(list(eos))


class RefLocal:
    def __init__(self, model: RefModel, top_count: int = 0):
        self.model = model
        err = C.create_string_buffer(256)
        self.handle = C.c_void_p(model.ref.lib.ref_local_new(model.handle, top_count, err, 256))
        assert self.handle.value, err.value

    def close(self):
        if self.handle:
            self.model.ref.lib.ref_local_free(self.handle)
            self.handle = None

    @property
    def length(self):
        return self.model.ref.lib.ref_local_length(self.handle)

    @length.setter
    def length(self, n):
        self.model.ref.lib.ref_local_set_length(self.handle, n)


class RefDecoder:
    def __init__(self, model: RefModel, memory: np.ndarray, capacity: int):
        self.model = model
        self.lib = model.ref.lib
        self.capacity = capacity
        self.memory_length = memory.shape[0]
        err = C.create_string_buffer(256)
        self.handle = C.c_void_p(self.lib.ref_decoder_new(model.handle, _fp(memory),
                                                          memory.shape[0], capacity, err, 256))
        assert self.handle.value, err.value

    def close(self):
        if self.handle:
            self.lib.ref_decoder_free(self.handle)
            self.handle = None

    def _view(self, name, shape):
        return np.ctypeslib.as_array(getattr(self.lib, f"ref_decoder_{name}")(self.handle), shape=shape)

    @property
    def self_k(self):
        s = self.model.synth.shape
        return self._view("self_k", (s.layers, self.capacity, s.width))

    @property
    def self_v(self):
        s = self.model.synth.shape
        return self._view("self_v", (s.layers, self.capacity, s.width))

    @property
    def cross_k(self):
        s = self.model.synth.shape
        return self._view("cross_k", (s.layers, self.memory_length, s.xattn_width))

    @property
    def cross_v(self):
        s = self.model.synth.shape
        return self._view("cross_v", (s.layers, self.memory_length, s.xattn_width))

    @property
    def length(self):
        return int(self.lib.ref_decoder_length(self.handle))

    @length.setter
    def length(self, n):
        self.lib.ref_decoder_set_length(self.handle, n)

    def set_layers(self, n):
        self.lib.ref_decoder_set_layers(self.handle, n)

    def step(self, row: np.ndarray) -> np.ndarray:
        return self.model.step_batch([self], row.reshape(1, -1))[0]

    def run(self, rows: np.ndarray) -> np.ndarray:
        """decoder_run (src/graph.c:3286-3654) over `rows` new rows; the output-norm row of
        the last one."""
        rows = np.ascontiguousarray(rows, np.float32).reshape(-1, self.model.synth.shape.width)
        out = np.empty((rows.shape[1],), np.float32)
        err = C.create_string_buffer(256)
        rc = self.lib.ref_decoder_run(self.model.handle, self.handle, _fp(rows), rows.shape[0], _fp(out), err, 256)
        assert rc == 0, err.value
        return out

    def download_kv(self):
        """Resident path only: copy the device self K/V back into the host cache arrays."""
        err = C.create_string_buffer(256)
        rc = self.lib.ref_decoder_download_kv(self.model.handle, self.handle, err, 256)
        assert rc == 0, err.value or b"no device cache"
