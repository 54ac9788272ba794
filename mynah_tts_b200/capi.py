"""ctypes binding of libmynah_b200.so (the C ABI of include/mynah_b200.h).

The library is the product; this module only loads it and gives the entry
points Python-friendly signatures for the tests and the benchmark.  There is no
fallback of any kind: if the shared library is missing, importing fails with
the build command to run.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libmynah_b200.so")

F32, INT8, INT4, F16 = 0, 1, 2, 3
QUANT = {"f32": F32, "int8": INT8, "int4": INT4, "f16": F16}
ERR_CAP = 512
PROFILE_CLASSES = 16

c_float_p = C.POINTER(C.c_float)
c_uint_p = C.POINTER(C.c_uint)
c_int_p = C.POINTER(C.c_int)
sz = C.c_size_t


class MynahB200Error(RuntimeError):
    pass


def load_library() -> C.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `make -C {os.path.join(HERE, 'csrc')}` "
            "(or `python -c 'import __graft_entry__ as g; g.build()'`); there is no CPU fallback")
    return C.CDLL(LIB_PATH)


class LayerWeights(C.Structure):
    _fields_ = [(n, c_float_p) for n in (
        "norm_self", "norm_xattn_query", "norm_pos_ff", "qkv_w", "o_self_w", "q_cross_w",
        "o_cross_w", "ffn_up_w", "ffn_down_w", "norm_xattn_memory", "kv_cross_w")]


class DecoderDesc(C.Structure):
    _fields_ = [
        ("layers", sz), ("width", sz), ("heads", sz), ("xattn_width", sz),
        ("memory_length", sz), ("capacity", sz), ("slots", sz), ("max_batch", sz),
        ("max_positions", sz), ("layer", C.POINTER(LayerWeights)),
        ("position", c_float_p), ("norm_out", c_float_p),
        ("tables", sz), ("vocab", sz), ("codebook_size", sz), ("eos_id", sz),
        ("embeddings", C.POINTER(c_float_p)), ("head_w", C.POINTER(c_float_p)),
        ("head_b", C.POINTER(c_float_p)),
        ("keep_f32_weights", C.c_int),
    ]


class LocalLayerWeights(C.Structure):
    _fields_ = [(n, c_float_p) for n in (
        "norm_self", "norm_pos_ff", "qkv_w", "o_w", "ffn_up_w", "ffn_down_w")]


class LocalDesc(C.Structure):
    _fields_ = [("layers", sz), ("layer", C.POINTER(LocalLayerWeights)), ("position", c_float_p),
                ("position_rows", sz), ("codebooks", sz)]


class EncoderLayerWeights(C.Structure):
    _fields_ = [(n, c_float_p) for n in ("norm_self", "norm_pos_ff", "qkv_w", "o_w", "ffn_proj_w", "ffn_out_w")]


class EncoderDesc(C.Structure):
    _fields_ = [("layers", sz), ("width", sz), ("heads", sz), ("kernel", sz), ("vocab", sz), ("max_length", sz),
                ("layer", C.POINTER(EncoderLayerWeights)), ("embedding", c_float_p), ("position", c_float_p),
                ("norm_out", c_float_p)]


class CodecBlock(C.Structure):
    _fields_ = [(n, c_float_p) for n in ("in_alpha", "in_w", "in_b", "skip_alpha", "skip_w", "skip_b")]


class CodecStage(C.Structure):
    _fields_ = [("alpha", c_float_p), ("up_w", c_float_p), ("up_b", c_float_p), ("block", (CodecBlock * 3) * 3)]


class CodecDesc(C.Structure):
    _fields_ = [("base", sz), ("max_frames", sz), ("pre_w", c_float_p), ("pre_b", c_float_p),
                ("stage", CodecStage * 5), ("post_alpha", c_float_p), ("post_w", c_float_p), ("post_b", c_float_p),
                ("arithmetic", C.c_int)]


class Sampler(C.Structure):
    _fields_ = [("temperature", C.c_float), ("topk", C.c_uint), ("rng_state", C.c_ulonglong),
                ("allow_eos", C.c_int)]


class Request(C.Structure):
    _fields_ = [("memory", c_float_p), ("memory_length", sz), ("start_codes", c_uint_p), ("max_frames", sz), ("min_frames", sz),
                ("sampler", Sampler), ("codes", c_uint_p), ("frames_done", sz), ("eos_frame", C.c_long),
                ("admitted_at", sz)]


MATMUL_FN = C.CFUNCTYPE(C.c_int, C.c_void_p, c_float_p, c_float_p, sz, sz, sz, c_float_p, c_float_p,
                        C.c_char_p, sz)
SGEMM_FN = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_int, C.c_int, sz, sz, sz, C.c_float, c_float_p, sz,
                       c_float_p, sz, C.c_float, c_float_p, sz, C.c_char_p, sz)
CLOSE_FN = C.CFUNCTYPE(None, C.c_void_p)
SELF_TEST_FN = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_char_p, sz)

# name -> (restype, argtypes); the trailing (char *error, size_t cap) pair is added
# for every entry whose last two argtypes are "ERR".
_E = "ERR"
SIGNATURES = {
    "mynah_backend_cuda_open": (C.c_int, [C.POINTER(C.c_void_p), C.POINTER(MATMUL_FN),
                                          C.POINTER(SGEMM_FN), C.POINTER(CLOSE_FN),
                                          C.POINTER(SELF_TEST_FN), _E]),
    "mynah_cuda_upload": (C.c_int, [C.c_void_p, c_float_p, sz, C.POINTER(C.c_void_p), _E]),
    "mynah_cuda_download": (C.c_int, [C.c_void_p, C.c_void_p, c_float_p, sz, _E]),
    "mynah_cuda_sync": (C.c_int, [C.c_void_p, _E]),
    "mynah_cuda_dev_alloc": (C.c_int, [C.c_void_p, sz, C.POINTER(C.c_void_p), _E]),
    "mynah_cuda_dev_free": (None, [C.c_void_p, C.c_void_p]),
    "mynah_cuda_h2d": (C.c_int, [C.c_void_p, c_float_p, C.c_void_p, sz, _E]),
    "mynah_cuda_d2h": (C.c_int, [C.c_void_p, C.c_void_p, c_float_p, sz, _E]),
    "mynah_cuda_gelu_dev": (C.c_int, [C.c_void_p, C.c_void_p, sz, _E]),
    "mynah_cuda_gelu_inplace": (C.c_int, [C.c_void_p, C.c_void_p, sz, _E]),
    "mynah_cuda_layer_norm_dev": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, c_float_p, c_float_p,
                                            sz, sz, _E]),
    "mynah_cuda_layer_norm_inplace": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, c_float_p, sz, sz, _E]),
    "mynah_cuda_residual_add_dev": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, sz, _E]),
    "mynah_cuda_residual_inplace": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, sz, _E]),
    "mynah_cuda_matmul_dev": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, sz, sz, sz, c_float_p, c_float_p, _E]),
    "mynah_cuda_matmul_d2d": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, sz, sz, sz, c_float_p, c_float_p, _E]),
    "mynah_cuda_matmul_to_dev": (C.c_int, [C.c_void_p, c_float_p, C.c_void_p, sz, sz, sz, c_float_p, c_float_p, _E]),
    "mynah_cuda_matmul_graph": (C.c_int, [C.c_void_p, c_float_p, c_float_p, sz, sz, sz, c_float_p, c_float_p, _E]),
    "mynah_cuda_matvec_dev": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, sz, sz, c_float_p, c_float_p, _E]),
    "mynah_cuda_sgemm_dev": (C.c_int, [C.c_void_p, C.c_int, C.c_int, sz, sz, sz, C.c_float, C.c_void_p, sz,
                                       C.c_void_p, sz, C.c_float, C.c_void_p, sz, _E]),
    "mynah_cuda_batch_begin": (C.c_int, [C.c_void_p, _E]),
    "mynah_cuda_self_attention_dev": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, sz, sz, sz, sz,
                                                sz, C.c_float, C.c_void_p, _E]),
    "mynah_cuda_cross_attention_dev": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, sz, sz, sz, sz,
                                                 C.c_float, C.c_void_p, _E]),
    "mynah_cuda_copy_dev": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, sz, _E]),
    "mynah_cuda_scale_dev": (C.c_int, [C.c_void_p, C.c_void_p, sz, C.c_float, _E]),
    "mynah_cuda_clip_dev": (C.c_int, [C.c_void_p, C.c_void_p, sz, _E]),
    "mynah_cuda_argmax_dev": (C.c_int, [C.c_void_p, C.c_void_p, sz, sz, sz, C.c_int, c_uint_p, _E]),
    "mynah_cuda_gelu_host": (C.c_int, [C.c_void_p, c_float_p, sz, _E]),
    "mynah_cuda_gelu_host_f64": (C.c_int, [C.c_void_p, c_float_p, sz, _E]),
    "mynah_cuda_snake_dev": (C.c_int, [C.c_void_p, C.c_void_p, c_float_p, sz, sz, sz, _E]),
    "mynah_cuda_im2col": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, _E]),
    "mynah_cuda_conv1d": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int,
                                    C.c_int, c_float_p, c_float_p, _E]),
    "mynah_cuda_conv_transpose_dev": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int,
                                                C.c_int, C.c_int, C.c_int, c_float_p, c_float_p, _E]),
    "mynah_b200_open": (C.c_int, [C.POINTER(C.c_void_p), C.c_int, C.c_int, C.c_int, _E]),
    "mynah_b200_close": (None, [C.c_void_p]),
    "mynah_b200_set_stream": (C.c_int, [C.c_void_p, C.c_void_p, _E]),
    "mynah_b200_timer_start": (C.c_int, [C.c_void_p, _E]),
    "mynah_b200_timer_stop": (C.c_int, [C.c_void_p, c_float_p, _E]),
    "mynah_b200_libm_exact": (C.c_int, [C.c_void_p]),
    "mynah_b200_quant": (C.c_int, [C.c_void_p]),
    "mynah_b200_strict": (C.c_int, [C.c_void_p]),
    "mynah_b200_launch_count": (C.c_ulonglong, [C.c_void_p]),
    "mynah_b200_pack_weight": (C.c_int, [C.c_void_p, C.c_int, c_float_p, sz, sz, C.c_void_p, c_float_p, _E]),
    "mynah_b200_quantize_act": (C.c_int, [C.c_void_p, c_float_p, sz, sz, C.c_void_p, c_float_p, _E]),
    "mynah_b200_qmat_linear": (C.c_int, [C.c_void_p, c_float_p, c_float_p, c_float_p, sz, sz, sz,
                                         c_float_p, c_float_p, _E]),
    "mynah_b200_time_product": (C.c_int, [C.c_void_p, sz, sz, sz, C.c_int, C.c_int, sz, c_float_p, _E]),
    "mynah_b200_pool_create": (C.c_int, [C.c_void_p, c_float_p, sz, sz, sz, c_float_p, c_float_p,
                                         C.POINTER(C.c_void_p), _E]),
    "mynah_b200_pool_destroy": (None, [C.c_void_p]),
    "mynah_b200_pool_linear": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, _E]),
    "mynah_b200_pool_bytes_per_pass": (sz, [C.c_void_p]),
    "mynah_b200_decoder_create": (C.c_int, [C.c_void_p, C.POINTER(DecoderDesc), C.POINTER(C.c_void_p), _E]),
    "mynah_b200_decoder_destroy": (None, [C.c_void_p]),
    "mynah_b200_decoder_slot_load": (C.c_int, [C.c_void_p, sz, c_float_p, c_float_p, sz, c_float_p, c_float_p, sz, _E]),
    "mynah_b200_decoder_slot_prefill": (C.c_int, [C.c_void_p, sz, c_float_p, sz, _E]),
    "mynah_b200_decoder_prefill": (C.c_int, [C.c_void_p, sz, c_float_p, sz, c_float_p, _E]),
    "mynah_b200_codec_create": (C.c_int, [C.c_void_p, C.POINTER(CodecDesc), C.POINTER(C.c_void_p), _E]),
    "mynah_b200_codec_destroy": (None, [C.c_void_p]),
    "mynah_b200_codec_samples_per_frame": (sz, []),
    "mynah_b200_codec_decode": (C.c_int, [C.c_void_p, c_uint_p, sz, c_float_p, C.POINTER(sz), _E]),
    "mynah_b200_codec_decode_partial": (C.c_int, [C.c_void_p, c_uint_p, sz, C.c_int, c_float_p, sz, C.POINTER(sz), _E]),
    "mynah_b200_codec_time": (C.c_int, [C.c_void_p, c_uint_p, sz, C.c_int, c_float_p, _E]),
    "mynah_b200_encoder_create": (C.c_int, [C.c_void_p, C.POINTER(EncoderDesc), C.POINTER(C.c_void_p), _E]),
    "mynah_b200_encoder_destroy": (None, [C.c_void_p]),
    "mynah_b200_encoder_encode": (C.c_int, [C.c_void_p, c_int_p, sz, c_float_p, _E]),
    "mynah_b200_decoder_slot_read_cross": (C.c_int, [C.c_void_p, sz, c_float_p, c_float_p, _E]),
    "mynah_b200_decoder_slot_length": (C.c_int, [C.c_void_p, sz, C.POINTER(sz), _E]),
    "mynah_b200_decoder_slot_set_length": (C.c_int, [C.c_void_p, sz, sz, _E]),
    "mynah_b200_decoder_slot_read_kv": (C.c_int, [C.c_void_p, sz, c_float_p, c_float_p, _E]),
    "mynah_b200_decoder_set_layers": (C.c_int, [C.c_void_p, sz, _E]),
    "mynah_b200_decoder_step_batch": (C.c_int, [C.c_void_p, c_uint_p, C.POINTER(c_float_p),
                                                C.POINTER(c_float_p), sz, _E]),
    "mynah_b200_decoder_frame_batch": (C.c_int, [C.c_void_p, c_uint_p, c_uint_p, c_int_p, c_uint_p,
                                                 c_float_p, sz, _E]),
    "mynah_b200_decoder_greedy": (C.c_int, [C.c_void_p, c_uint_p, sz, c_uint_p, C.POINTER(sz), sz,
                                            c_uint_p, C.POINTER(C.c_long), c_float_p, _E]),
    "mynah_b200_decoder_local_attach": (C.c_int, [C.c_void_p, C.POINTER(LocalDesc), _E]),
    "mynah_b200_decoder_local_frame": (C.c_int, [C.c_void_p, c_float_p, sz, C.POINTER(Sampler), c_uint_p,
                                                 c_uint_p, c_int_p, C.POINTER(C.c_long), _E]),
    "mynah_b200_decoder_generate": (C.c_int, [C.c_void_p, c_uint_p, sz, c_uint_p, C.POINTER(sz), sz,
                                              C.POINTER(Sampler), c_uint_p, C.POINTER(C.c_long), c_float_p, _E]),
    "mynah_b200_decoder_frame_batch_local": (C.c_int, [C.c_void_p, c_uint_p, c_uint_p, C.POINTER(Sampler),
                                                       c_uint_p, c_uint_p, c_int_p, C.POINTER(C.c_long), sz, _E]),
    "mynah_b200_decoder_serve": (C.c_int, [C.c_void_p, C.POINTER(Request), sz, C.POINTER(sz), _E]),
    "mynah_b200_decoder_profile": (C.c_int, [C.c_void_p, C.c_int, _E]),
    "mynah_b200_decoder_profile_read": (C.c_int, [C.c_void_p, C.POINTER(C.c_ulonglong),
                                                  C.POINTER(C.c_double), sz, _E]),
    "mynah_b200_profile_class_name": (C.c_char_p, [sz]),
    "mynah_b200_self_attention_static": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, sz, sz, sz, sz, sz,
                                                   C.c_float, C.c_void_p, C.c_void_p, _E]),
    "mynah_b200_decoder_weight_bytes": (sz, [C.c_void_p]),
    "mynah_b200_decoder_kv_bytes": (sz, [C.c_void_p, sz]),
}


def bind(lib: C.CDLL) -> C.CDLL:
    """Attach restype/argtypes to every declared entry point; a symbol the header
    declares but the library lacks raises AttributeError here."""
    for name, (restype, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = restype
        fn.argtypes = [a for a in args if a is not _E] + ([C.c_char_p, sz] if _E in args else [])
    return lib


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        _lib = bind(load_library())
    return _lib


def fp(a: np.ndarray):
    assert a.dtype == np.float32 and a.flags["C_CONTIGUOUS"], (a.dtype, a.flags)
    return a.ctypes.data_as(c_float_p)


def call(fn, *args):
    """Call an entry point that ends in (char *error, size_t cap); raise on -1."""
    err = C.create_string_buffer(ERR_CAP)
    rc = fn(*args, err, ERR_CAP)
    if rc != 0:
        raise MynahB200Error(err.value.decode(errors="replace") or f"{fn.__name__} failed ({rc})")
    return rc
