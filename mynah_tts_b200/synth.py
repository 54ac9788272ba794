"""Seeded synthetic Magpie-shaped decoder weights and inputs.

The real Magpie checkpoint is not available offline, so every test and
benchmark runs on random-init weights with the reference's tensor names, shapes
and layer structure (src/graph.c:2978-3079 in mynah-tts): per layer four
gain-only LayerNorms, qkv_net [3W,W], o_net [W,W], cross q_net [xw,W],
kv_net [2xw,W], o_net [W,xw], FFN proj [4W,W,1] and o_net [W,4W,1]; plus
position embeddings, the output norm, one embedding table and one logit head
(weight + bias) per stacked codebook stream; optionally the local transformer
(src/graph.c:1021-1056): its position rows and per layer two norms, qkv_net,
o_net and the two FFN matrices.

Distributions: linear weights, embeddings and position rows ~ N(0, 0.02);
LayerNorm gains ~ N(1, 0.01); head biases ~ N(0, 0.01); text-encoder memory
~ N(0, 1).  numpy's default_rng(seed) is bit-reproducible across machines, so
the same seed gives the same model here and on the GPU box.
"""
from __future__ import annotations

import json
import struct
from dataclasses import dataclass, field

import numpy as np


@dataclass(frozen=True)
class DecoderShape:
    layers: int = 12
    width: int = 768
    heads: int = 12            # fixed at 12 in the reference (src/graph.c:2971)
    xattn_width: int = 128     # q_net.shape[0] of the real checkpoint
    memory_length: int = 128   # text-encoder states
    max_positions: int = 2048  # rows of decoder.position_embeddings.weight
    tables: int = 8            # stacked codebook streams (stacking * codebooks)
    vocab: int = 2048
    codebook_size: int = 2016
    eos_id: int = 2017
    local_layers: int = 0      # layers of the local transformer (0: none; the real model has 2)

    @property
    def local_positions(self) -> int:
        return self.tables + 1   # rows the local transformer can attend (src/graph.c:1200)

    @property
    def head_width(self) -> int:
        return self.width // self.heads

    @property
    def ffn_width(self) -> int:
        return 4 * self.width   # src/graph.c:2973


MAGPIE_357M = DecoderShape()
# Small shape for fast CPU tests: same structure, 12 heads of 16.
TINY = DecoderShape(layers=2, width=192, xattn_width=32, memory_length=24,
                    max_positions=96, tables=4, vocab=64, codebook_size=56, eos_id=57)
# The same two with a local transformer; the full size has the real model's 16 stacked
# streams (8 codebooks x 2 frames) and 2 local layers.
MAGPIE_357M_LOCAL = DecoderShape(tables=16, local_layers=2)
TINY_LOCAL = DecoderShape(layers=2, width=192, xattn_width=32, memory_length=24,
                          max_positions=96, tables=4, vocab=64, codebook_size=56, eos_id=57,
                          local_layers=2)

LOCAL_LAYER_TENSORS = (
    ("norm_self.weight", "gain"),
    ("norm_pos_ff.weight", "gain"),
    ("self_attention.qkv_net.weight", "qkv"),
    ("self_attention.o_net.weight", "o_self"),
    ("pos_ff.proj.conv.weight", "ffn_up"),
    ("pos_ff.o_net.conv.weight", "ffn_down"),
)

LAYER_TENSORS = (
    ("norm_self.weight", "gain"),
    ("norm_xattn_query.weight", "gain"),
    ("norm_xattn_memory.weight", "gain"),
    ("norm_pos_ff.weight", "gain"),
    ("self_attention.qkv_net.weight", "qkv"),
    ("self_attention.o_net.weight", "o_self"),
    ("cross_attention.q_net.weight", "q_cross"),
    ("cross_attention.kv_net.weight", "kv_cross"),
    ("cross_attention.o_net.weight", "o_cross"),
    ("pos_ff.proj.conv.weight", "ffn_up"),
    ("pos_ff.o_net.conv.weight", "ffn_down"),
)


def _layer_shapes(s: DecoderShape) -> dict[str, tuple[int, ...]]:
    w, xw, f = s.width, s.xattn_width, s.ffn_width
    return {
        "gain": (w,),
        "qkv": (3 * w, w),
        "o_self": (w, w),
        "q_cross": (xw, w),
        "kv_cross": (2 * xw, w),
        "o_cross": (w, xw),
        "ffn_up": (f, w, 1),
        "ffn_down": (w, f, 1),
    }


@dataclass
class SynthModel:
    shape: DecoderShape
    seed: int
    tensors: dict[str, np.ndarray] = field(default_factory=dict)

    def layer(self, index: int, suffix: str) -> np.ndarray:
        return self.tensors[f"decoder.layers.{index}.{suffix}"]

    def embedding(self, table: int) -> np.ndarray:
        return self.tensors[f"audio_embeddings.{table}.weight"]

    def head_weight(self, table: int) -> np.ndarray:
        return self.tensors[f"local_transformer_out_projections.{table}.weight"]

    def head_bias(self, table: int) -> np.ndarray:
        return self.tensors[f"local_transformer_out_projections.{table}.bias"]

    def local_layer(self, index: int, suffix: str) -> np.ndarray:
        return self.tensors[f"local_transformer.layers.{index}.{suffix}"]

    @property
    def local_position(self) -> np.ndarray:
        return self.tensors["local_transformer.position_embeddings.weight"]

    @property
    def position(self) -> np.ndarray:
        return self.tensors["decoder.position_embeddings.weight"]

    @property
    def norm_out(self) -> np.ndarray:
        return self.tensors["decoder.norm_out.weight"]


def make_model(shape: DecoderShape = MAGPIE_357M, seed: int = 0) -> SynthModel:
    rng = np.random.default_rng(seed)
    t: dict[str, np.ndarray] = {}

    def normal(mean, std, dims):
        return np.ascontiguousarray(rng.normal(mean, std, size=dims).astype(np.float32))

    t["decoder.position_embeddings.weight"] = normal(0.0, 0.02, (shape.max_positions, shape.width))
    t["decoder.norm_out.weight"] = normal(1.0, 0.01, (shape.width,))
    shapes = _layer_shapes(shape)
    for layer in range(shape.layers):
        for suffix, kind in LAYER_TENSORS:
            name = f"decoder.layers.{layer}.{suffix}"
            if kind == "gain":
                t[name] = normal(1.0, 0.01, shapes[kind])
            else:
                t[name] = normal(0.0, 0.02, shapes[kind])
    for table in range(shape.tables):
        t[f"audio_embeddings.{table}.weight"] = normal(0.0, 0.02, (shape.vocab, shape.width))
        t[f"local_transformer_out_projections.{table}.weight"] = normal(
            0.0, 0.02, (shape.vocab, shape.width))
        t[f"local_transformer_out_projections.{table}.bias"] = normal(0.0, 0.01, (shape.vocab,))
    # Local transformer tensors are drawn last, so a shape with and without them shares every
    # other tensor (names and shapes: src/graph.c:1021-1056).
    if shape.local_layers:
        t["local_transformer.position_embeddings.weight"] = normal(0.0, 0.02, (shape.local_positions, shape.width))
        for layer in range(shape.local_layers):
            for suffix, kind in LOCAL_LAYER_TENSORS:
                name = f"local_transformer.layers.{layer}.{suffix}"
                t[name] = normal(1.0, 0.01, shapes[kind]) if kind == "gain" else normal(0.0, 0.02, shapes[kind])
    return SynthModel(shape=shape, seed=seed, tensors=t)


@dataclass(frozen=True)
class EncoderShape:
    """The text encoder (src/graph.c:709-748: `transformer_stack` over the "encoder" tensors):
    12 heads, FFN 4 x width with a causal convolution of kernel 3, no cross attention."""
    layers: int = 6
    width: int = 768
    heads: int = 12            # fixed in the reference (src/graph.c:735)
    kernel: int = 3            # fixed in the reference (src/graph.c:735)
    vocab: int = 96            # rows of text_embedding.weight (synthetic)
    max_length: int = 256      # rows of encoder.position_embeddings.weight / text_max_length

    @property
    def ffn_width(self) -> int:
        return 4 * self.width


TINY_ENCODER = EncoderShape(layers=2, width=192, vocab=40, max_length=48)


def add_encoder(model: "SynthModel | None", shape: EncoderShape, seed: int) -> dict[str, np.ndarray]:
    """Draws the text encoder's tensors (reference names) and returns them; with a model they
    also go into `model.tensors`, and the width must be the decoder's (the reference shares
    `hidden_dim`)."""
    assert model is None or shape.width == model.shape.width
    rng = np.random.default_rng([seed, 0x656E63])
    t: dict[str, np.ndarray] = {}

    def normal(mean, std, dims):
        return np.ascontiguousarray(rng.normal(mean, std, size=dims).astype(np.float32))

    W, F, K = shape.width, shape.ffn_width, shape.kernel
    t["text_embedding.weight"] = normal(0.0, 0.02, (shape.vocab, W))
    t["encoder.position_embeddings.weight"] = normal(0.0, 0.02, (shape.max_length, W))
    t["encoder.norm_out.weight"] = normal(1.0, 0.01, (W,))
    for layer in range(shape.layers):
        pre = f"encoder.layers.{layer}."
        t[pre + "norm_self.weight"] = normal(1.0, 0.01, (W,))
        t[pre + "norm_pos_ff.weight"] = normal(1.0, 0.01, (W,))
        t[pre + "self_attention.qkv_net.weight"] = normal(0.0, 0.02, (3 * W, W))
        t[pre + "self_attention.o_net.weight"] = normal(0.0, 0.02, (W, W))
        t[pre + "pos_ff.proj.conv.weight"] = normal(0.0, 0.02, (F, W, K))
        t[pre + "pos_ff.o_net.conv.weight"] = normal(0.0, 0.02, (W, F, K))
    if model is not None:
        model.tensors.update(t)
    return t


@dataclass(frozen=True)
class CodecShape:
    """The NanoCodec decoder (src/graph.c:2640-2780): 8 FSQ groups of 4 latent channels, a first
    convolution to `base` channels, five up-sampling stages that halve the channels.  The
    reference hard-codes base = 864; smaller multiples of 32 serve as test shapes."""
    base: int = 864
    rates: tuple = (8, 8, 4, 2, 2)
    kernels: tuple = (3, 7, 11)      # one residual branch per kernel
    dilations: tuple = (1, 3, 5)     # three blocks per branch
    groups: int = 8
    latent: int = 32
    fsq_codes: int = 2016            # 8 * 7 * 6 * 6 indices per group

    @property
    def samples_per_frame(self) -> int:
        return int(np.prod(self.rates))


TINY_CODEC = CodecShape(base=96)


def add_codec(model: "SynthModel | None", shape: CodecShape, seed: int) -> dict[str, np.ndarray]:
    """Draws the codec decoder's tensors under the names decode_codec resolves
    (src/graph.c:2545-2626, 2360-2395).  Convolution weights ~ N(0, 1/fan_in) so activations
    keep unit scale through the 19 convolutions of a stage; Snake alphas ~ N(1, 0.1)."""
    rng = np.random.default_rng([seed, 0x636463])
    t: dict[str, np.ndarray] = {}

    def conv(name, oc, ic, k, fan_in=None):
        std = 1.0 / np.sqrt(fan_in or ic * k)
        t[name + ".weight"] = np.ascontiguousarray(rng.normal(0.0, std, size=(oc, ic, k)).astype(np.float32))
        t[name + ".bias"] = np.ascontiguousarray(rng.normal(0.0, 0.02, size=(oc,)).astype(np.float32))

    def alpha(name, channels):
        t[name + ".activation.snake_act.alpha"] = np.ascontiguousarray(
            rng.normal(1.0, 0.1, size=(channels,)).astype(np.float32))

    conv("audio_decoder.pre_conv.conv", shape.base, shape.latent, 7)
    ch = shape.base
    for s, rate in enumerate(shape.rates):
        alpha(f"audio_decoder.activations.{s}", ch)
        nch = ch // 2
        # transposed convolution weight [in][out per group = 1][kernel]; every output sample
        # sums 2 channels x 2 taps
        conv(f"audio_decoder.up_sample_conv_layers.{s}.conv", ch, 1, 2 * rate, fan_in=4)
        t[f"audio_decoder.up_sample_conv_layers.{s}.conv.bias"] = np.ascontiguousarray(
            rng.normal(0.0, 0.02, size=(nch,)).astype(np.float32))
        for b, k in enumerate(shape.kernels):
            for d in range(len(shape.dilations)):
                pre = f"audio_decoder.res_layers.{s}.res_blocks.{b}.res_blocks.{d}."
                alpha(pre + "input_activation", nch)
                conv(pre + "input_conv.conv", nch, nch, k)
                alpha(pre + "skip_activation", nch)
                # the skip convolution's output joins the residual: keep it small
                conv(pre + "skip_conv.conv", nch, nch, k, fan_in=9 * nch * k)
        ch = nch
    alpha("audio_decoder.post_activation", ch)
    conv("audio_decoder.post_conv.conv", 1, ch, 3)
    if model is not None:
        model.tensors.update(t)
    return t


def make_codec_codes(shape: CodecShape, seed: int, frames: int) -> np.ndarray:
    """FSQ indices [groups, frames] uint32, uniform over the group's code space."""
    rng = np.random.default_rng([seed, 0x667371])
    return np.ascontiguousarray(rng.integers(0, shape.fsq_codes, size=(shape.groups, frames), dtype=np.uint32))


def make_memory(shape: DecoderShape, seed: int) -> np.ndarray:
    """Text-encoder output for one request: [memory_length, width] ~ N(0,1)."""
    rng = np.random.default_rng([seed, 0x6D656D])
    return np.ascontiguousarray(
        rng.normal(0.0, 1.0, size=(shape.memory_length, shape.width)).astype(np.float32))


def make_codes(shape: DecoderShape, seed: int, frames: int = 1) -> np.ndarray:
    """Uniform code ids in [0, codebook_size): [frames, tables] uint32."""
    rng = np.random.default_rng([seed, 0x636F64])
    return np.ascontiguousarray(
        rng.integers(0, shape.codebook_size, size=(frames, shape.tables), dtype=np.uint32))


def make_linear_case(seed: int, n: int = 3072, k: int = 768):
    """The single-op case: x ~ N(0,1) [1,k]; W ~ N(0,0.02) [n,k]; LayerNorm gain
    ~ N(1,0.01); bias ~ N(0,0.01)."""
    rng = np.random.default_rng([seed, 0x6C696E])
    x = rng.normal(0.0, 1.0, size=(1, k)).astype(np.float32)
    w = rng.normal(0.0, 0.02, size=(n, k)).astype(np.float32)
    gain = rng.normal(1.0, 0.01, size=(k,)).astype(np.float32)
    bias = rng.normal(0.0, 0.01, size=(n,)).astype(np.float32)
    return x, w, gain, bias


def write_safetensors(path: str, tensors: dict[str, np.ndarray]) -> None:
    """Minimal safetensors writer (F32 only): 8-byte little-endian header
    length, JSON header, then the raw tensors back to back."""
    header: dict[str, dict] = {}
    offset = 0
    for name, array in tensors.items():
        assert array.dtype == np.float32 and array.flags["C_CONTIGUOUS"]
        header[name] = {"dtype": "F32", "shape": list(array.shape),
                        "data_offsets": [offset, offset + array.nbytes]}
        offset += array.nbytes
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for array in tensors.values():
            f.write(array.tobytes())
