"""Host-side logic that needs no GPU: the synthetic-weight generator, the
safetensors writer, stream partitioning across ranks, and the cross-rank max
the benchmark uses (two gloo ranks on CPU)."""
import json
import os
import struct
import subprocess
import sys
import textwrap

import numpy as np
import pytest

import bench
from mynah_tts_b200 import synth

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_synthetic_model_is_reproducible_and_shaped():
    a = synth.make_model(synth.TINY, seed=3)
    b = synth.make_model(synth.TINY, seed=3)
    c = synth.make_model(synth.TINY, seed=4)
    assert a.tensors.keys() == b.tensors.keys()
    for name in a.tensors:
        assert np.array_equal(a.tensors[name], b.tensors[name])
    assert not np.array_equal(a.position, c.position)
    s = synth.TINY
    assert a.layer(0, "self_attention.qkv_net.weight").shape == (3 * s.width, s.width)
    assert a.layer(1, "pos_ff.proj.conv.weight").shape == (s.ffn_width, s.width, 1)
    assert a.layer(0, "cross_attention.kv_net.weight").shape == (2 * s.xattn_width, s.width)
    assert a.head_weight(s.tables - 1).shape == (s.vocab, s.width)
    full = synth.MAGPIE_357M
    assert (full.layers, full.width, full.heads, full.head_width, full.ffn_width) == (12, 768, 12, 64, 3072)
    codes = synth.make_codes(full, seed=1, frames=4)
    assert codes.shape == (4, 8) and codes.max() < full.codebook_size


def test_safetensors_writer_layout(tmp_path):
    t = {"a.weight": np.arange(6, dtype=np.float32).reshape(2, 3), "b": np.ones(4, np.float32)}
    path = tmp_path / "x.safetensors"
    synth.write_safetensors(str(path), t)
    raw = path.read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n])
    assert header["a.weight"] == {"dtype": "F32", "shape": [2, 3], "data_offsets": [0, 24]}
    assert header["b"]["data_offsets"] == [24, 40]
    body = raw[8 + n:]
    assert np.array_equal(np.frombuffer(body[:24], np.float32), np.arange(6, dtype=np.float32))
    assert len(body) == 40


def test_partition_streams_covers_every_stream_once():
    for total, world in ((8, 1), (64, 2), (64, 8), (256, 4), (7, 4), (3, 8)):
        parts = [bench.partition_streams(total, world, r) for r in range(world)]
        assert sorted(sum(parts, [])) == list(range(total))
        assert max(map(len, parts)) - min(map(len, parts)) <= 1


def test_algorithmic_bytes_match_the_documented_figures():
    shape = synth.MAGPIE_357M
    q = bench.weight_bytes_table(shape, "int8")
    per_layer = q["qkv"] + q["o_self"] + q["q_cross"] + q["o_cross"] + q["ffn_up"] + q["ffn_down"]
    # 7,274,496 weights + 7,808 row scales x 4 bytes per layer
    assert per_layer == 7274496 + 7808 * 4
    # self-attention at batch 1, position 256: K and V rows 0..256 of 768 floats
    b = bench.algorithmic_bytes(shape, "self attention", 1, 256, q)
    assert b >= 2 * 257 * 768 * 4 and b < 2 * 257 * 768 * 4 + 40000
    # 64 streams at position 257, the strict step's launch (f32 rows out, quantized by the next
    # launch): the figure of profiles/traffic.json; with the int8 row, one byte per column more
    split = bench.algorithmic_bytes(shape, "self attention", 64, 257, q, split_quant=True)
    assert split == 64 * (2 * 258 * 3072 + 2 * 3072 + 3 * 3072 + 3072) == 102629376
    assert bench.algorithmic_bytes(shape, "self attention", 64, 257, q) == split + 64 * 768
    # the quantization launches: hidden rows alone, or the mean of hidden and attention rows
    name = "row quantization (attention rows|hidden rows)"
    assert bench.algorithmic_bytes(shape, name, 64, 257, q) == 64 * 3072 * 5
    assert bench.algorithmic_bytes(shape, name, 64, 257, q, split_quant=True) == 64 * (3072 + 768) / 2 * 5


def test_reduce_max_over_two_gloo_ranks(tmp_path):
    script = tmp_path / "rank.py"
    script.write_text(textwrap.dedent(f"""
        import os, sys
        sys.path.insert(0, {ROOT!r})
        import torch.distributed as dist
        import bench
        dist.init_process_group("gloo")
        rank, world = dist.get_rank(), dist.get_world_size()
        mine = bench.partition_streams(9, world, rank)
        got = bench.reduce_max(10.0 + rank, world, device="cpu")
        assert got == 10.0 + world - 1, got
        total = bench.reduce_max(float(len(mine)), world, device="cpu")
        assert total == 5.0
        dist.barrier()
        dist.destroy_process_group()
        print("rank", rank, "ok")
    """))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29571", WORLD_SIZE="2")
    procs = [subprocess.Popen([sys.executable, str(script)], env=dict(env, RANK=str(r), LOCAL_RANK=str(r)),
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = [p.communicate(timeout=180)[0] for p in procs]
    for p, out in zip(procs, outs):
        assert p.returncode == 0, out


def test_reference_arm_prints_one_json_line():
    """`bench.py --impl reference` on a tiny sample: runs the CPU reference (or the
    restatement where it is absent) and prints the contract's line."""
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1",
                          "--warmup", "0", "--streams", "2", "--ref-frames", "2"],
                         capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["unit"] == "frames/s" and line["value"] > 0
    assert line["cpu_baseline"]["kind"] in ("reference", "port")
    assert line["e2e"]["h2d_bytes_per_step"] == 0
