"""Benchmark of the B200 decode path (and, with --impl reference, of the
reference's own CPU implementation of the same path).

Workload (the data-parallel serving configuration): int8 per-row weights,
`--streams` concurrent greedy streams per GPU, `--frames` frames each from an
empty KV cache, on a random-init Magpie-357M-shaped decoder (12 layers, d 768,
12 heads x 64, cross width 128 over 128 text states, FFN 3072, 8 embedding
tables and 8 logit heads over a 2048-entry vocabulary).  One "step" is one such
job: streams x frames frames.  Streams are independent, so with N GPUs every
rank runs its own streams on a full weight copy (weak scaling, no collective on
the data path; NCCL is used only for the barrier and the max over ranks).

    python bench.py --gpus 1 --steps 3 --warmup 3
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...
    python bench.py --impl reference

The timed mode is the strict one (reference summation order, the host libm's
expf/tanhf): the mode whose greedy token streams equal the reference's.  Lane 0
of rank 0 carries the fixture request of tests/golden/golden.npz (seed 21) inside
the timed job, and the line says whether its 512 tokens came out identical
(`token_parity`).  `--mode fast` times the tolerance-parity mode instead; by
default its throughput is reported beside the headline as `fast`.

Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from mynah_tts_b200 import synth  # noqa: E402

FRAME_RATE = 21.533          # audio frames per second of the real model (stacked frames)
SEED = 21


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f)["hbm_gbs"], "measured"
    return 6650.0, "fallback"


def partition_streams(total_streams: int, world: int, rank: int) -> list[int]:
    """Stream i runs on rank i mod world (the reference has no scheduler across
    devices; requests are independent, src/mynah_tts.h:79-91)."""
    return [i for i in range(total_streams) if i % world == rank]


def reduce_max(value: float, world: int, device: str = "cuda") -> float:
    """Max of a per-rank scalar over all ranks (the only cross-rank exchange of
    the benchmark; the data path has none)."""
    if world <= 1:
        return float(value)
    import torch
    import torch.distributed as dist
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def synthetic_cross_kv(shape, stream: int):
    """Cross K/V of one request, [layers][memory_length][xattn_width] each: the
    distribution LayerNorm(memory) @ kv_net^T has for N(0,1) memory and
    N(0,0.02) weights (std 0.02*sqrt(width))."""
    rng = np.random.default_rng([SEED, 0x6B76, stream])
    std = 0.02 * np.sqrt(shape.width)
    dims = (shape.layers, shape.memory_length, shape.xattn_width)
    return (rng.normal(0, std, dims).astype(np.float32), rng.normal(0, std, dims).astype(np.float32))


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device: int):
        self.device = device
        self.lines: list[str] = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "200", "-i", str(self.device)], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None,
                "sm_max_mhz": float(max(mx)) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# --------------------------------------------------------------- reference arm
def cpu_model_name() -> str:
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("model name"):
                    return line.split(":", 1)[1].strip()
    except OSError:
        pass
    return "unknown"


def cpu_reference_job(shape, model, streams: int, frames: int, threads: int | None, start: int = 0):
    """`streams` greedy streams x `frames` frames through the reference's own CPU
    code (oracle/_ref, its default x86 flags) in groups of at most 16 (its batch
    cap, src/graph.c:12), every stream starting with `start` rows already in its KV
    cache (zero rows: the cost of a step depends on how many rows it attends, not on
    what they hold); falls back to the C restatement where the compiled reference is
    absent.  Returns (frames/s, seconds, kind, cores)."""
    from oracle import oracle as O
    cores = threads or os.cpu_count() or 1
    memory = synth.make_memory(shape, seed=SEED + 100)
    codes = synth.make_codes(shape, seed=SEED + 200, frames=1)
    if O.have_ref("fast"):
        rm = O.RefModel(model, O.INT8, "fast", threads=cores)
        groups = [min(16, streams - g) for g in range(0, streams, 16)]
        decs = [[rm.new_decoder(memory, start + frames + 2) for _ in range(n)] for n in groups]
        rm.greedy_decode(decs[0][:1], codes, 1, 10 ** 6)          # packs the weights (first use)
        for group in decs:
            for d in group:
                d.length = start
        t0 = time.perf_counter()
        for group in decs:
            rm.greedy_decode(group, np.repeat(codes, len(group), axis=0), frames, 10 ** 6)
        dt = time.perf_counter() - t0
        for group in decs:
            for d in group:
                d.close()
        rm.close()
        return streams * frames / dt, dt, "reference", cores
    pm = O.PortModel(model, O.INT8)
    ps = [pm.new_stream(memory, start + frames + 2) for _ in range(streams)]
    for s in ps:
        s.length = start
    t0 = time.perf_counter()
    for s in ps:
        s.greedy_decode(codes[0], frames, 10 ** 6)
    dt = time.perf_counter() - t0
    for s in ps:
        s.close()
    pm.close()
    return streams * frames / dt, dt, "port", 1


def reference_sample(args):
    """The bounded sample of the workload the CPU arm times: at most 16 streams (the
    reference's batch cap) x --ref-frames frames centred on the job's mean position."""
    streams = min(args.streams, 16)
    mean_pos = args.start_position + (args.frames - 1) / 2.0
    start = max(0, int(round(mean_pos - (args.ref_frames - 1) / 2.0)))
    return streams, args.ref_frames, start


def one_thread_reference(args) -> dict | None:
    """The same sample on ONE host thread, in a process of its own (the reference sizes its
    thread pool once per process)."""
    cmd = [sys.executable, os.path.abspath(__file__), "--impl", "reference", "--steps", "1", "--warmup", "0",
           "--streams", str(args.streams), "--frames", str(args.frames), "--start-position", str(args.start_position),
           "--ref-frames", str(max(2, args.ref_frames // 4)), "--ref-threads", "1"]
    try:
        out = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
        line = [l for l in out.stdout.splitlines() if l.startswith("{")][-1]
        d = json.loads(line)
        return {"value": d["value"], "unit": "frames/s", "cores": 1, "sample": d["cpu_baseline"]["sample"]}
    except Exception as exc:  # noqa: BLE001 - a missing 1-thread figure must not lose the line
        return {"value": None, "error": str(exc)[:200]}


def local_generate_extra(backend, streams: int, args, cpu: bool = True) -> dict:
    """The sampled generation loop with the local transformer (16 stacked streams, 2 local
    layers): embed -> decoder step -> 16 local positions with top-k draws, per frame, for
    `streams` requests; plus the same loop through the reference's own CPU functions on a
    bounded sample."""
    from mynah_tts_b200.backend import Decoder
    from oracle import oracle as O
    shape = synth.MAGPIE_357M_LOCAL
    model = synth.make_model(shape, seed=SEED + 7)
    frames = 64 if cpu else max(1, min(64, args.frames))
    dec = Decoder(backend, model, capacity=frames + 8, slots=streams, max_batch=streams)
    for slot in range(streams):
        ck, cv = synthetic_cross_kv(shape, slot)
        dec.slot_load(slot, ck, cv)
    start = np.stack([synth.make_codes(shape, seed=SEED + 300 + b, frames=1)[0] for b in range(streams)])
    lanes = [(0.7, 80, 1000 + b, 1) for b in range(streams)]
    ms = 0.0
    for _ in range(3):
        for slot in range(streams):
            dec.slot_set_length(slot, 0)
        _, _, ms, _, _ = dec.generate(list(range(streams)), start, frames, 10 ** 6, lanes)
    out = {"workload": f"{streams} sampled streams x {frames} frames, 16 stacked streams, 2 local layers, "
                       "temperature 0.7, top-k 80", "frames_per_s": streams * frames / (ms / 1000.0),
           "us_per_frame": ms * 1000.0 / frames, "rtf_per_stream": (ms / 1000.0 / frames) * FRAME_RATE}
    dec.close()
    if cpu and O.have_ref("fast"):
        n, cpu_frames = min(streams, 16), 6
        rm = O.RefModel(model, O.INT8, "fast", threads=os.cpu_count() or 1)
        memory = synth.make_memory(shape, seed=SEED + 100)
        decs = [rm.new_decoder(memory, cpu_frames + 3) for _ in range(n)]
        locs = [rm.new_local(80) for _ in range(n)]
        codes = start[:n].copy()
        rng = [1000 + b for b in range(n)]
        t0 = 0.0
        for f in range(cpu_frames + 1):            # frame 0 packs the weights: not timed
            if f == 1:
                t0 = time.perf_counter()
            rows = np.stack([rm.embed_frame(codes[b]) for b in range(n)])
            hidden = rm.step_batch(decs, rows)
            codes, _, _, rng = rm.local_frame(locs, hidden, [0.7] * n, [80] * n, rng, [0] * n)
        dt = time.perf_counter() - t0
        for d in decs:
            d.close()
        for l in locs:
            l.close()
        rm.close()
        out["cpu_reference"] = {"frames_per_s": n * cpu_frames / dt, "cores": os.cpu_count() or 1,
                                "sample": f"{n} streams stepped together x {cpu_frames} frames ({dt:.1f} s)"}
    return out


def frontend_extra(device: int) -> dict:
    """The two ends of a request around the decoder loop: the text encoder (encode_text, 6 layers
    x 768, 128 ids) and the codec decoder (decode_codec at the reference's fixed size, 256 frames =
    11.9 s of audio), both modes, with the CPU code beside them on a bounded sample."""
    import ctypes as C
    from mynah_tts_b200.backend import Backend, Codec, TextEncoder
    out = {}
    eshape = synth.EncoderShape()
    etensors = synth.add_encoder(None, eshape, seed=SEED)
    ids = np.random.default_rng([SEED, 0x696473]).integers(0, eshape.vocab, size=128).astype(np.int32)
    cshape = synth.CodecShape()
    ctensors = synth.add_codec(None, cshape, seed=SEED)
    frames = 256
    codes = synth.make_codec_codes(cshape, SEED, frames)
    flop = 0.0          # multiply-adds of the codec's convolutions per frame, x2
    ch, length = cshape.base, 1
    flop += 2.0 * cshape.base * cshape.latent * 7
    for rate in cshape.rates:
        ch, length = ch // 2, length * rate
        flop += 2.0 * ch * 4 * length + 2.0 * 2 * 3 * sum(cshape.kernels) * ch * ch * length
    flop += 2.0 * ch * 3 * length
    enc = {"ids": 128, "shape": "6 layers x 768, 12 heads, kernel-3 causal convolution feed-forward, f32"}
    cod = {"frames": frames, "audio_s": frames / FRAME_RATE, "gflop_per_frame": flop / 1e9,
           "shape": "base 864, rates 8/8/4/2/2, f32; strict keeps one sequential f32 sum per output sample and "
                    "the host libm's sinf bits (bit-identical samples, SIMT); fast runs the residual-layer "
                    "convolutions on tcgen05 over split f16 planes (samples within 1e-4); a strict decoder may "
                    "be paired with either (the codec's `arithmetic`)"}
    for mode in ("strict", "fast"):
        be = Backend("int8", strict=mode == "strict", device=device)
        te = TextEncoder(be, etensors, eshape)
        te.encode(ids)
        t0 = time.perf_counter()
        for _ in range(3):
            te.encode(ids)
        enc[mode + "_ms"] = (time.perf_counter() - t0) * 1000.0 / 3
        te.close()
        cd = Codec(be, ctensors, cshape, max_frames=frames)
        ms = cd.time(codes, 3)
        t0 = time.perf_counter()
        cd.decode(codes)
        cod[mode] = {"device_ms": ms, "tflops": flop * frames / (ms * 1e-3) / 1e12, "x_realtime": frames / FRAME_RATE / (ms * 1e-3),
                     "host_call_ms": (time.perf_counter() - t0) * 1000.0}
        cd.close(); be.close()
    # CPU beside it: the restatement (pinned bit for bit against the reference) on one core
    from oracle import oracle as O
    t0 = time.perf_counter()
    O.Port.get().encode_text(etensors, eshape, ids[:32])
    enc["cpu_port_ms_32_ids"] = (time.perf_counter() - t0) * 1000.0
    t0 = time.perf_counter()
    O.Port.get().codec_decode(ctensors, cshape, codes[:, :2])
    cod["cpu_port_ms_per_frame"] = (time.perf_counter() - t0) * 1000.0 / 2
    cod["cpu_note"] = "scalar restatement of decode_codec, one core, 2 frames"
    out["text_encoder"] = enc
    out["codec"] = cod
    return out


def ragged_int4_extra(shape, model, device: int, streams: int) -> dict:
    """int4 (group 32) weights, `streams` greedy streams whose lengths are uniform in
    [128, 1024] from the seed; a stream leaves the batch at its length.  Aggregate frames/s
    of the device-resident loop."""
    from mynah_tts_b200.backend import Backend, Decoder
    rng = np.random.default_rng([SEED, 0x726167])
    lengths = [int(x) for x in rng.integers(128, 1025, size=streams)]
    backend = Backend("int4", strict=False, device=device)
    dec = Decoder(backend, model, capacity=max(lengths) + 8, slots=streams, max_batch=streams)
    for slot in range(streams):
        ck, cv = synthetic_cross_kv(shape, slot)
        dec.slot_load(slot, ck, cv)
    start = np.stack([synth.make_codes(shape, seed=SEED + 200 + b, frames=1)[0] for b in range(streams)])
    ms = 0.0
    for _ in range(2):
        for slot in range(streams):
            dec.slot_set_length(slot, 0)
        _, _, ms, _ = dec.greedy(list(range(streams)), start, lengths, min_frames=10 ** 6)
    dec.close()
    backend.close()
    return {"workload": f"int4 group-32 weights, {streams} greedy streams, lengths uniform[128,1024] "
                        f"(sum {sum(lengths)}, max {max(lengths)}), a stream leaves at its length",
            "frames_per_s": sum(lengths) / (ms / 1000.0), "ms": ms,
            "note": "int4 products: tcgen05 tiles while 48 or more lanes are live, the SIMT kernel below"}


def run_reference(args, rank: int):
    if rank != 0:
        return
    shape = synth.MAGPIE_357M
    model = synth.make_model(shape, seed=SEED)
    streams, frames, start = reference_sample(args)
    threads = args.ref_threads or None
    times = []
    kind = cores = None
    for step in range(args.warmup + args.steps):
        _, dt, kind, cores = cpu_reference_job(shape, model, streams, frames, threads, start)
        if step >= args.warmup:
            times.append(dt)
    ms = 1000.0 * float(np.mean(times))
    value = streams * frames / (ms / 1000.0)
    sample = (f"{streams} streams stepped together x {frames} frames per step, positions {start}..{start + frames - 1} "
              f"(centred on the job's mean position; the reference's batch cap is 16), {cores} thread(s), "
              f"{cpu_model_name()}")
    config = workload_config(args, shape)
    config["sampled"] = sample
    print(json.dumps({
        "impl": "reference", "metric": "frames_per_s", "value": value, "unit": "frames/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8",
        "data": "synthetic",
        "config": config,
        "cpu_baseline": {"value": value, "unit": "frames/s", "cores": cores, "kind": kind, "sample": sample,
                         "cpu": cpu_model_name()},
        "e2e": {"value": value, "unit": "frames/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def workload_config(args, shape):
    return {"workload": (f"C5 data-parallel serving: {args.quant} weights, {args.streams} concurrent greedy "
                         f"streams per GPU x {args.frames} frames from "
                         f"{'empty KV' if not args.start_position else str(args.start_position) + ' cached rows'}, Magpie-357M-shaped decoder "
                         f"(12L d768 12x64 heads, xw128 over 128 text states, ffn3072, 8 tables/heads x 2048)"),
            "streams_per_gpu": args.streams, "frames": args.frames, "quant": args.quant,
            "mode": args.mode + (" (reference summation order and host-libm bits: token-identical to the reference)"
                                 if args.mode == "strict" else " (tree reductions, CUDA expf/tanhf: tolerance parity)"),
            "l2": "working set (weights + f32 KV of all streams) exceeds the 126 MB L2",
            "parallelism": f"dp{args.gpus} replicas, no collective"}


# ------------------------------------------------------------------- own arm
def traffic_ratio(name: str):
    """Measured DRAM bytes / algorithmic bytes of one launch of call site `name`, from the ncu
    capture recorded in profiles/traffic.json -- valid only while the kernel's source is the
    one that was captured (the record carries its hash).  Returns (ratio or None, provenance)."""
    import hashlib
    path = os.path.join(ROOT, "profiles", "traffic.json")
    try:
        with open(path) as f:
            rec = json.load(f).get(name)
    except (OSError, ValueError):
        rec = None
    if not rec:
        return None, None
    h = hashlib.sha256()
    for rel in rec["sources"]:
        with open(os.path.join(ROOT, rel), "rb") as f:
            h.update(f.read())
    if h.hexdigest() != rec["sources_sha256"]:
        return None, f"stale: {rec['sources']} changed since the capture at commit {rec['commit']}"
    return rec["ratio"], (f"ncu dram__bytes_read.sum + dram__bytes_write.sum of one launch ({rec['case']}), captured at "
                          f"commit {rec['commit']}, scaled by algorithmic bytes")


def algorithmic_bytes(shape, name: str, batch: int, mean_len: float, qbytes: dict, split_quant: bool = False) -> float:
    """Bytes one launch of a call site must move, each counted once.  split_quant: the self
    attention leaves f32 rows only and a launch of its own quantizes them (strict mode, two or
    more lanes, quantized weights)."""
    W, F, XW, T = shape.width, shape.ffn_width, shape.xattn_width, shape.memory_length
    act = 1 if qbytes["quantized"] else 4

    def product(n, k, wname, out_f32=True):
        return qbytes[wname] + batch * (k * act + 4 + n * 4 * (2 if wname in ("o_self", "o_cross", "ffn_down") else 1))
    if name == "self attention":
        return batch * (2 * (mean_len + 1) * W * 4 + 2 * W * 4 + 3 * W * 4 + W * (4 + (0 if split_quant else act)))
    if name == "cross attention":
        return batch * (2 * T * XW * 4 + XW * 4 + XW * (4 + act))
    if name.startswith("cross block"):
        return batch * (2 * T * XW * 4 + W * (4 + 4 + act)) + qbytes["q_cross"] + qbytes["o_cross"] + 2 * W * 4
    table = {"qkv product": (3 * W, W, "qkv"), "o_self product": (W, W, "o_self"),
             "q_cross product": (XW, W, "q_cross"), "o_cross product": (W, XW, "o_cross"),
             "ffn_up product(+gelu)": (F, W, "ffn_up"), "ffn_down product": (W, F, "ffn_down"),
             "heads product": (shape.tables * shape.vocab, W, "heads")}
    if name in table:
        n, k, wname = table[name]
        return product(n, k, wname)
    if name == "layernorm(+quant)":
        return batch * W * (4 + 4 + act) + W * 4
    if name.startswith("row quantization"):
        # the feed-forward hidden rows, and in strict mode at 2+ lanes the self-attention rows
        # (one launch each per layer: the mean of the two)
        return batch * (F + W) / 2 * (4 + 1) if split_quant else batch * F * (4 + 1)
    return 0.0


def weight_bytes_table(shape, quant: str) -> dict:
    W, F, XW = shape.width, shape.ffn_width, shape.xattn_width

    def wb(n, k):
        if quant == "int8":
            return n * k + n * 4
        if quant == "int4":
            return n * k // 2 + n * (k // 32) * 4
        return n * k * (2 if quant == "f16" else 4)
    return {"qkv": wb(3 * W, W), "o_self": wb(W, W), "q_cross": wb(XW, W), "o_cross": wb(W, XW),
            "ffn_up": wb(F, W), "ffn_down": wb(W, F), "heads": wb(shape.tables * shape.vocab, W) + shape.tables * shape.vocab * 4,
            "quantized": quant in ("int8", "int4")}


def step_bytes(shape, quant: str, batch: int, mean_len: float) -> float:
    """Algorithmic bytes of one whole decoder step for `batch` streams at mean position
    mean_len: every weight once, per stream its self K/V rows, cross K/V and row I/O."""
    q = weight_bytes_table(shape, quant)
    per_layer = q["qkv"] + q["o_self"] + q["q_cross"] + q["o_cross"] + q["ffn_up"] + q["ffn_down"] + 3 * shape.width * 4
    weights = shape.layers * per_layer + q["heads"] + shape.width * 4
    per_stream = shape.layers * (2 * (mean_len + 1) * shape.width * 4 + 2 * shape.width * 4 +
                                 2 * shape.memory_length * shape.xattn_width * 4) + shape.tables * shape.width * 4
    return weights + batch * per_stream


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--mode", default="strict", choices=["strict", "fast"],
                    help="strict: reference summation order and host-libm bits (token-identical); "
                         "fast: tree reductions and CUDA expf/tanhf (tolerance parity)")
    ap.add_argument("--streams", type=int, default=64, help="concurrent streams per GPU")
    ap.add_argument("--total-streams", type=int, default=0,
                    help="strong scaling headline: this many streams in all, dealt round-robin to the ranks")
    ap.add_argument("--frames", type=int, default=512)
    ap.add_argument("--quant", default="int8", choices=["int8", "int4", "f16", "f32"])
    ap.add_argument("--ref-frames", type=int, default=24, help="frames per step of the CPU reference arm")
    ap.add_argument("--ref-threads", type=int, default=0, help="host threads of the CPU reference arm (0: all)")
    ap.add_argument("--cpu-frames", type=int, default=24, help="frames of the CPU baseline sample")
    ap.add_argument("--no-extras", action="store_true", help="only the headline job (no other mode, batch-1, "
                    "matrix-pool, partition sweep, f32 step, sampled loop, ragged int4, CPU baseline)")
    ap.add_argument("--only", default="", choices=["", "gemv_pool", "batch1", "frontend", "codec", "generate"],
                    help="profiling aid: run only this small case (a few launches, no JSON contract)")
    ap.add_argument("--start-position", type=int, default=0,
                    help="profiling aid: every job starts with this many (zero) rows already in each "
                         "stream's KV cache, so a few frames exercise long-context launches")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, rank)
        return

    import torch
    import torch.distributed as dist
    from mynah_tts_b200.backend import Backend, Decoder, MatrixPool

    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    shape = synth.MAGPIE_357M
    model = synth.make_model(shape, seed=SEED)
    frames = args.frames
    strict = args.mode == "strict"
    peak, peak_kind = load_peaks()

    def gemv_pool_case(backend):
        """The single [3072,768] op (LayerNorm + quantization + product) streamed over 512
        distinct matrices (1.2 GB > L2) per pass."""
        x, w, gain, bias = synth.make_linear_case(seed=1)
        groups = 512
        pool = MatrixPool(backend, w, groups, bias=bias, gain=gain)
        xs = np.repeat(x, groups, axis=0)
        dx = backend.to_device(xs)
        dy = backend.dev_alloc(groups * w.shape[0])
        for _ in range(3):
            pool.linear(dx, dy)
        backend.timer_start()
        passes = 10
        for _ in range(passes):
            pool.linear(dx, dy)
        pool_ms = backend.timer_stop() / passes
        gbs = pool.bytes_per_pass / (pool_ms / 1000.0) / 1e9
        out = {"matrix": "[3072,768] " + args.quant, "matrices_per_pass": groups,
               "bytes_per_pass": pool.bytes_per_pass, "ms_per_pass": pool_ms,
               "gbs": gbs, "frac_of_measured_hbm": gbs / peak, "frac_of_8tbs": gbs / 8000.0,
               "note": "LayerNorm+quant launch plus product launch per pass; cold (pool > L2)"}
        pool.close(); dx.free(); dy.free()
        return out

    if args.only == "frontend":
        print(json.dumps({"frontend": frontend_extra(local_rank)}))
        return
    if args.only == "generate":       # profiling aid: the sampled loop with the local transformer, --frames frames
        gbe = Backend(args.quant, strict=strict, device=local_rank)
        print(json.dumps({"generate": local_generate_extra(gbe, args.streams, args, cpu=False)}))
        gbe.close()
        return
    if args.only == "codec":          # profiling aid: one small decode (64 frames) in the chosen mode
        from mynah_tts_b200.backend import Codec
        cshape = synth.CodecShape()
        cbe = Backend("f32", strict=strict, device=local_rank)
        cd = Codec(cbe, synth.add_codec(None, cshape, seed=SEED), cshape, max_frames=64)
        samples = cd.decode(synth.make_codec_codes(cshape, SEED, 64))
        print(json.dumps({"codec": {"frames": 64, "samples": int(samples.size), "rms": float(samples.std())}}))
        cd.close(); cbe.close()
        return
    if args.only == "gemv_pool":
        backend = Backend(args.quant, strict=strict, device=local_rank)
        print(json.dumps({"gemv_pool": gemv_pool_case(backend)}))
        backend.close()
        return

    def make_decoder(backend, stream_ids, capacity, golden_lane=False):
        """A decoder holding one slot per stream of this rank; the cross K/V are synthetic except
        for the fixture request, whose cross K/V are made on the device from its text memory."""
        n = max(len(stream_ids), 1)
        dec = Decoder(backend, model, capacity=capacity, slots=n, max_batch=n)
        for slot, gid in enumerate(stream_ids):
            if golden_lane and gid == 0:
                dec.slot_prefill(slot, synth.make_memory(shape, seed=SEED + 100))
            else:
                ck, cv = synthetic_cross_kv(shape, gid)
                dec.slot_load(slot, ck, cv)
        return dec

    def start_codes_of(stream_ids):
        return np.stack([synth.make_codes(shape, seed=SEED + 200 + gid, frames=1)[0] for gid in stream_ids]) \
            if stream_ids else np.zeros((0, shape.tables), np.uint32)

    def timed_jobs(dec, slots, codes, n_frames, repeats, warmups, start=0):
        """Device time (CUDA events inside the library) of `repeats` jobs after `warmups`."""
        total = 0.0
        toks = None
        for it in range(warmups + repeats):
            for sl in slots:
                dec.slot_set_length(sl, start)
            if slots:
                toks, _, ms, _ = dec.greedy(slots, codes, n_frames, min_frames=10 ** 6)
                if it >= warmups:
                    total += ms
        return total, toks

    if args.total_streams:
        # strong scaling: a fixed set of streams dealt round-robin to the ranks
        my_streams = partition_streams(args.total_streams, world, rank)
        scaling, total_streams = "strong", args.total_streams
    else:
        my_streams = [rank * args.streams + i for i in range(args.streams)]
        scaling, total_streams = "weak", world * args.streams
    B = len(my_streams)
    backend = Backend(args.quant, strict=strict, device=local_rank)
    golden_ok = strict and args.quant in ("int8", "int4", "f32") and frames == 512 and args.start_position == 0
    dec = make_decoder(backend, my_streams, args.start_position + frames + 8, golden_lane=golden_ok)
    slots = list(range(B))
    start_codes = start_codes_of(my_streams)

    if args.only == "batch1":
        ms, _ = timed_jobs(dec, [0], start_codes[:1], frames, 1, 1, args.start_position)
        print(json.dumps({"batch1": {"us_per_frame": ms * 1000.0 / frames, "mode": args.mode}}))
        dec.close(); backend.close()
        return

    def reset():
        for s in slots:
            dec.slot_set_length(s, args.start_position)

    # ---- device-resident arm: `value` -------------------------------------------
    for _ in range(args.warmup):
        reset()
        dec.greedy(slots, start_codes, frames, min_frames=10 ** 6)
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches0 = backend.launch_count
    total_ms = 0.0
    tokens = None
    for _ in range(args.steps):
        reset()
        tokens, _, ms, _ = dec.greedy(slots, start_codes, frames, min_frames=10 ** 6)
        total_ms += ms                       # CUDA events on the launching stream, inside the library
    barrier()
    gpu_launches = backend.launch_count - launches0
    clocks = sampler.stop() if rank == 0 else None
    ms_per_step = reduce_max(total_ms, world) / args.steps
    value = total_streams * frames / (ms_per_step / 1000.0)

    # ---- host-buffer arm: `e2e` (one C-ABI call per frame, host codes in, host tokens out)
    pinned_codes = torch.empty((B, shape.tables), dtype=torch.int32).pin_memory().numpy().view(np.uint32)
    pinned_tokens = torch.empty((B, shape.tables), dtype=torch.int32).pin_memory().numpy().view(np.uint32)
    allow = [0] * B

    frame_step = dec.bind_frame_batch(slots, pinned_codes, allow, pinned_tokens)

    def e2e_job():
        reset()
        pinned_codes[:] = start_codes
        for _ in range(frames):
            frame_step()                          # mynah_b200_decoder_frame_batch on the two host buffers
            pinned_codes[:] = pinned_tokens       # EOS is not allowed here, so every pick is a code
        return pinned_tokens
    for _ in range(min(args.warmup, 1) or 1):
        e2e_job()
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        e2e_job()
    barrier()
    e2e_s = reduce_max(time.perf_counter() - t0, world)
    e2e_value = total_streams * frames * args.steps / e2e_s
    # per frame the call copies one staging block in (slots, positions, EOS rule, EOS flags:
    # 4 ints per lane of the decoder's batch capacity; 4 ints of lane count and frame index;
    # the codes) and one block out (4 ints of status, the tokens)
    h2d = frames * (4 * B * 4 + 16 + B * shape.tables * 4)
    d2h = frames * (16 + B * shape.tables * 4)

    # ---- the partition sweep: 8, 64 and 256 streams in all, dealt over the ranks -----------
    # (every rank takes part: the time of a total is the max over ranks)
    strong = None
    if not args.no_extras and not args.total_streams and args.start_position == 0:
        strong = {}
        for total in (8, 64, 256):
            mine = partition_streams(total, world, rank)
            if total == args.streams and world == 1:
                job_ms = ms_per_step                      # the headline job itself
            else:
                sdec = make_decoder(backend, mine, frames + 8) if mine else None
                ms_rank, _ = timed_jobs(sdec, list(range(len(mine))), start_codes_of(mine), frames, 1, 1) if mine else (0.0, None)
                if sdec is not None:
                    sdec.close()
                barrier()
                job_ms = reduce_max(ms_rank, world)
            strong[str(total)] = {"streams_per_gpu": [len(partition_streams(total, world, r)) for r in range(world)],
                                  "frames_per_s": total * frames / (job_ms / 1000.0), "ms_per_job": job_ms,
                                  "rtf_per_stream": (job_ms / 1000.0 / frames) * FRAME_RATE}

    result = None
    if rank == 0:
        # ---- per-call-site device times over one more job -> roofline of the dominant kernel
        reset()
        dec.profile(True)
        dec.greedy(slots, start_codes, frames, min_frames=10 ** 6)
        prof = dec.profile_read()
        dec.profile(False)
        total = sum(v[1] for v in prof.values()) or 1.0
        name, (n_launch, t_ms) = max(prof.items(), key=lambda kv: kv[1][1])
        qbytes = weight_bytes_table(shape, args.quant)
        mean_len = args.start_position + (frames - 1) / 2.0
        split_quant = (args.mode == "strict" and B >= 2 and qbytes["quantized"] and
                       os.environ.get("MYNAH_B200_NO_SPLIT_QUANT", "0") in ("", "0"))
        bytes_per_launch = algorithmic_bytes(shape, name, B, mean_len, qbytes, split_quant)
        avg_s = t_ms / 1000.0 / max(n_launch, 1)
        achieved = bytes_per_launch / avg_s / 1e9
        ratio, provenance = traffic_ratio(name)
        roofline = {"bound": "hbm", "kernel": name, "achieved": achieved, "peak": peak, "unit": "GB/s",
                    "frac": achieved / peak, "of": peak_kind,
                    "traffic": bytes_per_launch * ratio if ratio is not None else None,
                    "traffic_source": provenance,
                    "bytes_per_launch": bytes_per_launch, "avg_launch_us": avg_s * 1e6,
                    "share_of_step": t_ms / total,
                    "timing": "CUDA events around each launch, eager replay of one job"}
        shares = {k: {"launches": v[0], "ms": round(v[1], 3), "share": round(v[1] / total, 4)}
                  for k, v in prof.items() if v[0]}
        # the whole step against HBM: algorithmic bytes of a step at the job's mean position
        step_b = step_bytes(shape, args.quant, B, mean_len)
        step_us = ms_per_step * 1000.0 / frames
        step_roof = {"bytes_per_step": step_b, "us_per_step": step_us, "gbs": step_b / (step_us * 1e-6) / 1e9,
                     "frac_of_measured_hbm": step_b / (step_us * 1e-6) / 1e9 / peak}
        token_parity = None
        if golden_ok and my_streams and my_streams[0] == 0:
            gold = os.path.join(ROOT, "tests", "golden", "golden.npz")
            key = f"full_{args.quant}_s{SEED}_tokens"
            with np.load(gold) as g:
                if key in g:
                    want = g[key].astype(np.uint32)
                    got = np.asarray(tokens)[:, 0]
                    bad = np.nonzero((got != want).any(axis=-1))[0]
                    token_parity = {"lane": 0, "frames": int(frames), "fixture": f"tests/golden/golden.npz:{key}",
                                    "identical_to_reference": bool(len(bad) == 0),
                                    "first_divergence": int(bad[0]) if len(bad) else -1,
                                    "where": "inside the timed job"}
        extras = {}
        if not args.no_extras:
            # batch-1 decode (weights stay L2-resident between steps: labelled so)
            ms1, _ = timed_jobs(dec, [0], start_codes[:1], frames, 1, 1, args.start_position)
            b1_bytes = step_bytes(shape, args.quant, 1, mean_len)
            extras["batch1"] = {"frames_per_s": frames / (ms1 / 1000.0), "us_per_frame": ms1 * 1000.0 / frames,
                                "rtf": (ms1 / 1000.0 / frames) * FRAME_RATE, "mode": args.mode,
                                "frac_of_measured_hbm": b1_bytes / (ms1 * 1e-3 / frames) / 1e9 / peak,
                                "note": "weights L2-resident"}
            # the other mode on the same jobs
            other = "fast" if strict else "strict"
            obe = Backend(args.quant, strict=not strict, device=local_rank)
            odec = make_decoder(obe, my_streams, args.start_position + frames + 8)
            oms, _ = timed_jobs(odec, slots, start_codes, frames, max(1, min(args.steps, 3)), 1, args.start_position)
            oms /= max(1, min(args.steps, 3))
            oms1, _ = timed_jobs(odec, [0], start_codes[:1], frames, 1, 1, args.start_position)
            extras[other] = {"frames_per_s": B * frames / (oms / 1000.0), "ms_per_step": oms,
                             "batch1_us_per_frame": oms1 * 1000.0 / frames,
                             "ratio_to_headline": (B * frames / (oms / 1000.0)) / (value / world),
                             "parity": ("tolerance (hidden rows within 1e-3 f32/f16, 2e-2 int8/int4; picks may part at "
                                        "narrow margins)" if other == "fast" else "token-identical to the reference")}
            odec.close(); obe.close()
            extras["gemv_pool"] = gemv_pool_case(backend)
            # one f32 decoder step at position 256, batch 1 (BASELINE config 2), in both modes:
            # strict f32 products keep the reference's sequential sum (one thread per output)
            fbytes = step_bytes(shape, "f32", 1, 256 + 15.5)
            f32 = {"bytes_per_step": fbytes,
                   "note": "f32 weights (349 MB) exceed L2: every step streams them from HBM; 32 steps from "
                           "position 256, batch 1"}
            for fmode in ("fast", "strict"):
                fbe = Backend("f32", strict=fmode == "strict", device=local_rank)
                fdec = make_decoder(fbe, [0], 256 + 40)
                fms, _ = timed_jobs(fdec, [0], start_codes_of([0]), 32, 1, 1, 256)
                f32[fmode] = {"us_per_step": fms * 1000.0 / 32, "gbs": fbytes / (fms * 1e-3 / 32) / 1e9,
                              "frac_of_measured_hbm": fbytes / (fms * 1e-3 / 32) / 1e9 / peak}
                fdec.close(); fbe.close()
            extras["f32_step_position_256"] = f32
            # the context prefill (decoder_run with count > 1): 217 rows of one request at once,
            # the real model's context length (src/graph.c:2786-2787); a quantized model
            # multiplies them with its f32 weights, as the reference does
            pre = {"rows": 217, "note": "217 rows pushed through the stack together (f32 weights for more than 16 "
                                        "rows, as in the reference); strict keeps sequential f32 sums"}
            prows = np.random.default_rng([SEED, 0x707265]).normal(0, 0.05, size=(217, shape.width)).astype(np.float32)
            for pmode in ("fast", "strict"):
                pbe = Backend(args.quant, strict=pmode == "strict", device=local_rank)
                pdec = Decoder(pbe, model, capacity=256, slots=1, max_batch=217, keep_f32_weights=True)
                ck, cv = synthetic_cross_kv(shape, 0)
                pdec.slot_load(0, ck, cv)
                pdec.prefill(0, prows)
                pdec.slot_set_length(0, 0)
                t0 = time.perf_counter()
                pdec.prefill(0, prows)
                pre[pmode + "_ms"] = (time.perf_counter() - t0) * 1000.0
                pdec.close(); pbe.close()
            extras["prefill"] = pre
            extras["generate"] = local_generate_extra(backend, B, args)
            extras["ragged_int4"] = ragged_int4_extra(shape, model, local_rank, B)
            extras["frontend"] = frontend_extra(local_rank)
        cpu = None
        if world == 1 and not args.no_extras:
            n_cpu, f_cpu, start_cpu = reference_sample(args)
            f_cpu = args.cpu_frames
            v, dt, kind, cores = cpu_reference_job(shape, model, n_cpu, f_cpu, None, start_cpu)
            cpu = {"value": v, "unit": "frames/s", "cores": cores, "kind": kind, "cpu": cpu_model_name(),
                   "sample": f"{n_cpu} streams stepped together x {f_cpu} frames, positions {start_cpu}..{start_cpu + f_cpu - 1} "
                             f"({dt:.1f} s; the reference's batch cap is 16)",
                   "one_thread": one_thread_reference(args)}
        result = {
            "metric": "frames_per_s", "value": value, "unit": "frames/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": scaling, "vs_baseline": None,
            "dtype": "int8 weights x int8 activations, int32 accumulate, f32 glue" if args.quant == "int8" else args.quant,
            "data": "synthetic", "config": workload_config(args, shape),
            "rtf_per_stream": (ms_per_step / 1000.0 / frames) * FRAME_RATE,
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "frames/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "call": "mynah_b200_decoder_frame_batch per frame, pinned host codes in / tokens out"},
            "gpu_launches": int(gpu_launches),
            "roofline": roofline, "step_vs_hbm": step_roof, "call_sites": shares, "cpu_baseline": cpu,
            "token_parity": token_parity,
            "tokens_checksum": int(np.asarray(tokens, np.uint64).sum()),
        }
        if strong is not None:
            result["strong"] = strong
        result.update(extras)
    dec.close()
    backend.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(result))


if __name__ == "__main__":
    main()
