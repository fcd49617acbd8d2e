#!/usr/bin/env python
"""Benchmark of the hot path: decode-shaped int8 quantized dense on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--m 16] [--impl reference]

Workload (the third benchmark configuration): x bf16 [M, 4096], W int8 [4096, 14336], group-128
float32 scales along K, SiLU, output bf16.  One *step* runs the projection for LAYERS distinct,
independent weight matrices (LAYERS x 58.7 MB > the 126 MB L2, so the weights stream from HBM) as ONE
grouped launch: the digit kernel for all activations, then one persistent kernel over the column
tiles of all layers.  With N GPUs every projection is sharded along its output columns (each rank
holds columns [r*N/g, (r+1)*N/g) of every layer; x is replicated) and the kernel stores its slices
straight into every rank's result buffers over NVLink (or one NCCL all-gather per step).

Prints ONE JSON line (rank 0).  `value` = algorithmic bytes of the whole job per second with inputs
resident in HBM; `e2e` = the same metric through the Backend / Executable interface (the calls a cgo
shim binds): every step uploads its activations with BufferFromFlatData, runs Executable.Execute and
reads every result with Buffer.ToFlatData, all inside the timed region (weights stay resident as
parameter buffers, as model variables do).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

K_DIM, N_DIM, GROUP = 4096, 14336, 128
LAYERS = 8
METRIC = "int8 quantized-dense GB/s & TFLOP/s vs roofline (1/2/4/8 B200) vs gobackend AVX"
FALLBACK_HBM_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum of one grouped launch (8 layers) from the ncu capture summarised under
# profiles/ (qdense_decode_tc_group_config3_M16); None where no capture of that batch size exists.
NCU_TRAFFIC_BYTES = {16: 480_726_016}


def algorithmic_bytes(M: int, n_cols: int) -> int:
    """int8 W + f32 group scales + bf16 x + bf16 out for one layer over n_cols columns."""
    return K_DIM * n_cols + 4 * (K_DIM // GROUP) * n_cols + 2 * M * K_DIM + 2 * M * n_cols


def bf16_bits(a: np.ndarray) -> np.ndarray:
    """float32 -> bfloat16 bit patterns, round to nearest even (finite inputs)."""
    b = np.ascontiguousarray(a, np.float32).view(np.uint32)
    return ((b + 0x7FFF + ((b >> 16) & 1)) >> 16).astype(np.uint16)


def bf16_floats(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << 16).view(np.float32)


def measured_peak(key="hbm_gbs", fallback=FALLBACK_HBM_GBS):
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)[key]), "measured"
    except Exception:
        return fallback, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100", "-i", str(self.gpu)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                self.proc.kill()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                smax.append(float(r[2]))
                for name, val in zip(names, r[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            except Exception:
                pass
        # the busiest samples are the ones taken under load
        under = sorted(sm)[len(sm) // 2:] if sm else []
        return {"sm_mhz": statistics.median(under) if under else None,
                "sm_max_mhz": max(smax) if smax else None, "reasons": sorted(reasons), "samples": len(sm)}


def make_layer(seed: int, cols: slice):
    """Seeded synthetic weights of one layer, restricted to this rank's columns."""
    rng = np.random.default_rng(seed)
    w = rng.integers(-127, 128, size=(K_DIM, N_DIM), dtype=np.int8)
    s = rng.uniform(0.001, 0.02, size=(K_DIM // GROUP, N_DIM)).astype(np.float32)
    return np.ascontiguousarray(w[:, cols]), np.ascontiguousarray(s[:, cols])


def host_threads() -> int:
    """All host cores this process may use (torchrun sets OMP_NUM_THREADS=1, which the CPU arm must not inherit)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


# --------------------------------------------------------------------------- other kernels of the path
def time_plan(dv, dev, stream, plan, ins, outs, reps, warm=3):
    ws = plan.new_workspace()
    e0, e1 = dv.Event(dev), dv.Event(dev)
    for it in range(reps + warm):
        if it == warm:
            e0.record(stream)
        plan.launch(ins, outs, ws.ptr if ws else None, stream)
    e1.record(stream)
    stream.sync()
    plan.check_status(ws.ptr if ws else None)
    return e0.elapsed_ms(e1) * 1e3 / reps


def other_kernels(dv, dev, stream):
    """The other rows of the path, timed alone (CUDA events, inputs resident): DotGeneral 4096^3 bf16 / f32 and the
    batched variant (second configuration), prefill quantized dense, causal SDPA (fourth configuration), fused row ops."""
    tpeak, _ = measured_peak("bf16_tflops", 1590.0)
    hpeak, _ = measured_peak()
    rng = np.random.default_rng(3)

    def rand_bf16(n):
        return dv.DeviceMem.from_numpy(bf16_bits(rng.standard_normal(n, dtype=np.float32) * 0.05), dev)

    res = {}
    n = 4096
    a, b, c = rand_bf16(n * n), rand_bf16(n * n), dv.DeviceMem(n * n * 2, dev)
    plan = dv.Plan.dot(1, n, n, n, dv.BF16, dev=dev)
    us = time_plan(dv, dev, stream, plan, [a.ptr, b.ptr], [c.ptr], 20)
    tf = 2.0 * n ** 3 / us / 1e6
    res["dot_general_4096_bf16"] = {"kernel": plan.kernel_name, "us": us, "TFLOP/s": tf, "frac_of_measured_bf16_peak": tf / tpeak}
    for m in (a, b, c):
        m.free()
    af = dv.DeviceMem.from_numpy(rng.standard_normal(n * n, dtype=np.float32) * 0.05, dev)
    bf = dv.DeviceMem.from_numpy(rng.standard_normal(n * n, dtype=np.float32) * 0.05, dev)
    cf = dv.DeviceMem(n * n * 4, dev)
    plan = dv.Plan.dot(1, n, n, n, dv.F32, dev=dev)
    us = time_plan(dv, dev, stream, plan, [af.ptr, bf.ptr], [cf.ptr], 10)
    res["dot_general_4096_f32"] = {"kernel": plan.kernel_name, "us": us, "TFLOP/s": 2.0 * n ** 3 / us / 1e6,
                                   "note": "float32 result from bf16 plane products; includes the split launches"}
    for m in (af, bf, cf):
        m.free()
    a, b, c = rand_bf16(32 * 512 * 128), rand_bf16(32 * 128 * 512), dv.DeviceMem(32 * 512 * 512 * 2, dev)
    plan = dv.Plan.dot(32, 512, 512, 128, dv.BF16, dev=dev)
    us = time_plan(dv, dev, stream, plan, [a.ptr, b.ptr], [c.ptr], 50)
    gbs = (2 * 32 * 512 * 128 * 2 + 32 * 512 * 512 * 2) / us / 1e3
    res["dot_general_batched_32x512x128x512_bf16"] = {"kernel": plan.kernel_name, "us": us, "GB/s": gbs, "frac_of_measured_hbm": gbs / hpeak}
    for m in (a, b, c):
        m.free()
    Mp = 2048
    x = rand_bf16(Mp * K_DIM)
    w = dv.DeviceMem.from_numpy(rng.integers(-127, 128, size=K_DIM * N_DIM, dtype=np.int8), dev)
    sc = dv.DeviceMem.from_numpy(rng.uniform(0.001, 0.02, size=N_DIM).astype(np.float32), dev)
    y = dv.DeviceMem(Mp * N_DIM * 2, dev)
    plan = dv.Plan.qdense(Mp, K_DIM, N_DIM, dv.BF16, dv.I8, dv.SCALE_CHANNEL, 0, False, False, dv.ACT_SILU, dev=dev)
    us = time_plan(dv, dev, stream, plan, [x.ptr, w.ptr, sc.ptr], [y.ptr], 10)
    tf = 2.0 * Mp * K_DIM * N_DIM / us / 1e6
    res["quantized_dense_prefill_2048x4096x14336_bf16"] = {"kernel": plan.kernel_name, "us": us, "TFLOP/s": tf,
                                                          "frac_of_measured_bf16_peak": tf / tpeak,
                                                          "note": "includes expanding the int8 weights to bf16"}
    for m in (x, w, sc, y):
        m.free()
    res["sdpa_causal_b8_h32_8_s2048_d128_bf16"] = sdpa_leg(dv, dev, stream, 32, 8, tpeak)
    # float32 attention with head_dim 64 (an encoder layer of a sentence-embedding model): the tiled CUDA-core kernel
    Be, He, Se, De = 32, 12, 128, 64
    qe, ke, ve = (dv.DeviceMem.from_numpy(rng.standard_normal(Be * He * Se * De, dtype=np.float32), dev) for _ in range(3))
    oe = dv.DeviceMem(Be * He * Se * De * 4, dev)
    plan = dv.Plan.sdpa(Be, He, He, Se, Se, De, dv.F32, dev=dev)
    us = time_plan(dv, dev, stream, plan, [qe.ptr, ke.ptr, ve.ptr], [oe.ptr], 20)
    res["sdpa_f32_b32_h12_s128_d64"] = {"kernel": plan.kernel_name, "us": us, "TFLOP/s": 4.0 * Be * He * Se * Se * De / us / 1e6}
    for m in (qe, ke, ve, oe):
        m.free()
    rows, L = 65536, 4096
    xf = dv.DeviceMem.from_numpy(rng.standard_normal(rows * L, dtype=np.float32), dev)
    gf = dv.DeviceMem.from_numpy(rng.standard_normal(L, dtype=np.float32), dev)
    yf = dv.DeviceMem(rows * L * 4, dev)
    for name, plan, ins in (("fused_softmax_65536x4096_f32", dv.Plan.softmax(dv.F32, rows, L, 1, dev=dev), [xf.ptr]),
                            ("fused_layer_norm_65536x4096_f32", dv.Plan.layernorm(dv.F32, rows, L, 1e-5, True, True, dev=dev), [xf.ptr, gf.ptr, gf.ptr]),
                            ("fused_gelu_268M_f32", dv.Plan.gelu(dv.F32, rows * L, True, dev=dev), [xf.ptr]),
                            ("rms_norm_65536x4096_f32", dv.Plan.rms_norm(dv.F32, rows, L, 1e-5, True, dev=dev), [xf.ptr, gf.ptr])):
        us = time_plan(dv, dev, stream, plan, ins, [yf.ptr], 10)
        gbs = 2.0 * rows * L * 4 / us / 1e3
        res[name] = {"kernel": plan.kernel_name, "us": us, "GB/s": gbs, "frac_of_measured_hbm": gbs / hpeak}
    for m in (xf, gf, yf):
        m.free()
    return res


def weight_format_legs(dv, dev, stream):
    """The same 4096 x 14336 projection with the other weight formats of the op (GGML blocks, packed NF4 / Int4 with the
    reference's [K, N/64] scales), float32 activations as the reference takes them: decode at M = 1 and 16 over eight
    copies of the weights used in turn (more bytes than the L2 holds between two uses of a copy), and 2048 rows at once.
    Random block bytes with a finite half-precision scale in every block."""
    hpeak, _ = measured_peak()
    rng = np.random.default_rng(17)
    K, N, copies = K_DIM, N_DIM, 8
    res = {}

    def timed(plan, x, ws_list, extra, y, reps):
        ws = plan.new_workspace()
        e0, e1 = dv.Event(dev), dv.Event(dev)
        for it in range(reps + 2):
            if it == 2:
                e0.record(stream)
            for w in ws_list:
                plan.launch([x.ptr, w.ptr] + extra, [y.ptr], ws.ptr if ws else None, stream)
        e1.record(stream)
        stream.sync()
        plan.check_status(ws.ptr if ws else None)
        if ws:
            ws.free()
        return e0.elapsed_ms(e1) * 1e3 / (reps * len(ws_list))

    xs = {M: dv.DeviceMem.from_numpy(rng.standard_normal((M, K)).astype(np.float32), dev) for M in (1, 16, 2048)}
    y = dv.DeviceMem(2048 * N * 4, dev)
    formats = (("q4_0", dv.GGML_Q4_0, 32, 18, (0,)), ("q8_0", dv.GGML_Q8_0, 32, 34, (0,)), ("iq4_nl", dv.GGML_IQ4_NL, 32, 18, (0,)),
               ("q4_k", dv.GGML_Q4_K, 256, 144, (0, 2)), ("q6_k", dv.GGML_Q6_K, 256, 210, (208,)))
    for name, gt, values, bb, scale_at in formats:
        blocks = rng.integers(0, 256, size=(N, K // values, bb), dtype=np.uint8)
        for o in scale_at:
            blocks[:, :, o:o + 2] = np.frombuffer(np.float16(0.03125).tobytes(), np.uint8)
        wbufs = [dv.DeviceMem.from_numpy(blocks.reshape(N, -1), dev) for _ in range(copies)]
        leg = {"weight_bytes": int(blocks.nbytes)}
        for M in (1, 16, 2048):
            plan = dv.Plan.qdense(M, K, N, dv.F32, dv.U8, scheme=dv.QUANT_GGML, ggml_type=gt, dev=dev)
            us = timed(plan, xs[M], wbufs if M <= 16 else wbufs[:1], [], y, 5)
            leg[f"M{M}"] = {"kernel": plan.kernel_name, "us": us}
            if M <= 16:
                leg[f"M{M}"]["frac_of_measured_hbm"] = blocks.nbytes / us / 1e3 / hpeak
            else:
                leg[f"M{M}"]["TFLOP/s"] = 2.0 * M * K * N / us / 1e6
        res["ggml_" + name] = leg
        for w in wbufs:
            w.free()
    nblk = N // 64
    sc = dv.DeviceMem.from_numpy(rng.uniform(0.001, 0.02, size=K * nblk).astype(np.float32), dev)
    wbufs = [dv.DeviceMem.from_numpy(rng.integers(0, 256, size=K * N // 2, dtype=np.uint8), dev) for _ in range(copies)]
    for name, scheme, wd in (("nf4_packed", dv.QUANT_NF4, dv.U4), ("int4_packed", dv.QUANT_LINEAR, dv.I4)):
        leg = {"weight_and_scale_bytes": K * N // 2 + K * nblk * 4}
        for M in (1, 16, 2048):
            plan = dv.Plan.qdense(M, K, N, dv.F32, wd, dv.SCALE_REF, 64, scheme=scheme, dev=dev)
            us = timed(plan, xs[M], wbufs if M <= 16 else wbufs[:1], [sc.ptr], y, 5)
            leg[f"M{M}"] = {"kernel": plan.kernel_name, "us": us}
            if M <= 16:
                leg[f"M{M}"]["frac_of_measured_hbm"] = leg["weight_and_scale_bytes"] / us / 1e3 / hpeak
            else:
                leg[f"M{M}"]["TFLOP/s"] = 2.0 * M * K * N / us / 1e6
        res[name] = leg
    for m in [sc, y] + wbufs + list(xs.values()):
        m.free()
    return res


def block_projection_legs(dv, dev, stream):
    """The four projection launches of the fifth configuration's decoder block on their own, one projection per launch in
    a chain of launches (16 rows of bfloat16 x, int8 weights, per-channel scales), over distinct copies of the weights used
    in turn (more bytes than the L2 holds between two uses of a copy).  The first three have few column tiles: their
    tiles are shared by clusters of CTAs."""
    hpeak, _ = measured_peak()
    rng = np.random.default_rng(23)
    res = {}
    for name, K, N, copies in (("o_4096x4096", 4096, 4096, 10), ("qkv_4096x6144", 4096, 6144, 8), ("down_14336x4096", 14336, 4096, 4),
                               ("gate_up_4096x28672", 4096, 28672, 2)):
        M = 16
        x = dv.DeviceMem.from_numpy((rng.standard_normal((M, K)).astype(np.float32).view(np.uint32) >> 16).astype(np.uint16), dev)
        sc = dv.DeviceMem.from_numpy(rng.uniform(0.001, 0.02, size=N).astype(np.float32), dev)
        wbufs = [dv.DeviceMem.from_numpy(rng.integers(-127, 128, size=(K, N), dtype=np.int8), dev) for _ in range(copies)]
        y = dv.DeviceMem(M * N * 2, dev)
        plan = dv.Plan.qdense(M, K, N, dv.BF16, dv.I8, dv.SCALE_CHANNEL, 0, False, False, dv.ACT_NONE, dev=dev)
        wss = [plan.new_workspace() for _ in range(copies)]
        seq = dv.BoundSequence([plan.bind([x.ptr, w.ptr, sc.ptr], [y.ptr], ws.ptr) for w, ws in zip(wbufs, wss)])
        reps = 20
        e0, e1 = dv.Event(dev), dv.Event(dev)
        for it in range(reps + 3):
            if it == 3:
                e0.record(stream)
            seq.launch(stream)
        e1.record(stream)
        stream.sync()
        for ws in wss:
            plan.check_status(ws.ptr)
        us = e0.elapsed_ms(e1) * 1e3 / (reps * copies)
        tiles = (N + 127) // 128
        bts = K * N + 4 * N + 2 * M * K + 2 * M * N
        res[name] = {"kernel": plan.kernel_name, "grid": plan.blocks, "column_tiles": tiles,
                     "ctas_per_tile": plan.blocks // tiles if plan.blocks % tiles == 0 and plan.blocks >= tiles else None,
                     "us_per_launch": us, "GB/s": bts / us / 1e3, "frac_of_measured_hbm": bts / us / 1e3 / hpeak}
        for m in [x, sc, y] + wbufs + wss:
            m.free()
    return res


def sdpa_leg(dv, dev, stream, hq, hkv, tpeak, check=False):
    """Causal SDPA of the fourth configuration restricted to `hq` query heads / `hkv` KV heads (all of them on one GPU,
    a KV-head group per rank when sharded: attention of a (batch, KV head) pair reads no other head).  With `check`
    one (batch, KV-head) group is compared with the oracle."""
    B, S, D = 8, 2048, 128
    rng = np.random.default_rng(40 + dev)
    qh = bf16_bits(rng.standard_normal((B, hq, S, D), dtype=np.float32))
    kh = bf16_bits(rng.standard_normal((B, hkv, S, D), dtype=np.float32))
    vh = bf16_bits(rng.standard_normal((B, hkv, S, D), dtype=np.float32))
    q, k, v = (dv.DeviceMem.from_numpy(t, dev) for t in (qh, kh, vh))
    o = dv.DeviceMem(B * hq * S * D * 2, dev)
    plan = dv.Plan.sdpa(B, hq, hkv, S, S, D, dv.BF16, causal=True, dev=dev)
    us = time_plan(dv, dev, stream, plan, [q.ptr, k.ptr, v.ptr], [o.ptr], 10)
    tf = 4.0 * B * hq * D * (S * (S + 1) / 2) / us / 1e6
    out = {"kernel": plan.kernel_name, "us": us, "TFLOP/s": tf, "frac_of_measured_bf16_peak": tf / tpeak,
           "query_heads": hq, "kv_heads": hkv}
    if check:
        from oracle import oracle as orc
        grp = hq // hkv
        b0, h0 = B - 1, hkv - 1            # the last batch and KV head: late tiles of the heaviest-first grid
        got = bf16_floats(o.download((B, hq, S, D), np.uint16)[b0, h0 * grp:(h0 + 1) * grp])
        want = orc.sdpa(bf16_floats(qh[b0:b0 + 1, h0 * grp:(h0 + 1) * grp]), bf16_floats(kh[b0:b0 + 1, h0:h0 + 1]),
                        bf16_floats(vh[b0:b0 + 1, h0:h0 + 1]), causal=True)[0]
        err = float(np.abs(got - want).max() / np.abs(want).max())
        out["checked"] = {"batch": b0, "kv_head": h0, "max_err": err, "tolerance": 2e-2}
        if not err < 2e-2:
            raise RuntimeError(f"sharded SDPA disagrees with the oracle: {err}")
    for m in (q, k, v, o):
        m.free()
    return out


def decoder_block_legs():
    """The fifth configuration: one Llama-style decoder block (hidden 4096, 32 / 8 heads of 128, MLP 14336, int8
    per-channel projections, bf16 activations) as one Executable, prefill 4 x 512 tokens and decode 16 x 1 token over a
    key / value cache of 2048 positions.  Inputs are resident buffers; the time is wall clock per Executable.Execute
    (launches plus the final sync), results finalised every step."""
    from compute_b200 import backend as be, decoder_block as blk
    cfg = blk.BlockConfig()
    backend = be.New("")
    weights = blk.make_block_weights(cfg, 5)
    rng = np.random.default_rng(9)
    out = {}
    for mode, (B, S, kv) in (("config5_decode_16x1_kv2048", (16, 1, 2048)), ("config5_prefill_4x512", (4, 512, 0))):
        exe, names = blk.compile_block(backend, cfg, B, S, kv)
        host = dict(weights)
        host["x"] = bf16_bits(rng.standard_normal((B, S, cfg.hidden), dtype=np.float32))
        if kv:
            host["cache_k"] = bf16_bits(rng.standard_normal((B, kv, cfg.kv_heads, cfg.head_dim), dtype=np.float32))
            host["cache_v"] = bf16_bits(rng.standard_normal((B, kv, cfg.kv_heads, cfg.head_dim), dtype=np.float32))
        bufs = [backend.BufferFromFlatData(0, host[n], blk.parameter_shape(n, cfg, B, S, kv)) for n in names]

        def step():
            for o in exe.Execute(bufs, None, 0):
                o.Finalize()
        for _ in range(3):
            step()
        reps = 30 if kv else 10
        t0 = time.perf_counter()
        for _ in range(reps):
            step()
        ms_block = (time.perf_counter() - t0) / reps * 1e3
        tokens = B * S
        weight_bytes = sum(int(np.prod(v.shape)) for k_, v in weights.items() if k_ in blk.PROJECTIONS)
        flops = 2.0 * tokens * weight_bytes + (4.0 * B * cfg.heads * cfg.head_dim * (S * (S + 1) / 2 if not kv else kv))
        out[mode] = {"ms_per_block": ms_block, "tokens": tokens, "kernels": exe.KernelNames(),
                     "weight_GB/s": weight_bytes / ms_block / 1e6, "TFLOP/s": flops / ms_block / 1e9}
        for b in bufs:
            b.Finalize()
        exe.Finalize()
    backend.Finalize()
    return out


# --------------------------------------------------------------------------- CPU baselines
def cpu_baseline(M: int, seconds: float = 12.0):
    """The oracle port (the reference's scalar loop nest with its row / N-tile parallel split) timed on the host
    cores over repeated launches of one layer."""
    from oracle import oracle as orc
    orc.build()
    threads = host_threads()
    rng = np.random.default_rng(1)
    x = bf16_floats(bf16_bits(rng.standard_normal((M, K_DIM), dtype=np.float32)))
    w, s = make_layer(100, slice(0, N_DIM))
    se = orc.expand_scales(s, "kgroup", K_DIM, N_DIM, GROUP)
    reps, t0 = 0, time.perf_counter()
    while True:
        orc.qdense_linear(x, w, se, None, None, 1, orc.ACT_SILU, threads=threads, fast=True)
        reps += 1
        el = time.perf_counter() - t0
        if el > seconds or reps >= 50:
            break
    gbs = reps * algorithmic_bytes(M, N_DIM) / el / 1e9
    return {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port",
            "sample": f"{reps} launches of one 4096x14336 layer at M={M} (f32 x, reference scale layout expanded), {el:.1f} s",
            "ms_per_launch": el / reps * 1e3}


def cpu_baseline_other():
    """Bounded CPU samples of the other two ops of the path: the AVX-512 GotoBLAS restatement of the reference's large
    float32 matmul (block sizes of dot/matmul/avx512.go) on a 2048^3 product, and its serial scalar SDPA loops on one
    (batch, KV-head) group of the fourth configuration at S = 512."""
    from oracle import oracle as orc
    orc.build()
    threads = host_threads()
    rng = np.random.default_rng(2)
    n = 2048
    a = rng.standard_normal((n, n), dtype=np.float32) / 45.0
    b = rng.standard_normal((n, n), dtype=np.float32) / 45.0
    orc.gemm_f32_blocked(a[:256], b, threads)
    t0 = time.perf_counter()
    orc.gemm_f32_blocked(a, b, threads)
    t_gemm = time.perf_counter() - t0
    S, D, grp = 512, 128, 4
    q = rng.standard_normal((1, grp, S, D), dtype=np.float32)
    k = rng.standard_normal((1, 1, S, D), dtype=np.float32)
    v = rng.standard_normal((1, 1, S, D), dtype=np.float32)
    t0 = time.perf_counter()
    orc.sdpa(q, k, v, causal=True)
    t_sdpa = time.perf_counter() - t0
    return {"dot_general_f32": {"value": 2.0 * n ** 3 / t_gemm / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                                "sample": f"one {n}^3 float32 product, {t_gemm:.2f} s"},
            "sdpa_causal_f32": {"value": 4.0 * grp * D * (S * (S + 1) / 2) / t_sdpa / 1e12, "unit": "TFLOP/s", "cores": 1, "kind": "port",
                                "sample": f"one (batch, KV head) group of 4 query heads, S={S}, D={D}, serial as in the reference, {t_sdpa:.2f} s"}}


def run_reference(args):
    """The reference arithmetic on the host cores.  One step = one launch over the first `cols` output columns of
    the 4096 x 14336 layer; `cols` is chosen from one timed full-layer launch so that the K steps fit ~90 s."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    M = args.m
    from oracle import oracle as orc
    orc.build()
    threads = host_threads()
    rng = np.random.default_rng(1)
    x = bf16_floats(bf16_bits(rng.standard_normal((M, K_DIM), dtype=np.float32)))
    w, s = make_layer(100, slice(0, N_DIM))
    se = orc.expand_scales(s, "kgroup", K_DIM, N_DIM, GROUP)
    full = lambda: orc.qdense_linear(x, w, se, None, None, 1, orc.ACT_SILU, threads=threads, fast=True)
    full()
    t0 = time.perf_counter()
    full()
    t_full = time.perf_counter() - t0
    frac = min(1.0, 90.0 / max(args.steps * t_full, 1e-9))
    cols = max(128, int(N_DIM * frac) // 128 * 128)
    wc, sc = np.ascontiguousarray(w[:, :cols]), np.ascontiguousarray(se[:, :cols])
    run = lambda: orc.qdense_linear(x, wc, sc, None, None, 1, orc.ACT_SILU, threads=threads, fast=True)
    for _ in range(min(args.warmup, 3)):
        run()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        run()
    el = time.perf_counter() - t0
    val = args.steps * algorithmic_bytes(M, cols) / el / 1e9
    sample = (f"each step = one launch over the first {cols} of {N_DIM} output columns of one 4096x{N_DIM} layer at M={M} "
              f"on {threads} host threads (a full layer takes {t_full * 1e3:.1f} ms)")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": val, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": el / args.steps * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic (seeded)",
        "config": {"workload": f"config3 decode quantized dense M={M} K={K_DIM} N={N_DIM} int8 W group-{GROUP} scales SiLU; "
                               "reference arithmetic (oracle port of gobackend's scalar kernel; no Go toolchain on this image)",
                   "sample": sample},
        "cpu_baseline": {"value": val, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# --------------------------------------------------------------------------- end to end through the Backend interface
def e2e_plugin(M, x_bits, layers_host, steps, warm):
    """The step through Backend / Builder / Executable / Buffer: 8 FusedQuantizedDense nodes on 8 activation parameters
    (the compiler groups them into one launch); weights and scales are parameter buffers created once.  Per step, inside
    the timed region: BufferFromFlatData of every activation (host -> device), Execute, ToFlatData of every result."""
    from compute_b200 import backend as be, device as dv
    backend = be.New("")
    builder = backend.Builder("decode-step")
    f = builder.Main()
    xs, ws, ss, outs = [], [], [], []
    for l in range(LAYERS):
        xs.append(f.Parameter(f"x{l}", be.make_shape(dv.BF16, M, K_DIM)))
    for l in range(LAYERS):
        ws.append(f.Parameter(f"w{l}", be.make_shape(dv.I8, K_DIM, N_DIM)))
        ss.append(f.Parameter(f"s{l}", be.make_shape(dv.F32, K_DIM // GROUP, N_DIM)))
    for l in range(LAYERS):
        outs.append(f.FusedQuantizedDense(xs[l], ws[l], None, be.Quantization(be.QUANT_LINEAR, ss[l], None, BlockAxis=0, BlockSize=GROUP), dv.ACT_SILU))
    f.Return(outs)
    exe = builder.Compile()
    kernels = exe.KernelNames()
    wbufs = []
    for l in range(LAYERS):
        w, s = layers_host[l]
        wbufs.append(backend.BufferFromFlatData(0, w, be.make_shape(dv.I8, K_DIM, N_DIM)))
        wbufs.append(backend.BufferFromFlatData(0, s, be.make_shape(dv.F32, K_DIM // GROUP, N_DIM)))
    x_shape = be.make_shape(dv.BF16, M, K_DIM)
    # the caller's flat slices live in page-locked memory (cb_host_alloc): transfers go straight to and from them
    x_pin = dv.PinnedHost((LAYERS, M, K_DIM), np.uint16)
    x_pin.array[...] = x_bits
    x_bits = x_pin.array
    y_pin = dv.PinnedHost((LAYERS, M, N_DIM), np.uint16)
    y_host = y_pin.array

    def step():
        xb = [backend.BufferFromFlatData(0, x_bits[l], x_shape) for l in range(LAYERS)]
        res = exe.Execute(xb + wbufs, None, 0)
        for l in range(LAYERS):
            res[l].ToFlatData(y_host[l])
            res[l].Finalize()
        for b in xb:
            b.Finalize()

    for _ in range(warm):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    el = time.perf_counter() - t0
    first = y_host.copy()
    exe.Finalize()
    for b in wbufs:
        b.Finalize()
    backend.Finalize()
    return el, kernels, first


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=500)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--m", type=int, default=16, help="decode batch (tokens per launch): 1, 4 or 16")
    ap.add_argument("--impl", default="cuda", choices=["cuda", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extra", action="store_true")
    ap.add_argument("--gather", default="fused", choices=["fused", "nccl"],
                    help="multi-GPU: column slices stored straight into every rank's result buffers by the kernel over NVLink "
                         "(default), or one NCCL all-gather per step")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "cuda" else args.warmup
    if args.impl == "reference":
        return run_reference(args)

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    g = world
    assert N_DIM % (g * 128) == 0, "shards must be whole column tiles"

    from compute_b200 import device as dv
    dv.init()
    lib = dv._lib.load()
    dev = local
    M = args.m
    n_loc = N_DIM // g
    cols = slice(rank * n_loc, (rank + 1) * n_loc)
    fused = dist is not None and args.gather == "fused"

    stream = dv.Stream(dev)
    rng = np.random.default_rng(7)
    x_bits = bf16_bits(rng.standard_normal((LAYERS, M, K_DIM), dtype=np.float32))
    layers_host = [make_layer(100 + layer, slice(0, N_DIM)) if g == 1 else make_layer(100 + layer, cols) for layer in range(LAYERS)]
    w_dev = [dv.DeviceMem.from_numpy(w, dev) for w, _ in layers_host]
    s_dev = [dv.DeviceMem.from_numpy(s, dev) for _, s in layers_host]
    x_host = dv.PinnedHost((LAYERS, M, K_DIM), np.uint16)
    x_host.array[...] = x_bits
    x_dev = dv.DeviceMem.from_numpy(x_bits, dev)
    x_stride, y_stride, full_stride = M * K_DIM * 2, M * n_loc * 2, M * N_DIM * 2
    members = [(n_loc, False, dv.ACT_SILU)] * LAYERS

    def group_inputs(xptr):
        ins = []
        for l in range(LAYERS):
            ins += [xptr + l * x_stride, w_dev[l].ptr, s_dev[l].ptr]
        return ins

    # ---- the step: one grouped launch over the LAYERS projections (or their column shards)
    # Multi-GPU.  torch.distributed only hands out handles / ids and the barriers; the data path is this library's:
    #  fused: the kernel stores its column slices into the result buffers of every rank over NVLink (buffers opened with
    #         cb_ipc_open); one cb_peer_signal_wait per step makes the stream wait for the slices of all ranks.
    #         Two sets of result buffers alternate, so a rank that runs one step ahead never overwrites results a slower
    #         rank has not consumed yet.
    #  nccl:  every rank computes into its own slice buffers, then one cb_comm_allgather per step.
    plan = dv.Plan.qdense_group(M, K_DIM, members, dv.BF16, dv.I8, dv.SCALE_KGROUP, GROUP, dev=dev,
                                gather_ranks=g if fused else 0, gather_rank=rank if fused else 0)
    state = {"steps": 0}
    comm = None
    if fused:
        y_full = [dv.DeviceMem(LAYERS * full_stride, dev) for _ in range(2)]
        flags = dv.DeviceMem(256, dev)          # words [0, g): arrivals per source rank; word 16: wait status
        flags.zero()
        for yb in y_full:
            yb.zero()
        mine = [dv.ipc_export(y_full[0]), dv.ipc_export(y_full[1]), dv.ipc_export(flags)]
        everyone = [None] * g
        dist.all_gather_object(everyone, mine)
        peer_y = [[y_full[bb].ptr if r == rank else dv.ipc_open(dev, everyone[r][bb]) for bb in range(2)] for r in range(g)]
        peer_flags = [flags.ptr if r == rank else dv.ipc_open(dev, everyone[r][2]) for r in range(g)]
        wss = [plan.new_workspace() for _ in range(2)]
        bounds = [plan.bind(group_inputs(x_dev.ptr), [peer_y[r][bb] + l * full_stride for l in range(LAYERS) for r in range(g)], wss[bb].ptr)
                  for bb in range(2)]
        peer_barrier = dv.PeerBarrier(dev, peer_flags, rank, flags.ptr, flags.ptr + 64)
        dist.barrier()
    else:
        y_dev = dv.DeviceMem(LAYERS * y_stride, dev)
        wss = [plan.new_workspace()]
        bounds = [plan.bind(group_inputs(x_dev.ptr), [y_dev.ptr + l * y_stride for l in range(LAYERS)], wss[0].ptr)]
        if dist is not None:
            ids = [dv.Comm.unique_id() if rank == 0 else None]
            dist.broadcast_object_list(ids, src=0)
            comm = dv.Comm(dev, g, rank, ids[0])
            y_all = dv.DeviceMem(g * LAYERS * y_stride, dev)

    def step():
        if fused:
            bb = state["steps"] & 1
            bounds[bb].launch(stream)
            state["steps"] += 1
            peer_barrier.signal_wait(state["steps"], stream)
            return
        bounds[0].launch(stream)
        if comm is not None:
            comm.allgather(y_dev.ptr, y_all.ptr, LAYERS * y_stride, stream)

    def sync():
        dv.check(lib.cb_stream_sync(dev, stream.handle))
        if dist is not None:
            import torch
            torch.cuda.synchronize()

    def barrier():
        sync()
        if dist is not None:
            dist.barrier()
            sync()

    def check_all():
        for ws in wss:
            plan.check_status(ws.ptr)
        if fused and int(flags.download((64,), np.uint32)[16]):
            raise RuntimeError(f"rank {rank}: a slice of another rank did not arrive")

    def timed(fn, steps: int):
        """CUDA events on the launching stream around `steps` calls; also the wall time the host needs to issue them."""
        e0, e1 = dv.Event(dev), dv.Event(dev)
        barrier()
        e0.record(stream)
        t0 = time.perf_counter()
        for _ in range(steps):
            fn()
        t_issue = time.perf_counter() - t0
        e1.record(stream)
        sync()
        ms = e0.elapsed_ms(e1)
        barrier()
        if dist is not None:
            import torch
            t = torch.tensor([ms], device=f"cuda:{local}")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms, t_issue

    for _ in range(args.warmup):
        step()
    sync()
    check_all()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    ms, t_issue = timed(step, args.steps)
    clocks = sampler.stop() if rank == 0 else None
    check_all()
    kernels_per_step = 2 + (1 if fused else 0)          # digit kernel + main kernel (+ the signal-and-wait kernel)

    # ---- the gathered result is checked, outside the timed region: every rank's buffer against the bits of the
    # unsharded plan on rank 0's GPU, and one layer against the oracle
    gather_check = None
    if dist is not None:
        import torch
        sync()
        if fused:
            got = y_full[(state["steps"] - 1) & 1].download((LAYERS, M, N_DIM), np.uint16)
        else:
            ya = y_all.download((g, LAYERS, M, n_loc), np.uint16)
            got = np.ascontiguousarray(np.transpose(ya, (1, 2, 0, 3))).reshape(LAYERS, M, N_DIM)
        digest = torch.tensor(np.frombuffer(np.ascontiguousarray(got).tobytes(), np.uint8).astype(np.int64).reshape(-1, 4096).sum(1)[:4096], device=f"cuda:{local}")
        ref = digest.clone()
        dist.broadcast(ref, src=0)
        same_everywhere = torch.tensor([int(bool(torch.equal(ref, digest)))], device=f"cuda:{local}")
        dist.all_reduce(same_everywhere, op=dist.ReduceOp.MIN)
        if rank == 0:
            from oracle import oracle as orc
            check_layer = LAYERS - 1
            wf, sf = make_layer(100 + check_layer, slice(0, N_DIM))
            single = dv.Plan.qdense(M, K_DIM, N_DIM, dv.BF16, dv.I8, dv.SCALE_KGROUP, GROUP, False, False, dv.ACT_SILU, dev=dev)
            sws = single.new_workspace()
            wd, sd, yd = dv.DeviceMem.from_numpy(wf, dev), dv.DeviceMem.from_numpy(sf, dev), dv.DeviceMem(full_stride, dev)
            single.launch([x_dev.ptr + check_layer * x_stride, wd.ptr, sd.ptr], [yd.ptr], sws.ptr, stream)
            stream.sync()
            one_gpu = yd.download((M, N_DIM), np.uint16)
            xf = bf16_floats(x_bits[check_layer])
            want = orc.qdense_linear(xf, wf, orc.expand_scales(sf, "kgroup", K_DIM, N_DIM, GROUP), None, None, 1, orc.ACT_SILU,
                                     threads=host_threads(), fast=True)
            err = float(np.abs(bf16_floats(got[check_layer]) - want).max() / np.abs(want).max())
            err_1gpu = float(np.abs(bf16_floats(got[check_layer]) - bf16_floats(one_gpu)).max() / np.abs(want).max())
            gather_check = {"gather_checked": True, "layer": check_layer, "max_err_vs_oracle": err, "tolerance": 2e-2,
                            "max_diff_vs_unsharded_plan": err_1gpu, "all_ranks_hold_the_same_bytes": bool(same_everywhere.item())}
            if not (err < 2e-2 and err_1gpu < 2.0 ** -7 and same_everywhere.item()):
                raise RuntimeError(f"gathered result is wrong: {gather_check}")
            for m in (wd, sd, yd):
                m.free()
        # multi-rank AllReduce through the C ABI: every rank contributes rank + 1
        if comm is None:
            ids = [dv.Comm.unique_id() if rank == 0 else None]
            dist.broadcast_object_list(ids, src=0)
            comm = dv.Comm(dev, g, rank, ids[0])
        buf = dv.DeviceMem.from_numpy(np.full(1024, rank + 1, np.float32), dev)
        comm.allreduce(buf.ptr, buf.ptr, 1024, dv.F32, dv.REDUCE_SUM, stream)
        stream.sync()
        red = buf.download((1024,), np.float32)
        if not np.all(red == g * (g + 1) / 2):
            raise RuntimeError(f"rank {rank}: all-reduce gave {red[:4]}")
        if gather_check is not None:
            gather_check["allreduce_checked"] = True
        dist.barrier()

    # ---- sharded SDPA leg (fourth configuration by KV-head groups): per-GPU time, one group checked against the oracle
    sdpa_sharded = None
    if dist is not None and 8 % g == 0:
        import torch
        tpeak, _ = measured_peak("bf16_tflops", 1590.0)
        leg = sdpa_leg(dv, dev, stream, 32 // g, 8 // g, tpeak, check=(rank == 0))
        t = torch.tensor([leg["us"]], device=f"cuda:{local}")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        leg["us_max_over_ranks"] = float(t.item())
        leg["whole_job_TFLOP/s"] = 4.0 * 8 * 32 * 128 * (2048 * 2049 / 2) / leg["us_max_over_ranks"] / 1e6
        sdpa_sharded = leg

    # ---- multi-GPU end-to-end leg through the C ABI (every rank takes part): activations in from pinned host memory,
    # the step, the gathered result out to pinned host memory, every step
    ms_e2e_multi = None
    if dist is not None:
        y_host_full = dv.PinnedHost((LAYERS, M, N_DIM), np.uint16)

        def step_e2e():
            dv.check(lib.cb_h2d(dev, x_dev.ptr, x_host.ptr, LAYERS * x_stride, stream.handle))
            step()
            if fused:
                dv.check(lib.cb_d2h(dev, y_host_full.ptr, y_full[(state["steps"] - 1) & 1].ptr, LAYERS * full_stride, stream.handle))
            else:
                dv.check(lib.cb_d2h(dev, y_host_full.ptr, y_all.ptr, g * LAYERS * y_stride, stream.handle))
        for _ in range(3):
            step_e2e()
        ms_e2e_multi, _ = timed(step_e2e, args.steps)
        check_all()

    bytes_layer = algorithmic_bytes(M, n_loc)
    bytes_launch = LAYERS * bytes_layer
    job_bytes_step = LAYERS * (algorithmic_bytes(M, N_DIM) if g == 1 else g * bytes_layer)
    flops_step = LAYERS * 2 * M * K_DIM * N_DIM
    value = job_bytes_step * args.steps / (ms * 1e-3) / 1e9
    peak, peak_kind = measured_peak()
    launch_us = ms * 1e3 / args.steps                   # one grouped launch per step (includes the per-step gather when g > 1)
    achieved = bytes_launch / (launch_us * 1e-6) / 1e9

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    out = {
        "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": g, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "int8 weights x int8 digits of the bf16 activations, s32 accumulate per 128-k unit, f32 across units", "data": "synthetic (seeded)",
        "config": {"workload": f"config3 decode quantized dense: x bf16 [{M},{K_DIM}], W int8 [{K_DIM},{N_DIM}], "
                               f"group-{GROUP} f32 scales along K, SiLU, bf16 out; {LAYERS} distinct independent layers per step, one grouped launch",
                   "M": M, "K": K_DIM, "N": N_DIM, "layers_per_step": LAYERS,
                   "parallelism": ("single GPU" if g == 1 else
                                   f"N-sharded x{g}, column slices stored into every rank's result buffers by the kernel (peer stores over NVLink), one flag wait per step"
                                   if fused else f"N-sharded x{g}, one NCCL all-gather per step"),
                   "l2": f"{LAYERS} distinct weight matrices per step ({LAYERS * K_DIM * N_DIM // g >> 20} MiB per GPU) exceed the 126 MB L2" if LAYERS * K_DIM * N_DIM // g > 126e6 else
                         "per-GPU weights of a step fit in L2 at this shard count; launches may be served from L2",
                   "kernel": plan.kernel_name, "grid": [plan.blocks, plan.threads], "dyn_smem": plan.dyn_smem},
        "tflops": flops_step * args.steps / (ms * 1e-3) / 1e12,
        "gpu_launches": args.steps * kernels_per_step,
        "host_issue_us_per_step": t_issue * 1e6 / args.steps,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": NCU_TRAFFIC_BYTES.get(M) if g == 1 else None, "peak_kind": f"of {peak_kind}",
                     "algorithmic_bytes_per_launch": bytes_launch, "us_per_launch": launch_us, "layers_per_launch": LAYERS,
                     "us_per_layer": launch_us / LAYERS, "frac_of_nominal_8TBs": achieved / 8000.0},
        "clocks": clocks,
    }
    if gather_check is not None:
        out.update(gather_check)
    if sdpa_sharded is not None:
        out["sdpa_sharded_by_kv_head_groups"] = sdpa_sharded
    if g == 1:
        # ---- the same layers as LAYERS separate, dependent-style launches (one projection per launch, issued from C)
        single = dv.Plan.qdense(M, K_DIM, N_DIM, dv.BF16, dv.I8, dv.SCALE_KGROUP, GROUP, False, False, dv.ACT_SILU, dev=dev)
        sws = [single.new_workspace() for _ in range(LAYERS)]
        y2 = dv.DeviceMem(LAYERS * y_stride, dev)
        seq = dv.BoundSequence([single.bind([x_dev.ptr + l * x_stride, w_dev[l].ptr, s_dev[l].ptr], [y2.ptr + l * y_stride], sws[l].ptr)
                                for l in range(LAYERS)])
        for _ in range(5):
            seq.launch(stream)
        ms1, t1 = timed(lambda: seq.launch(stream), max(args.steps // 2, 5))
        n1 = max(args.steps // 2, 5) * LAYERS
        us1 = ms1 * 1e3 / n1
        out["one_projection_per_launch"] = {"kernel": single.kernel_name, "us_per_launch": us1, "GB/s": bytes_layer / us1 / 1e3,
                                            "frac_of_measured_hbm": bytes_layer / us1 / 1e3 / peak, "host_issue_us_per_launch": t1 * 1e6 / n1,
                                            "note": "what a chain of dependent layers pays: every launch fills and drains its own pipeline"}
        grouped_bits = y_dev.download((LAYERS, M, n_loc), np.uint16)
        per_launch_bits = y2.download((LAYERS, M, n_loc), np.uint16)
        diff = float(np.abs(bf16_floats(grouped_bits) - bf16_floats(per_launch_bits)).max() / np.abs(bf16_floats(per_launch_bits)).max())
        if not diff < 2.0 ** -7:
            raise RuntimeError(f"grouped and per-layer launches disagree: {diff}")
        out["one_projection_per_launch"]["max_diff_vs_grouped_launch"] = diff

        # ---- end to end through the Backend interface (the headline e2e) and the pipelined C-ABI figure
        n_e2e = max(min(args.steps, 200), 5)
        el, kernels, y_plugin = e2e_plugin(M, x_bits, layers_host, n_e2e, 3)
        diff = float(np.abs(bf16_floats(y_plugin) - bf16_floats(grouped_bits)).max() / np.abs(bf16_floats(grouped_bits)).max())
        if not diff < 2.0 ** -7:
            raise RuntimeError(f"the Executable's result differs from the bound launch: {diff}")
        out["e2e"] = {"value": job_bytes_step * n_e2e / el / 1e9, "unit": "GB/s", "h2d_bytes_per_step": LAYERS * x_stride,
                      "d2h_bytes_per_step": LAYERS * y_stride, "ms_per_step": el / n_e2e * 1e3, "steps": n_e2e, "copies_declared": True,
                      "through": "Backend.BufferFromFlatData x8 -> Executable.Execute -> Buffer.ToFlatData x8 (the calls a cgo shim binds) on page-locked flat slices, wall clock, one step at a time",
                      "kernels": kernels, "max_diff_vs_bound_launch": diff}
        # pipelined: copies of neighbouring steps overlap the kernels (two activation and two result buffers, a copy-in and
        # a copy-out stream, events between them); every step still copies its inputs and results inside the timed region
        y_host = [dv.PinnedHost((LAYERS, M, n_loc), np.uint16) for _ in range(2)]
        xb = [x_dev, dv.DeviceMem(LAYERS * x_stride, dev)]
        yb = [y_dev, dv.DeviceMem(LAYERS * y_stride, dev)]
        pws = [wss[0], plan.new_workspace()]
        pb = [bounds[0], plan.bind(group_inputs(xb[1].ptr), [yb[1].ptr + l * y_stride for l in range(LAYERS)], pws[1].ptr)]
        s_in, s_out = dv.Stream(dev), dv.Stream(dev)
        ev_in, ev_done, ev_out = ([dv.Event(dev), dv.Event(dev)] for _ in range(3))

        def run_pipelined(steps):
            e0, e1 = dv.Event(dev), dv.Event(dev)
            sync(); s_in.sync(); s_out.sync()
            e0.record(s_in)
            for i in range(steps):
                b = i & 1
                if i >= 2:
                    s_in.wait_event(ev_done[b])          # x buffer b was read by the kernels of step i-2
                dv.check(lib.cb_h2d(dev, xb[b].ptr, x_host.ptr, LAYERS * x_stride, s_in.handle))
                ev_in[b].record(s_in)
                stream.wait_event(ev_in[b])
                if i >= 2:
                    stream.wait_event(ev_out[b])         # y buffer b was copied out by step i-2
                pb[b].launch(stream)
                ev_done[b].record(stream)
                s_out.wait_event(ev_done[b])
                dv.check(lib.cb_d2h(dev, y_host[b].ptr, yb[b].ptr, LAYERS * y_stride, s_out.handle))
                ev_out[b].record(s_out)
            e1.record(s_out)
            s_out.sync(); sync(); s_in.sync()
            return e0.elapsed_ms(e1)

        run_pipelined(3)
        ms_p = run_pipelined(args.steps)
        out["e2e_pipelined"] = {"value": job_bytes_step * args.steps / (ms_p * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": ms_p / args.steps,
                                "h2d_bytes_per_step": LAYERS * x_stride, "d2h_bytes_per_step": LAYERS * y_stride,
                                "through": "C ABI: cb_h2d / cb_bound_launch / cb_d2h on three streams, pinned host buffers, CUDA events"}
        if not args.no_extra:
            extra = {}
            for m_other in (1, 4, 16):
                if m_other == M:
                    continue
                p2 = dv.Plan.qdense_group(m_other, K_DIM, members, dv.BF16, dv.I8, dv.SCALE_KGROUP, GROUP, dev=dev)
                ws2 = p2.new_workspace()
                ins2 = []
                for l in range(LAYERS):
                    ins2 += [x_dev.ptr + l * m_other * K_DIM * 2, w_dev[l].ptr, s_dev[l].ptr]
                b2 = p2.bind(ins2, [y_dev.ptr + l * m_other * n_loc * 2 for l in range(LAYERS)], ws2.ptr)
                for _ in range(5):
                    b2.launch(stream)
                ms2, _ = timed(lambda: b2.launch(stream), max(args.steps // 2, 5))
                us = ms2 * 1e3 / max(args.steps // 2, 5)
                bts = LAYERS * algorithmic_bytes(m_other, N_DIM)
                extra[f"M={m_other}"] = {"us_per_launch": us, "us_per_layer": us / LAYERS, "GB/s": bts / us / 1e3,
                                         "frac_of_measured_hbm": bts / us / 1e3 / peak, "kernel": p2.kernel_name}
                p2.check_status(ws2.ptr)
            out["other_decode_batches"] = extra
            out["other_path_kernels"] = other_kernels(dv, dev, stream)
            out["other_weight_formats"] = weight_format_legs(dv, dev, stream)
            out["decoder_block"] = decoder_block_legs()
            out["decoder_block_projections"] = block_projection_legs(dv, dev, stream)
        if not args.no_cpu_baseline:
            out["cpu_baseline"] = cpu_baseline(M)
            if not args.no_extra:
                out["cpu_baseline_other_ops"] = cpu_baseline_other()
    else:
        out["e2e"] = {"value": job_bytes_step * args.steps / (ms_e2e_multi * 1e-3) / 1e9, "unit": "GB/s", "h2d_bytes_per_step": LAYERS * x_stride,
                      "d2h_bytes_per_step": LAYERS * full_stride, "ms_per_step": ms_e2e_multi / args.steps, "copies_declared": True,
                      "through": "C ABI on every rank: cb_h2d of the activations, the grouped launch with its gather, cb_d2h of the gathered result, one stream"}
    print(json.dumps(out))
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
