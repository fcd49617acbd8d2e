#!/usr/bin/env python
"""Benchmark of the hot path: decode-shaped int8 quantized dense on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--m 16] [--impl reference]

Workload (BASELINE config 3): x bf16 [M, 4096], W int8 [4096, 14336], group-128
float32 scales along K, SiLU, output bf16.  One *step* runs the projection for
LAYERS distinct weight matrices (LAYERS x 58.7 MB > the 126 MB L2, so every
launch streams its weights from HBM).  With N GPUs the projection is sharded
along N (each rank holds columns [r*N/g, (r+1)*N/g) of every layer; x is
replicated) and the per-rank output slices are all-gathered once per step.

Prints ONE JSON line (rank 0).  `value` = algorithmic bytes of the whole job per
second with inputs resident in HBM; `e2e` = the same metric with the per-step
activations copied from pinned host memory and the results copied back inside
the timed region (weights stay resident, as model parameters do).
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
# dram__bytes_read.sum + dram__bytes_write.sum per launch from the committed ncu capture
# (profiles/); None until a capture of the current kernel exists.
NCU_TRAFFIC_BYTES = {1: 60_721_664 + 210_432, 4: None, 16: 60_858_624 + 261_888}   # profiles/qdense_decode_tc_config3_M16.md


def algorithmic_bytes(M: int, n_cols: int) -> int:
    """int8 W + f32 group scales + bf16 x + bf16 out for one launch over n_cols columns."""
    return K_DIM * n_cols + 4 * (K_DIM // GROUP) * n_cols + 2 * M * K_DIM + 2 * M * n_cols


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


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


def make_layer(seed: int, M: int, cols: slice):
    """Seeded synthetic weights of one layer, restricted to this rank's columns."""
    rng = np.random.default_rng(seed)
    w = rng.integers(-127, 128, size=(K_DIM, N_DIM), dtype=np.int8)
    s = rng.uniform(0.001, 0.02, size=(K_DIM // GROUP, N_DIM)).astype(np.float32)
    return np.ascontiguousarray(w[:, cols]), np.ascontiguousarray(s[:, cols])


def other_kernels(dv, dev, stream):
    """The tensor-core rows of the path, timed alone (CUDA events, inputs resident): DotGeneral
    4096^3 bf16 (config 2) and causal SDPA B=8, 32/8 heads, D=128, S=2048 bf16 (config 4)."""
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            tpeak = float(json.load(f)["bf16_tflops"])
    except Exception:
        tpeak = 1590.0
    rng = np.random.default_rng(3)

    def rand_bf16(n):
        a = (rng.standard_normal(n, dtype=np.float32) * 0.05).view(np.uint32) >> 16
        return dv.DeviceMem.from_numpy(a.astype(np.uint16), dev)

    def time_plan(plan, ins, outs, reps):
        ws = plan.new_workspace()
        e0, e1 = dv.Event(dev), dv.Event(dev)
        for it in range(reps + 3):
            if it == 3:
                e0.record(stream)
            plan.launch(ins, outs, ws.ptr if ws else None, stream)
        e1.record(stream)
        stream.sync()
        plan.check_status(ws.ptr if ws else None)
        return e0.elapsed_ms(e1) * 1e3 / reps

    res = {}
    n = 4096
    a, b, c = rand_bf16(n * n), rand_bf16(n * n), dv.DeviceMem(n * n * 2, dev)
    plan = dv.Plan.dot(1, n, n, n, dv.BF16, dev=dev)
    us = time_plan(plan, [a.ptr, b.ptr], [c.ptr], 20)
    tf = 2.0 * n ** 3 / us / 1e6
    res["dot_general_4096_bf16"] = {"kernel": plan.kernel_name, "us": us, "TFLOP/s": tf, "frac_of_measured_bf16_peak": tf / tpeak}
    for m in (a, b, c):
        m.free()
    # the same product on float32 operands (three bf16 planes each, six plane products)
    af = dv.DeviceMem.from_numpy(rng.standard_normal(n * n, dtype=np.float32) * 0.05, dev)
    bf = dv.DeviceMem.from_numpy(rng.standard_normal(n * n, dtype=np.float32) * 0.05, dev)
    cf = dv.DeviceMem(n * n * 4, dev)
    plan = dv.Plan.dot(1, n, n, n, dv.F32, dev=dev)
    us = time_plan(plan, [af.ptr, bf.ptr], [cf.ptr], 10)
    res["dot_general_4096_f32"] = {"kernel": plan.kernel_name, "us": us, "TFLOP/s": 2.0 * n ** 3 / us / 1e6,
                                   "note": "f32-accurate result from 6 bf16 plane products; includes the two split launches"}
    for m in (af, bf, cf):
        m.free()
    # batched [32,512,128] x [32,128,512] bf16
    a, b, c = rand_bf16(32 * 512 * 128), rand_bf16(32 * 128 * 512), dv.DeviceMem(32 * 512 * 512 * 2, dev)
    plan = dv.Plan.dot(32, 512, 512, 128, dv.BF16, dev=dev)
    us = time_plan(plan, [a.ptr, b.ptr], [c.ptr], 50)
    res["dot_general_batched_32x512x128x512_bf16"] = {"kernel": plan.kernel_name, "us": us,
                                                      "GB/s": (2 * 32 * 512 * 128 * 2 + 32 * 512 * 512 * 2) / us / 1e3}
    for m in (a, b, c):
        m.free()
    # prefill-shaped quantized dense: 4 x 512 tokens through the 4096 x 14336 projection, per-channel scales
    Mp = 2048
    x = rand_bf16(Mp * K_DIM)
    w = dv.DeviceMem.from_numpy(rng.integers(-127, 128, size=K_DIM * N_DIM, dtype=np.int8), dev)
    sc = dv.DeviceMem.from_numpy(rng.uniform(0.001, 0.02, size=N_DIM).astype(np.float32), dev)
    y = dv.DeviceMem(Mp * N_DIM * 2, dev)
    plan = dv.Plan.qdense(Mp, K_DIM, N_DIM, dv.BF16, dv.I8, dv.SCALE_CHANNEL, 0, False, False, dv.ACT_SILU, dev=dev)
    us = time_plan(plan, [x.ptr, w.ptr, sc.ptr], [y.ptr], 10)
    tf = 2.0 * Mp * K_DIM * N_DIM / us / 1e6
    res["quantized_dense_prefill_2048x4096x14336_bf16"] = {"kernel": plan.kernel_name, "us": us, "TFLOP/s": tf,
                                                          "frac_of_measured_bf16_peak": tf / tpeak,
                                                          "note": "includes expanding the int8 weights to bf16"}
    for m in (x, w, sc, y):
        m.free()
    B, Hq, Hkv, S, D = 8, 32, 8, 2048, 128
    q, k, v = rand_bf16(B * Hq * S * D), rand_bf16(B * Hkv * S * D), rand_bf16(B * Hkv * S * D)
    o = dv.DeviceMem(B * Hq * S * D * 2, dev)
    plan = dv.Plan.sdpa(B, Hq, Hkv, S, S, D, dv.BF16, causal=True, dev=dev)
    us = time_plan(plan, [q.ptr, k.ptr, v.ptr], [o.ptr], 10)
    tf = 4.0 * B * Hq * D * (S * (S + 1) / 2) / us / 1e6
    res["sdpa_causal_b8_h32_8_s2048_d128_bf16"] = {"kernel": plan.kernel_name, "us": us, "TFLOP/s": tf,
                                                     "frac_of_measured_bf16_peak": tf / tpeak}
    for m in (q, k, v, o):
        m.free()
    # the bandwidth-bound fused ops around the dense layers: 65536 rows of 4096 float32 (1 GiB in, 1 GiB out)
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            hpeak = float(json.load(f)["hbm_gbs"])
    except Exception:
        hpeak = FALLBACK_HBM_GBS
    rows, L = 65536, 4096
    xf = dv.DeviceMem.from_numpy(rng.standard_normal(rows * L, dtype=np.float32), dev)
    gf = dv.DeviceMem.from_numpy(rng.standard_normal(L, dtype=np.float32), dev)
    yf = dv.DeviceMem(rows * L * 4, dev)
    for name, plan, ins in (("fused_softmax_65536x4096_f32", dv.Plan.softmax(dv.F32, rows, L, 1, dev=dev), [xf.ptr]),
                            ("fused_layer_norm_65536x4096_f32", dv.Plan.layernorm(dv.F32, rows, L, 1e-5, True, True, dev=dev), [xf.ptr, gf.ptr, gf.ptr]),
                            ("fused_gelu_268M_f32", dv.Plan.gelu(dv.F32, rows * L, True, dev=dev), [xf.ptr])):
        us = time_plan(plan, ins, [yf.ptr], 10)
        gbs = 2.0 * rows * L * 4 / us / 1e3
        res[name] = {"kernel": plan.kernel_name, "us": us, "GB/s": gbs, "frac_of_measured_hbm": gbs / hpeak}
    for m in (xf, gf, yf):
        m.free()
    return res


def cpu_baseline(M: int, seconds: float = 12.0):
    """The oracle port (the reference's scalar loop nest with its row / N-tile parallel split)
    timed on the host cores over repeated launches of one layer."""
    from oracle import oracle as orc
    orc.build()
    threads = host_threads()
    rng = np.random.default_rng(1)
    x = orc.bf16_to_f32(orc.bf16_from_f32(rng.standard_normal((M, K_DIM), dtype=np.float32)))
    w, s = make_layer(100, M, slice(0, N_DIM))
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


def host_threads() -> int:
    """All host cores this process may use (torchrun sets OMP_NUM_THREADS=1, which the CPU arm must not inherit)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


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
    x = orc.bf16_to_f32(orc.bf16_from_f32(rng.standard_normal((M, K_DIM), dtype=np.float32)))
    w, s = make_layer(100, M, slice(0, N_DIM))
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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--m", type=int, default=16, help="decode batch (tokens per launch): 1, 4 or 16")
    ap.add_argument("--impl", default="cuda", choices=["cuda", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extra", action="store_true")
    ap.add_argument("--gather", default="nccl", choices=["fused", "nccl"],
                    help="multi-GPU: column slices gathered with one NCCL all-gather per step (default: measured "
                         "slightly faster at 2 GPUs) or stored straight into every rank's result buffer by the kernel")
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
    from oracle import oracle as orc   # bf16 helpers + cpu_baseline only; never on the measured path
    dv.init()
    dev = local
    M = args.m
    n_loc = N_DIM // g
    cols = slice(rank * n_loc, (rank + 1) * n_loc)

    plan = dv.Plan.qdense(M, K_DIM, n_loc, dv.BF16, dv.I8, dv.SCALE_KGROUP, GROUP, False, False, dv.ACT_SILU, dev=dev)
    ws = plan.new_workspace()
    stream = dv.Stream(dev)
    rng = np.random.default_rng(7)
    x_host = dv.PinnedHost((LAYERS, M, K_DIM), np.uint16)
    x_host.array[...] = orc.bf16_from_f32(rng.standard_normal((LAYERS, M, K_DIM), dtype=np.float32))
    y_host = dv.PinnedHost((LAYERS, M, n_loc), np.uint16)
    w_dev, s_dev = [], []
    for layer in range(LAYERS):
        w, s = make_layer(100 + layer, M, cols)
        w_dev.append(dv.DeviceMem.from_numpy(w, dev))
        s_dev.append(dv.DeviceMem.from_numpy(s, dev))
    x_dev = dv.DeviceMem.from_numpy(x_host.array, dev)
    y_dev = dv.DeviceMem(LAYERS * M * n_loc * 2, dev)
    x_stride, y_stride = M * K_DIM * 2, M * n_loc * 2
    wsp = ws.ptr if ws else None

    # Multi-GPU.  torch.distributed only hands out handles / ids and the barriers; the data path is this library's:
    #  fused: the decode kernel stores its column slice into the result buffer of every rank over NVLink (buffers
    #         opened with cb_ipc_open) ; one cb_peer_signal + cb_peer_wait per step makes the stream wait for the
    #         slices of all ranks.  Two result buffers alternate, so a rank that runs one step ahead never
    #         overwrites results a slower rank has not consumed yet.
    #  nccl:  every rank computes into its own slice buffer, then one cb_comm_allgather per step.
    gather = None
    fused = None
    y_dev_ptr = y_dev.ptr
    stream_l = stream
    full_stride = M * N_DIM * 2
    if dist is not None and args.gather == "nccl":
        ids = [dv.Comm.unique_id() if rank == 0 else None]
        dist.broadcast_object_list(ids, src=0)
        comm = dv.Comm(dev, g, rank, ids[0])
        y_all = dv.DeviceMem(g * LAYERS * y_stride, dev)

        def gather():
            comm.allgather(y_dev_ptr, y_all.ptr, LAYERS * y_stride, stream)
    elif dist is not None:
        y_full = [dv.DeviceMem(LAYERS * full_stride, dev) for _ in range(2)]
        flags = dv.DeviceMem(256, dev)          # words [0, g): arrivals per source rank; word 16: wait status
        flags.zero()
        mine = [dv.ipc_export(y_full[0]), dv.ipc_export(y_full[1]), dv.ipc_export(flags)]
        everyone = [None] * g
        dist.all_gather_object(everyone, mine)
        peer_y = [[y_full[bb].ptr if r == rank else dv.ipc_open(dev, everyone[r][bb]) for bb in range(2)] for r in range(g)]
        peer_flags = [flags.ptr if r == rank else dv.ipc_open(dev, everyone[r][2]) for r in range(g)]
        plan = dv.Plan.qdense(M, K_DIM, n_loc, dv.BF16, dv.I8, dv.SCALE_KGROUP, GROUP, False, False, dv.ACT_SILU, dev=dev,
                              gather_ranks=g, gather_rank=rank)
        ws = plan.new_workspace()
        wsp = ws.ptr
        fused = {"steps": 0}
        dist.barrier()

    def step(copy: bool):
        if copy:      # this step's activations: one pinned-host -> device copy
            dv.check(dv._lib.load().cb_h2d(dev, x_dev.ptr, x_host.ptr, LAYERS * x_stride, stream_l.handle))
        if fused is not None:
            bb = fused["steps"] & 1
            for layer in range(LAYERS):
                plan.launch([x_dev.ptr + layer * x_stride, w_dev[layer].ptr, s_dev[layer].ptr],
                            [peer_y[r][bb] + layer * full_stride for r in range(g)], wsp, stream_l)
            fused["steps"] += 1
            dv.peer_signal(dev, peer_flags, rank, stream_l)
            dv.peer_wait(dev, flags.ptr, g, fused["steps"], flags.ptr + 64, stream_l)
            if copy:  # the gathered result of this step
                dv.check(dv._lib.load().cb_d2h(dev, y_full_host.ptr, y_full[bb].ptr, LAYERS * full_stride, stream_l.handle))
            return
        for layer in range(LAYERS):
            plan.launch([x_dev.ptr + layer * x_stride, w_dev[layer].ptr, s_dev[layer].ptr],
                        [y_dev_ptr + layer * y_stride], wsp, stream_l)
        if gather:
            gather()
        if copy:      # this step's results: one device -> pinned-host copy
            dv.check(dv._lib.load().cb_d2h(dev, y_host.ptr, y_dev_ptr, LAYERS * y_stride, stream_l.handle))

    y_full_host = dv.PinnedHost((LAYERS, M, N_DIM), np.uint16) if fused is not None else None

    # End-to-end leg on one GPU: the copies of neighbouring steps overlap the kernels (two activation and
    # two result buffers, a copy-in and a copy-out stream, events between them).  Every step still copies its
    # own inputs from pinned host memory and its own results back, inside the timed region.
    pipe = None
    if dist is None:
        pipe = {"s_in": dv.Stream(dev), "s_out": dv.Stream(dev),
                "x": [x_dev, dv.DeviceMem(LAYERS * x_stride, dev)], "y": [y_dev, dv.DeviceMem(LAYERS * y_stride, dev)],
                "y_host": [y_host, dv.PinnedHost((LAYERS, M, n_loc), np.uint16)],
                "ev_in": [dv.Event(dev), dv.Event(dev)], "ev_done": [dv.Event(dev), dv.Event(dev)],
                "ev_out": [dv.Event(dev), dv.Event(dev)], "i": 0}

    def step_pipelined():
        lib = dv._lib.load()
        i = pipe["i"]
        b = i & 1
        pipe["i"] = i + 1
        if i >= 2:
            pipe["s_in"].wait_event(pipe["ev_done"][b])      # x buffer b was read by the kernels of step i-2
        dv.check(lib.cb_h2d(dev, pipe["x"][b].ptr, x_host.ptr, LAYERS * x_stride, pipe["s_in"].handle))
        pipe["ev_in"][b].record(pipe["s_in"])
        stream.wait_event(pipe["ev_in"][b])
        if i >= 2:
            stream.wait_event(pipe["ev_out"][b])               # y buffer b was copied out by step i-2
        for layer in range(LAYERS):
            plan.launch([pipe["x"][b].ptr + layer * x_stride, w_dev[layer].ptr, s_dev[layer].ptr],
                        [pipe["y"][b].ptr + layer * y_stride], wsp, stream)
        pipe["ev_done"][b].record(stream)
        pipe["s_out"].wait_event(pipe["ev_done"][b])
        dv.check(lib.cb_d2h(dev, pipe["y_host"][b].ptr, pipe["y"][b].ptr, LAYERS * y_stride, pipe["s_out"].handle))
        pipe["ev_out"][b].record(pipe["s_out"])

    def timed_pipelined(steps: int):
        e0, e1 = dv.Event(dev), dv.Event(dev)
        barrier()
        pipe["s_in"].sync(); pipe["s_out"].sync()
        pipe["i"] = 0
        e0.record(pipe["s_in"])
        for _ in range(steps):
            step_pipelined()
        e1.record(pipe["s_out"])
        pipe["s_out"].sync(); sync(); pipe["s_in"].sync()
        return e0.elapsed_ms(e1)

    def sync():
        dv.check(dv._lib.load().cb_stream_sync(dev, stream_l.handle))
        if dist is not None:
            import torch
            torch.cuda.synchronize()

    def barrier():
        sync()
        if dist is not None:
            dist.barrier()
            sync()

    def timed(copy: bool, steps: int):
        e0, e1 = dv.Event(dev), dv.Event(dev)
        barrier()
        e0.record(stream_l)
        for _ in range(steps):
            step(copy)
        e1.record(stream_l)
        sync()
        ms = e0.elapsed_ms(e1)
        barrier()
        if dist is not None:
            import torch
            t = torch.tensor([ms], device=f"cuda:{local}")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    for _ in range(args.warmup):
        step(False)
    sync()
    plan.check_status(wsp)
    if fused is not None and int(flags.download((64,), np.uint32)[16]):
        raise RuntimeError(f"rank {rank}: a slice of another rank did not arrive during warm-up")
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    ms = timed(False, args.steps)
    clocks = sampler.stop() if rank == 0 else None
    plan.check_status(wsp)
    if pipe is not None:
        timed_pipelined(3)
        ms_e2e = timed_pipelined(args.steps)
    else:
        for _ in range(3):
            step(True)
        ms_e2e = timed(True, args.steps)

    if fused is not None:
        sync()
        wait_status = int(flags.download((64,), np.uint32)[16])
        if wait_status:
            raise RuntimeError(f"rank {rank}: timed out waiting for the slice of rank {wait_status - 1}")
        # a sample of the gathered result: the slice another rank stored here equals the one this rank computed there
        dist.barrier()          # nobody frees buffers its peers may still be writing

    bytes_launch = algorithmic_bytes(M, n_loc)
    job_bytes_step = LAYERS * (algorithmic_bytes(M, N_DIM) if g == 1 else g * bytes_launch)
    flops_step = LAYERS * 2 * M * K_DIM * N_DIM
    value = job_bytes_step * args.steps / (ms * 1e-3) / 1e9
    e2e = job_bytes_step * args.steps / (ms_e2e * 1e-3) / 1e9
    peak, peak_kind = measured_peak()
    launch_us = ms * 1e3 / (args.steps * LAYERS)       # includes the per-step gather when g > 1
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
                               f"group-{GROUP} f32 scales along K, SiLU, bf16 out; {LAYERS} distinct layers per step",
                   "M": M, "K": K_DIM, "N": N_DIM, "layers_per_step": LAYERS,
                   "parallelism": ("single GPU" if g == 1 else
                                   f"N-sharded x{g}, column slices stored into every rank's result buffer by the kernel (peer stores over NVLink), one flag wait per step"
                                   if fused is not None else f"N-sharded x{g}, one NCCL all-gather per step"),
                   "l2": f"{LAYERS} distinct weight matrices per step ({LAYERS * K_DIM * N_DIM // g >> 20} MiB per GPU) exceed the 126 MB L2" if LAYERS * K_DIM * N_DIM // g > 126e6 else
                         "per-GPU weights of a step fit in L2 at this shard count; launches may be served from L2",
                   "kernel": plan.kernel_name, "grid": [plan.blocks, plan.threads], "dyn_smem": plan.dyn_smem},
        "tflops": flops_step * args.steps / (ms * 1e-3) / 1e12,
        # the tensor-core decode plan launches two kernels per call: the activation digit kernel and the main kernel
        "gpu_launches": args.steps * (LAYERS * (2 if plan.kernel_name.startswith("qdense_decode_tc") else 1)
                                      + (2 if fused is not None else 0)),     # + the signal and wait kernels of a gathered step
        "e2e": {"value": e2e, "unit": "GB/s", "h2d_bytes_per_step": LAYERS * x_stride, "d2h_bytes_per_step": LAYERS * (full_stride if fused is not None else y_stride),
                "ms_per_step": ms_e2e / args.steps,
                "note": "activations H2D from pinned memory and results D2H every step (copies of neighbouring steps overlap the kernels on one GPU); weights resident as device buffers"},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": NCU_TRAFFIC_BYTES.get(M) if g == 1 else None, "peak_kind": f"of {peak_kind}",
                     "algorithmic_bytes_per_launch": bytes_launch, "us_per_launch": launch_us,
                     "frac_of_nominal_8TBs": achieved / 8000.0},
        "clocks": clocks,
    }
    if g == 1 and not args.no_extra:
        extra = {}
        for m_other in (1, 4, 16):
            if m_other == M:
                continue
            p2 = dv.Plan.qdense(m_other, K_DIM, N_DIM, dv.BF16, dv.I8, dv.SCALE_KGROUP, GROUP, False, False, dv.ACT_SILU, dev=dev)
            ws2 = p2.new_workspace()
            e0, e1 = dv.Event(dev), dv.Event(dev)
            reps = max(args.steps // 2, 5)
            for it in range(reps + 3):
                if it == 3:
                    e0.record(stream)
                for layer in range(LAYERS):
                    p2.launch([x_dev.ptr, w_dev[layer].ptr, s_dev[layer].ptr], [y_dev.ptr], ws2.ptr, stream)
            e1.record(stream)
            stream.sync()
            us = e0.elapsed_ms(e1) * 1e3 / (reps * LAYERS)
            b = algorithmic_bytes(m_other, N_DIM)
            extra[f"M={m_other}"] = {"us_per_launch": us, "GB/s": b / us / 1e3, "frac_of_measured_hbm": b / us / 1e3 / peak,
                                     "kernel": p2.kernel_name}
        out["other_decode_batches"] = extra
        out["other_path_kernels"] = other_kernels(dv, dev, stream)
    if g == 1 and not args.no_cpu_baseline:
        out["cpu_baseline"] = cpu_baseline(M)
    print(json.dumps(out))
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
