"""Runs one kernel of the library on a named synthetic case and prints its device time.

    python -m compute_b200.run_case gemm --dtype bf16 --b 1 --m 4096 --n 4096 --k 4096
    python -m compute_b200.run_case sdpa --b 8 --hq 32 --hkv 8 --s 2048 --d 128 --causal
    python -m compute_b200.run_case sdpa --b 16 --sq 1 --s 2048 --bshd      # one new token against a 2048-key cache
    python -m compute_b200.run_case qdense --m 16            # decode (M <= 16) or prefill (M > 16)
    python -m compute_b200.run_case qdense --m 16 --layers 8 # eight independent projections as one grouped launch
    python -m compute_b200.run_case softmax --m 65536 --n 4096   # also: gelu, layernorm (rows --m, row length --n)

A small stand-alone driver for timing or profiling a single plan (inputs are seeded random
data resident on the device; time is taken with CUDA events on the launching stream).  The
profile summaries of this repository were captured from these commands.
"""
from __future__ import annotations

import argparse
import json

import numpy as np

from . import device as dv


def _bf16(rng, n, sigma=0.05):
    a = (rng.standard_normal(n, dtype=np.float32) * sigma).view(np.uint32) >> 16
    return a.astype(np.uint16)


def _time(plan, ins, outs, dev, stream, reps, warmup):
    ws = plan.new_workspace()
    e0, e1 = dv.Event(dev), dv.Event(dev)
    for it in range(reps + warmup):
        if it == warmup:
            e0.record(stream)
        plan.launch(ins, outs, ws.ptr if ws else None, stream)
    e1.record(stream)
    stream.sync()
    plan.check_status(ws.ptr if ws else None)
    return e0.elapsed_ms(e1) * 1e3 / reps


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("case", choices=["gemm", "sdpa", "qdense", "softmax", "gelu", "layernorm"])
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "f32"])
    ap.add_argument("--b", type=int, default=1)
    ap.add_argument("--m", type=int, default=4096)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--hq", type=int, default=32)
    ap.add_argument("--hkv", type=int, default=8)
    ap.add_argument("--s", type=int, default=2048)
    ap.add_argument("--d", type=int, default=128)
    ap.add_argument("--sq", type=int, default=0, help="query length when it differs from the key length --s")
    ap.add_argument("--bshd", action="store_true", help="[batch, seq, heads, dim] operands instead of [batch, heads, seq, dim]")
    ap.add_argument("--layers", type=int, default=1, help="qdense: this many independent projections as one grouped launch")
    ap.add_argument("--ggml", default="", choices=["", "q4_0", "q8_0", "iq4_nl", "q4_k", "q6_k"],
                    help="qdense: weights in this GGML block format instead of int8 with separate scales")
    ap.add_argument("--packed4", default="", choices=["", "i4", "u4", "nf4"],
                    help="qdense: packed 4-bit weights (Int4 / Uint4 Linear, or NF4 on Uint4) with the reference's [K, N / group] scales")
    ap.add_argument("--causal", action="store_true")
    ap.add_argument("--layout", default="kgroup", choices=["channel", "kgroup"])
    ap.add_argument("--group", type=int, default=128)
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--dev", type=int, default=0)
    a = ap.parse_args()
    dev = a.dev
    dv.init()
    stream = dv.Stream(dev)
    rng = np.random.default_rng(1)
    out = {"case": a.case}
    if a.case == "gemm":
        code = dv.BF16 if a.dtype == "bf16" else dv.F32
        size = 2 if a.dtype == "bf16" else 4
        mk = (lambda n: _bf16(rng, n)) if a.dtype == "bf16" else (lambda n: rng.standard_normal(n, dtype=np.float32) * np.float32(0.05))
        lhs = dv.DeviceMem.from_numpy(mk(a.b * a.m * a.k), dev)
        rhs = dv.DeviceMem.from_numpy(mk(a.b * a.k * a.n), dev)
        res = dv.DeviceMem(a.b * a.m * a.n * size, dev)
        plan = dv.Plan.dot(a.b, a.m, a.n, a.k, code, dev=dev)
        us = _time(plan, [lhs.ptr, rhs.ptr], [res.ptr], dev, stream, a.reps, a.warmup)
        out.update(kernel=plan.kernel_name, us=us, tflops=2.0 * a.b * a.m * a.n * a.k / us / 1e6)
    elif a.case == "sdpa":
        sq = a.sq or a.s
        f32 = a.dtype == "f32"                      # float32 operands: the tiled CUDA-core kernel
        mk = (lambda n: rng.standard_normal(n, dtype=np.float32)) if f32 else (lambda n: _bf16(rng, n, 1.0))
        q = dv.DeviceMem.from_numpy(mk(a.b * a.hq * sq * a.d), dev)
        k = dv.DeviceMem.from_numpy(mk(a.b * a.hkv * a.s * a.d), dev)
        v = dv.DeviceMem.from_numpy(mk(a.b * a.hkv * a.s * a.d), dev)
        o = dv.DeviceMem(a.b * a.hq * sq * a.d * (4 if f32 else 2), dev)
        plan = dv.Plan.sdpa(a.b, a.hq, a.hkv, sq, a.s, a.d, dv.F32 if f32 else dv.BF16, causal=a.causal,
                            layout=dv.LAYOUT_BSHD if a.bshd else dv.LAYOUT_BHSD, dev=dev)
        us = _time(plan, [q.ptr, k.ptr, v.ptr], [o.ptr], dev, stream, a.reps, a.warmup)
        pairs = (a.s * (a.s + 1) / 2 if a.causal else a.s * a.s) if sq == a.s else sq * a.s
        out.update(kernel=plan.kernel_name, us=us, tflops=4.0 * a.b * a.hq * a.d * pairs / us / 1e6,
                   kv_GBps=2.0 * a.b * a.hkv * a.s * a.d * (4 if f32 else 2) / us / 1e3)
    elif a.case in ("softmax", "gelu", "layernorm"):
        code = dv.BF16 if a.dtype == "bf16" else dv.F32
        size = 2 if a.dtype == "bf16" else 4
        rows, L = a.m, a.n
        x = dv.DeviceMem.from_numpy(_bf16(rng, rows * L, 1.0) if a.dtype == "bf16" else rng.standard_normal(rows * L, dtype=np.float32), dev)
        y = dv.DeviceMem(rows * L * size, dev)
        ins = [x.ptr]
        if a.case == "softmax":
            plan = dv.Plan.softmax(code, rows, L, 1, dev=dev)
        elif a.case == "gelu":
            plan = dv.Plan.gelu(code, rows * L, True, dev=dev)
        else:
            g = dv.DeviceMem.from_numpy(_bf16(rng, L, 1.0) if a.dtype == "bf16" else rng.standard_normal(L, dtype=np.float32), dev)
            plan = dv.Plan.layernorm(code, rows, L, 1e-5, True, True, dev=dev)
            ins += [g.ptr, g.ptr]
        us = _time(plan, ins, [y.ptr], dev, stream, a.reps, a.warmup)
        out.update(kernel=plan.kernel_name, us=us, GBps=2.0 * rows * L * size / us / 1e3)
    else:
        K, N = a.k, a.n if a.n != 4096 else 14336
        code = dv.BF16 if a.dtype == "bf16" else dv.F32
        x = dv.DeviceMem.from_numpy(_bf16(rng, a.m * K, 1.0) if a.dtype == "bf16" else rng.standard_normal(a.m * K, dtype=np.float32), dev)
        w = dv.DeviceMem.from_numpy(rng.integers(-127, 128, size=K * N, dtype=np.int8), dev)
        rows = 1 if a.layout == "channel" else -(-K // a.group)
        sc = dv.DeviceMem.from_numpy(rng.uniform(0.001, 0.02, size=rows * N).astype(np.float32), dev)
        y = dv.DeviceMem(a.m * N * (2 if a.dtype == "bf16" else 4), dev)
        layout = dv.SCALE_CHANNEL if a.layout == "channel" else dv.SCALE_KGROUP
        if a.packed4:
            nblk = -(-N // a.group)
            scr = dv.DeviceMem.from_numpy(rng.uniform(0.001, 0.02, size=K * nblk).astype(np.float32), dev)
            # --layers copies of the weights, one launch each in turn
            wps = [dv.DeviceMem.from_numpy(rng.integers(0, 256, size=K * N // 2, dtype=np.uint8), dev) for _ in range(a.layers)]
            plan = dv.Plan.qdense(a.m, K, N, code, dv.I4 if a.packed4 == "i4" else dv.U4, dv.SCALE_REF, a.group, activation=dv.ACT_SILU,
                                  scheme=dv.QUANT_NF4 if a.packed4 == "nf4" else dv.QUANT_LINEAR, dev=dev)
            ws = plan.new_workspace()
            e0, e1 = dv.Event(dev), dv.Event(dev)
            for it in range(a.reps + a.warmup):
                if it == a.warmup:
                    e0.record(stream)
                for wp in wps:
                    plan.launch([x.ptr, wp.ptr, scr.ptr], [y.ptr], ws.ptr if ws else None, stream)
            e1.record(stream)
            stream.sync()
            us = e0.elapsed_ms(e1) * 1e3 / (a.reps * a.layers)
            out.update(kernel=plan.kernel_name, blocks=plan.blocks, us=us, weight_GBps=(K * N / 2 + K * nblk * 4) / us / 1e3,
                       tflops=2.0 * a.m * K * N / us / 1e6)
            print(json.dumps(out))
            return
        if a.ggml:
            # random block bytes with a finite half-precision scale in every block
            gt, values, bb, scale_at = {"q4_0": (dv.GGML_Q4_0, 32, 18, (0,)), "q8_0": (dv.GGML_Q8_0, 32, 34, (0,)),
                                        "iq4_nl": (dv.GGML_IQ4_NL, 32, 18, (0,)), "q4_k": (dv.GGML_Q4_K, 256, 144, (0, 2)),
                                        "q6_k": (dv.GGML_Q6_K, 256, 210, (208,))}[a.ggml]
            blocks = rng.integers(0, 256, size=(N, K // values, bb), dtype=np.uint8)
            for o in scale_at:
                blocks[:, :, o:o + 2] = np.frombuffer(np.float16(0.03125).tobytes(), np.uint8)
            # --layers copies of the weights, one launch each in turn: more bytes than the L2 holds between two uses of a copy
            wgs = [dv.DeviceMem.from_numpy(blocks.reshape(N, -1), dev) for _ in range(a.layers)]
            plan = dv.Plan.qdense(a.m, K, N, code, dv.U8, has_bias=False, activation=dv.ACT_SILU, scheme=dv.QUANT_GGML, ggml_type=gt, dev=dev)
            ws = plan.new_workspace()
            e0, e1 = dv.Event(dev), dv.Event(dev)
            for it in range(a.reps + a.warmup):
                if it == a.warmup:
                    e0.record(stream)
                for wg in wgs:
                    plan.launch([x.ptr, wg.ptr], [y.ptr], ws.ptr if ws else None, stream)
            e1.record(stream)
            stream.sync()
            plan.check_status(ws.ptr if ws else None)
            us = e0.elapsed_ms(e1) * 1e3 / (a.reps * a.layers)
            out.update(kernel=plan.kernel_name, blocks=plan.blocks, us=us, weight_GBps=blocks.nbytes / us / 1e3,
                       tflops=2.0 * a.m * K * N / us / 1e6)
            print(json.dumps(out))
            return
        if a.layers > 1:
            # independent projections (own weights, scales, outputs; one shared activation) as one launch
            ws_ = [w] + [dv.DeviceMem.from_numpy(rng.integers(-127, 128, size=K * N, dtype=np.int8), dev) for _ in range(a.layers - 1)]
            ys = [y] + [dv.DeviceMem(a.m * N * (2 if a.dtype == "bf16" else 4), dev) for _ in range(a.layers - 1)]
            plan = dv.Plan.qdense_group(a.m, K, [(N, False, dv.ACT_SILU)] * a.layers, code, dv.I8, layout, a.group, dev=dev)
            ins = []
            for wl in ws_:
                ins += [x.ptr, wl.ptr, sc.ptr]
            us = _time(plan, ins, [t.ptr for t in ys], dev, stream, a.reps, a.warmup)
        else:
            plan = dv.Plan.qdense(a.m, K, N, code, dv.I8, layout, a.group, False, False, dv.ACT_SILU, dev=dev)
            us = _time(plan, [x.ptr, w.ptr, sc.ptr], [y.ptr], dev, stream, a.reps, a.warmup)
        out.update(kernel=plan.kernel_name, blocks=plan.blocks, us=us, weight_GBps=a.layers * K * N / us / 1e3,
                   tflops=2.0 * a.layers * a.m * K * N / us / 1e6)
    print(json.dumps(out))


if __name__ == "__main__":
    main()
