"""Shared helpers of the test-suite: golden-fixture loading, dtype names, seeded inputs."""
import json
import os

import numpy as np

from oracle import oracle as orc

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
DT = {"f32": orc.F32, "f64": orc.F64, "bf16": orc.BF16, "f16": orc.F16,
      "i32": orc.I32, "i64": orc.I64, "i8": orc.I8, "u8": orc.U8, "bool": orc.BOOL}
ACT = {"none": orc.ACT_NONE, "gelu": orc.ACT_GELU, "relu": orc.ACT_RELU, "silu": orc.ACT_SILU,
       "hard_swish": orc.ACT_HARDSWISH, "tanh": orc.ACT_TANH}


def load_golden(name):
    with open(os.path.join(GOLDEN, name)) as f:
        return json.load(f)


def tensor(spec, dtype_name):
    """JSON {shape, data} -> array in the carrier type of dtype_name (uint16 for halves)."""
    a = np.array(spec["data"], np.float64).reshape(spec["shape"])
    code = DT[spec.get("dtype", dtype_name)]
    if code in (orc.BF16, orc.F16):
        return orc.from_f32(a.astype(np.float32), code)
    if code == orc.BOOL:
        return a.astype(np.bool_)
    return a.astype({orc.F32: np.float32, orc.F64: np.float64, orc.I32: np.int32, orc.I64: np.int64,
                     orc.I8: np.int8, orc.U8: np.uint8}[code])


def as_f64(a, code):
    if code in (orc.BF16, orc.F16):
        return orc.to_f32(a, code).astype(np.float64)
    return np.asarray(a).astype(np.float64)


def max_abs_normalised(got, want):
    """max |got-want| / max |want| — the error measure of the parity tolerances."""
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    denom = max(float(np.max(np.abs(want))) if want.size else 0.0, 1e-30)
    return float(np.max(np.abs(got - want))) / denom if want.size else 0.0


def qdense_inputs(seed, M, K, N, x_dtype="f32", scale_layout="channel", group=128, bias=True,
                  unsigned=False, block_size=None):
    """Seeded synthetic inputs with the distributions of the benchmark configs:
    x ~ N(0,1), W uniform integers in [-127,127], scales ~ U(0.001,0.02), bias ~ N(0,0.1)."""
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((M, K), dtype=np.float32)
    if x_dtype == "bf16":
        x = orc.bf16_to_f32(orc.bf16_from_f32(x))      # values exactly representable in bf16
    if unsigned:
        w = rng.integers(0, 256, size=(K, N), dtype=np.int64).astype(np.uint8)
    else:
        w = rng.integers(-127, 128, size=(K, N), dtype=np.int64).astype(np.int8)
    if scale_layout == "channel":
        s = rng.uniform(0.001, 0.02, size=(N,)).astype(np.float32)
    elif scale_layout == "kgroup":
        s = rng.uniform(0.001, 0.02, size=((K + group - 1) // group, N)).astype(np.float32)
    else:  # "ref": [K, ceil(N/block_size)]
        s = rng.uniform(0.001, 0.02, size=(K, (N + block_size - 1) // block_size)).astype(np.float32)
    b = (rng.standard_normal(N) * 0.1).astype(np.float32) if bias else None
    return x, w, s, b
