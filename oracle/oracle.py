"""ctypes/numpy front end of the CPU oracle — TEST INFRASTRUCTURE ONLY.

Only the test-suite, the smoke check and the benchmark's CPU-baseline leg may
import this module; the product package never does.  See oracle.h for which
reference function each entry point restates and how parity is pinned
(FusedQuantizedDense: parity unpinned — the reference has no asserting test).

Half-precision arrays travel as ``np.uint16`` bit patterns together with an
explicit dtype code (the codes of gomlx/compute dtypes/dtype_enum.go:18-120).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))

BOOL, I8, I16, I32, I64, U8, U16, U32, U64, F16, F32, F64, BF16 = range(1, 14)
ACT_NONE, ACT_GELU, ACT_RELU, ACT_SILU, ACT_HARDSWISH, ACT_TANH = range(6)

_NP_OF = {BOOL: np.bool_, I8: np.int8, I16: np.int16, I32: np.int32, I64: np.int64,
          U8: np.uint8, U16: np.uint16, U32: np.uint32, U64: np.uint64,
          F16: np.uint16, F32: np.float32, F64: np.float64, BF16: np.uint16}


def build(force: bool = False) -> None:
    """Compile liboracle.so / liboracle_fast.so with the Makefile beside this file."""
    need = force or not all(os.path.exists(os.path.join(HERE, n))
                            for n in ("liboracle.so", "liboracle_fast.so"))
    if need:
        subprocess.run(["make", "-C", HERE, "-s"] + (["-B"] if force else []), check=True)


_libs: dict = {}


def lib(fast: bool = False):
    name = "liboracle_fast.so" if fast else "liboracle.so"
    if name not in _libs:
        path = os.path.join(HERE, name)
        if not os.path.exists(path):
            build()
        L = C.CDLL(path)
        L.orc_bf16_from_f32_n.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
        L.orc_bf16_to_f32_n.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
        L.orc_f16_from_f32.argtypes = [C.c_float]
        L.orc_f16_from_f32.restype = C.c_uint16
        L.orc_f16_to_f32.argtypes = [C.c_uint16]
        L.orc_f16_to_f32.restype = C.c_float
        L.orc_qdense_linear.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p,
                                        C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64,
                                        C.c_int64, C.c_int, C.c_int]
        L.orc_activation_f32.argtypes = [C.c_void_p, C.c_size_t, C.c_int]
        L.orc_unpack_int4.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
        L.orc_unpack_uint4.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
        L.orc_nf4_values.argtypes = []
        L.orc_nf4_values.restype = C.POINTER(C.c_float)
        L.orc_qdense_nf4.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                     C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_int, C.c_int]
        L.orc_dot_general.argtypes = [C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p,
                                      C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p,
                                      C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int]
        L.orc_dot_general.restype = C.c_int
        L.orc_sdpa_f32.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p,
                                   C.c_void_p, C.c_int, C.c_int, C.c_void_p,
                                   C.c_void_p, C.c_int, C.c_void_p,
                                   C.c_void_p, C.c_void_p, C.c_void_p,
                                   C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_int64,
                                   C.c_int, C.c_double, C.c_int]
        L.orc_sdpa_f32_slice.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                         C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_int64,
                                         C.c_int, C.c_double, C.c_int,
                                         C.c_int64, C.c_int64, C.c_int64, C.c_int64]
        L.orc_gemm_f32_blocked.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p,
                                           C.c_int64, C.c_int64, C.c_int64, C.c_int]
        L.orc_max_threads.restype = C.c_int
        _libs[name] = L
    return _libs[name]


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _c(a, dt):
    return np.ascontiguousarray(a, dtype=dt)


def max_threads() -> int:
    return int(lib().orc_max_threads())


# ---------------------------------------------------------------- half types
def bf16_from_f32(a) -> np.ndarray:
    a = _c(a, np.float32)
    out = np.empty(a.shape, np.uint16)
    lib().orc_bf16_from_f32_n(_p(a), _p(out), a.size)
    return out


def bf16_to_f32(a) -> np.ndarray:
    a = _c(a, np.uint16)
    out = np.empty(a.shape, np.float32)
    lib().orc_bf16_to_f32_n(_p(a), _p(out), a.size)
    return out


def f16_from_f32(a) -> np.ndarray:
    a = _c(a, np.float32)
    L = lib()
    return np.array([L.orc_f16_from_f32(float(v)) for v in a.ravel()], np.uint16).reshape(a.shape)


def f16_to_f32(a) -> np.ndarray:
    a = _c(a, np.uint16)
    L = lib()
    return np.array([L.orc_f16_to_f32(int(v)) for v in a.ravel()], np.float32).reshape(a.shape)


def to_f32(a, dtype: int) -> np.ndarray:
    if dtype == BF16:
        return bf16_to_f32(a)
    if dtype == F16:
        return np.asarray(a, np.uint16).view(np.float16).astype(np.float32)
    return np.asarray(a).astype(np.float32)


def from_f32(a, dtype: int) -> np.ndarray:
    if dtype == BF16:
        return bf16_from_f32(a)
    if dtype == F16:
        return np.asarray(a, np.float32).astype(np.float16).view(np.uint16)
    return np.asarray(a).astype(_NP_OF[dtype])


# ---------------------------------------------------------------- quantized dense
def expand_scales(scales, layout: str, K: int, N: int, group: int = 0) -> np.ndarray:
    """Compact scale layouts -> the reference form ``[K, N]`` with BlockSize = 1.

    ``layout``: "channel" (``[N]``, one scale per output column) or "kgroup"
    (``[K/group, N]``, one scale per `group` consecutive input rows and column).
    The expanded tensor makes the reference arithmetic element-wise identical.
    """
    s = np.asarray(scales, np.float32)
    if layout == "channel":
        return np.ascontiguousarray(np.broadcast_to(s.reshape(1, N), (K, N)))
    if layout == "kgroup":
        return np.ascontiguousarray(np.repeat(s.reshape(-1, N), group, axis=0)[:K])
    raise ValueError(layout)


def qdense_linear(x, w, scales, zero_points=None, bias=None, block_size: int = 1,
                  activation: int = ACT_NONE, threads: int = 1, fast: bool = False) -> np.ndarray:
    """Reference FusedQuantizedDense, Linear scheme (quantizeddense.go:616-650)."""
    x = _c(x, np.float32)
    K = x.shape[-1]
    M = x.size // K if K else 0
    w = np.ascontiguousarray(w)
    assert w.dtype in (np.int8, np.uint8) and w.shape[0] == K
    N = w.shape[1]
    nblk = (N + block_size - 1) // block_size
    scales = _c(scales, np.float32)
    assert scales.shape == (K, nblk), (scales.shape, (K, nblk))
    zp = None if zero_points is None else _c(zero_points, np.float32)
    b = None if bias is None else _c(bias, np.float32)
    out = np.empty(x.shape[:-1] + (N,), np.float32)
    lib(fast).orc_qdense_linear(_p(x), _p(w), int(w.dtype == np.uint8), _p(scales), _p(zp), _p(b),
                                _p(out), M, K, N, block_size, activation, threads)
    return out


def unpack_int4(packed, n: int) -> np.ndarray:
    """Packed Int4 bytes -> the first `n` int8 values (convertdtype.go:199-214: low nibble first)."""
    b = np.ascontiguousarray(packed, np.uint8).reshape(-1)
    out = np.empty(2 * b.size, np.int8)
    lib().orc_unpack_int4(_p(b), _p(out), b.size)
    return out[:n]


def unpack_uint4(packed, n: int) -> np.ndarray:
    """Packed Uint4 bytes -> the first `n` uint8 values (convertdtype.go:216-226)."""
    b = np.ascontiguousarray(packed, np.uint8).reshape(-1)
    out = np.empty(2 * b.size, np.uint8)
    lib().orc_unpack_uint4(_p(b), _p(out), b.size)
    return out[:n]


def pack_nibbles(values) -> np.ndarray:
    """Flat 4-bit values (signed or unsigned) -> packed bytes, low nibble first (the inverse of unpack_*)."""
    v = (np.asarray(values).astype(np.int16).reshape(-1) & 0x0F).astype(np.uint8)
    if v.size % 2:
        v = np.concatenate([v, np.zeros(1, np.uint8)])
    return (v[0::2] | (v[1::2] << 4)).astype(np.uint8)


def nf4_values() -> np.ndarray:
    """The 16 NormalFloat4 table values (fused_ops.go:114-121)."""
    ptr = lib().orc_nf4_values()
    return np.array([ptr[i] for i in range(16)], np.float32)


def qdense_nf4(x, w, scales, bias=None, block_size: int = 1, activation: int = ACT_NONE) -> np.ndarray:
    """Reference FusedQuantizedDense, NF4 scheme (quantizeddense.go:586-609); `w` holds one int8 /
    uint8 per element, of which the low nibble indexes the table."""
    x = _c(x, np.float32)
    K = x.shape[-1]
    M = x.size // K if K else 0
    w = np.ascontiguousarray(w)
    assert w.dtype in (np.int8, np.uint8) and w.shape[0] == K
    N = w.shape[1]
    nblk = (N + block_size - 1) // block_size
    scales = _c(scales, np.float32)
    assert scales.shape == (K, nblk), (scales.shape, (K, nblk))
    b = None if bias is None else _c(bias, np.float32)
    out = np.empty(x.shape[:-1] + (N,), np.float32)
    lib().orc_qdense_nf4(_p(x), _p(w), _p(scales), _p(b), _p(out), M, K, N, block_size, activation, 1)
    return out


def activation_f64(y: np.ndarray, activation: int) -> np.ndarray:
    """Mathematical definition of the activations in float64 (an independent check)."""
    from math import erf
    y = np.asarray(y, np.float64)
    if activation == ACT_NONE:
        return y
    if activation == ACT_RELU:
        return np.maximum(y, 0)
    if activation == ACT_SILU:
        return y / (1.0 + np.exp(-y))
    if activation == ACT_TANH:
        return np.tanh(y)
    if activation == ACT_HARDSWISH:
        return y * np.clip(y / 6.0 + 0.5, 0, 1)
    if activation == ACT_GELU:
        return y * 0.5 * (1.0 + np.vectorize(erf)(y / np.sqrt(2.0)))
    raise ValueError(activation)


def qdense_decomposed(x, w, scales, zero_points=None, bias=None, block_size: int = 1,
                      activation: int = ACT_NONE) -> np.ndarray:
    """The reference's decomposed formulation (benchmarks.go:510-545) in float64:
    dequantise the weights, matmul, add bias, activation.  Independent of the
    fused loop order, so it cross-checks the restatement above."""
    x = np.asarray(x, np.float64)
    w = np.asarray(w)
    K, N = w.shape
    cols = np.arange(N) // block_size
    wd = w.astype(np.float64) * np.asarray(scales, np.float64)[:, cols]
    if zero_points is not None:
        wd = wd + np.asarray(zero_points, np.float64)[:, cols]
    y = x.reshape(-1, K) @ wd
    if bias is not None:
        y = y + np.asarray(bias, np.float64)[None, :]
    return activation_f64(y, activation).reshape(x.shape[:-1] + (N,))


# ---------------------------------------------------------------- DotGeneral
def dot_output_dims(lhs_dims, lhs_contract, lhs_batch, rhs_dims, rhs_contract, rhs_batch):
    """shapeinference/dotgeneral.go:99-147: batch..., lhs cross..., rhs cross..."""
    out = [lhs_dims[a] for a in lhs_batch]
    out += [d for a, d in enumerate(lhs_dims) if a not in lhs_contract and a not in lhs_batch]
    out += [d for a, d in enumerate(rhs_dims) if a not in rhs_contract and a not in rhs_batch]
    return out


def dot_general(lhs, lhs_contract, lhs_batch, rhs, rhs_contract, rhs_batch, in_dtype: int,
                acc_dtype: int = 0, out_dtype: int = 0, acc_f64: bool = False) -> np.ndarray:
    lhs = _c(lhs, _NP_OF[in_dtype])
    rhs = _c(rhs, _NP_OF[in_dtype])
    od = out_dtype or in_dtype
    dims = dot_output_dims(list(lhs.shape), list(lhs_contract), list(lhs_batch),
                           list(rhs.shape), list(rhs_contract), list(rhs_batch))
    out = np.empty(dims, _NP_OF[od])
    ld = np.array(lhs.shape, np.int64)
    rd = np.array(rhs.shape, np.int64)
    lc = np.array(list(lhs_contract), np.int32)
    lb = np.array(list(lhs_batch), np.int32)
    rc = np.array(list(rhs_contract), np.int32)
    rb = np.array(list(rhs_batch), np.int32)
    rcode = lib().orc_dot_general(in_dtype, _p(lhs), lhs.ndim, _p(ld), _p(lc), _p(lb),
                                  _p(rhs), rhs.ndim, _p(rd), _p(rc), _p(rb),
                                  len(lc), len(lb), acc_dtype, od, _p(out), int(acc_f64))
    if rcode != 0:
        raise ValueError(f"orc_dot_general failed: {rcode}")
    return out


def gemm_f32_blocked(a, b, threads: int) -> np.ndarray:
    a = _c(a, np.float32)
    b = _c(b, np.float32)
    out = np.empty((a.shape[0], b.shape[1]), np.float32)
    lib(True).orc_gemm_f32_blocked(_p(a), _p(b), _p(out), a.shape[0], a.shape[1], b.shape[1], threads)
    return out


# ---------------------------------------------------------------- SDPA
def sdpa(q, k, v, mask=None, bias=None, q_len=None, kv_len=None, layout: str = "BHSD",
         scale: float = 0.0, causal: bool = False, fast: bool = False) -> np.ndarray:
    """Reference fused SDPA on float32 (sdpa.go:373-636)."""
    q = _c(q, np.float32)
    k = _c(k, np.float32)
    v = _c(v, np.float32)
    bshd = int(layout == "BSHD")
    if bshd:
        B, S, Hq, D = q.shape
        Skv, Hkv = k.shape[1], k.shape[2]
    else:
        B, Hq, S, D = q.shape
        Hkv, Skv = k.shape[1], k.shape[2]
    m = md = None
    mbool = 0
    if mask is not None:
        mask = np.asarray(mask)
        if bshd and mask.ndim == 4:       # sdpa.go:259-274: [B,S,H,Skv] -> [B,H,S,Skv]
            mask = mask.transpose(0, 2, 1, 3)
        mbool = int(mask.dtype == np.bool_)
        m = np.ascontiguousarray(mask, np.uint8 if mbool else np.float32)
        md = np.array(m.shape, np.int64)
    bs = bd = None
    if bias is not None:
        bias = np.asarray(bias, np.float32)
        if bshd and bias.ndim == 4:
            bias = bias.transpose(0, 2, 1, 3)
        bs = np.ascontiguousarray(bias)
        bd = np.array(bs.shape, np.int64)
    ql = None if q_len is None else _c(q_len, np.int32)
    kl = None if kv_len is None else _c(kv_len, np.int32)
    out = np.empty_like(q)
    lib(fast).orc_sdpa_f32(_p(q), _p(k), _p(v), _p(m), mbool, 0 if m is None else m.ndim, _p(md),
                           _p(bs), 0 if bs is None else bs.ndim, _p(bd), _p(ql), _p(kl), _p(out),
                           B, Hq, Hkv, S, Skv, D, bshd, float(scale), int(causal))
    return out


def sdpa_slice(q, k, v, b0, b1, h0, h1, layout="BHSD", scale=0.0, causal=False) -> np.ndarray:
    """Only batches [b0,b1) and kv heads [h0,h1) are computed (others left zero)."""
    q = _c(q, np.float32)
    k = _c(k, np.float32)
    v = _c(v, np.float32)
    bshd = int(layout == "BSHD")
    if bshd:
        B, S, Hq, D = q.shape
        Skv, Hkv = k.shape[1], k.shape[2]
    else:
        B, Hq, S, D = q.shape
        Hkv, Skv = k.shape[1], k.shape[2]
    out = np.zeros_like(q)
    lib(True).orc_sdpa_f32_slice(_p(q), _p(k), _p(v), _p(out), B, Hq, Hkv, S, Skv, D, bshd,
                                 float(scale), int(causal), b0, b1, h0, h1)
    return out


# ---------------------------------------------------------------- FusedDense
def activation_f32(y: np.ndarray, activation: int) -> np.ndarray:
    """fusedDenseApplyActivation on float32 data (dense.go:176-205), a copy is returned."""
    out = np.array(y, np.float32, copy=True, order="C")
    lib().orc_activation_f32(_p(out), out.size, activation)
    return out


def fused_dense(x, weight, bias=None, activation: int = ACT_NONE, outputs_input: bool = False, in_dtype: int = F32) -> np.ndarray:
    """Reference FusedDense (fusedops/dense.go:34-163): DotGeneral contracting x's last axis with the weight's
    first axis (or its last, `outputs_input`), bias added per flat out-feature index (`i % outFeatures`,
    dense.go:166-174), then the activation; float32 and float64 as in the reference."""
    assert in_dtype in (F32, F64)
    x = _c(x, _NP_OF[in_dtype])
    weight = _c(weight, _NP_OF[in_dtype])
    y = dot_general(x, [x.ndim - 1], [], weight, [weight.ndim - 1 if outputs_input else 0], [], in_dtype)
    if bias is not None:
        b = _c(bias, _NP_OF[in_dtype]).reshape(-1)
        y = (y.reshape(-1, b.size) + b[None, :]).astype(_NP_OF[in_dtype]).reshape(y.shape)
    if in_dtype == F32:
        return activation_f32(y, activation).reshape(y.shape)
    return activation_f64(y, activation)


# ---------------------------------------------------------------- FusedSoftmax / FusedGelu / FusedLayerNorm
def _fp(a):
    a = np.ascontiguousarray(a)
    if a.dtype not in (np.float32, np.float64):
        a = a.astype(np.float32)
    return a, ("f32" if a.dtype == np.float32 else "f64")


def softmax(x, axis: int) -> np.ndarray:
    """Reference FusedSoftmax (softmax.go:83-118) along one non-negative axis."""
    x, suf = _fp(x)
    outer = int(np.prod(x.shape[:axis], dtype=np.int64))
    inner = int(np.prod(x.shape[axis + 1:], dtype=np.int64))
    y = np.empty_like(x)
    fn = getattr(lib(), "orc_softmax_" + suf)
    fn.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64]
    fn(_p(x), _p(y), outer, x.shape[axis], inner)
    return y


def gelu(x, exact: bool = True) -> np.ndarray:
    """Reference FusedGelu (gelu.go:113-126)."""
    x, suf = _fp(x)
    y = np.empty_like(x)
    fn = getattr(lib(), "orc_gelu_" + suf)
    fn.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_int]
    fn(_p(x), _p(y), x.size, int(exact))
    return y


def layer_norm(x, axes, epsilon: float, gamma=None, beta=None) -> np.ndarray:
    """Reference FusedLayerNorm (layernorm.go:96-246): axes (negative = from the end) are moved to the end in
    the order given, each row normalised, and the result moved back; gamma / beta are indexed by the flat
    position inside the normalised axes."""
    x, suf = _fp(x)
    rank = x.ndim
    norm = [a + rank if a < 0 else a for a in axes]
    perm = [a for a in range(rank) if a not in norm] + norm
    xt = np.ascontiguousarray(np.transpose(x, perm))
    L = int(np.prod([x.shape[a] for a in norm], dtype=np.int64))
    rows = xt.size // L if L else 0
    y = np.empty_like(xt)
    g = None if gamma is None else np.ascontiguousarray(gamma, x.dtype).reshape(-1)
    b = None if beta is None else np.ascontiguousarray(beta, x.dtype).reshape(-1)
    fn = getattr(lib(), "orc_layernorm_" + suf)
    fn.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_double]
    fn(_p(xt), _p(g), _p(b), _p(y), rows, L, float(epsilon))
    return np.ascontiguousarray(np.transpose(y, np.argsort(perm)))


def qkv_projection(x, w_qkv, bias_q, bias_k, bias_v, query_dim: int, key_value_dim: int, in_dtype: int = F32):
    """Reference FusedAttentionQKVProjection (attentionqkv.go:38-199): DotGeneral of x's last axis with wQKV's first,
    the three column ranges of the result, each plus its bias (in the dtype of x)."""
    x = _c(x, _NP_OF[in_dtype])
    y = dot_general(x, [x.ndim - 1], [], _c(w_qkv, _NP_OF[in_dtype]), [0], [], in_dtype)
    outs, first = [], 0
    for width, b in ((query_dim, bias_q), (key_value_dim, bias_k), (key_value_dim, bias_v)):
        part = np.ascontiguousarray(y[..., first:first + width])
        if b is not None:
            part = (part + _c(b, _NP_OF[in_dtype]).reshape(width)).astype(_NP_OF[in_dtype])
        outs.append(part)
        first += width
    return tuple(outs)


# ---------------------------------------------------------------- GGML block formats
# compute.GGMLQuantType (fused_ops.go:132-145): codes, bytes per block and values per block (:148-176)
GGML_Q4_0, GGML_Q8_0, GGML_IQ4_NL, GGML_Q4_K, GGML_Q6_K = 0, 1, 2, 5, 7
GGML_BLOCK_BYTES = {GGML_Q4_0: 18, GGML_Q8_0: 34, GGML_IQ4_NL: 18, GGML_Q4_K: 144, GGML_Q6_K: 210}
GGML_BLOCK_VALUES = {GGML_Q4_0: 32, GGML_Q8_0: 32, GGML_IQ4_NL: 32, GGML_Q4_K: 256, GGML_Q6_K: 256}
GGML_NAMES = {GGML_Q4_0: "q4_0", GGML_Q8_0: "q8_0", GGML_IQ4_NL: "iq4_nl", GGML_Q4_K: "q4_k", GGML_Q6_K: "q6_k"}
IQ4NL_TABLE = np.array([-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113], np.float32)   # fused_ops.go:127-130


def ggml_random_rows(rng, N: int, K: int, ggml_type: int) -> np.ndarray:
    """Test data: [N, bytesPerRow] native blocks with every quant / packed-scale byte random (all bit patterns are
    legal there) and the fp16 block scales drawn from U(0.001, 0.02)."""
    vpb, bb = GGML_BLOCK_VALUES[ggml_type], GGML_BLOCK_BYTES[ggml_type]
    assert K % vpb == 0
    nb = K // vpb
    out = rng.integers(0, 256, size=(N, nb, bb), dtype=np.int64).astype(np.uint8)
    def put_f16(offset):
        d = rng.uniform(0.001, 0.02, size=(N, nb)).astype(np.float16)
        out[..., offset:offset + 2] = d.view(np.uint16)[..., None].view(np.uint8).reshape(N, nb, 2)
    if ggml_type == GGML_Q6_K:
        put_f16(208)
    else:
        put_f16(0)
        if ggml_type == GGML_Q4_K:
            put_f16(2)
    return np.ascontiguousarray(out.reshape(N, nb * bb))


def ggml_dequant_rows_numpy(data: np.ndarray, ggml_type: int) -> np.ndarray:
    """A second, vectorised restatement of quantizeddense_ggml.go:157-302 (float32 arithmetic in the reference's
    order); tests hold it against the C one bit for bit."""
    data = np.ascontiguousarray(data, np.uint8)
    N, bpr = data.shape
    bb, vpb = GGML_BLOCK_BYTES[ggml_type], GGML_BLOCK_VALUES[ggml_type]
    blk = data.reshape(N, bpr // bb, bb)
    f16 = lambda o: np.ascontiguousarray(blk[..., o:o + 2]).view(np.float16)[..., 0].astype(np.float32)
    f32 = np.float32
    if ggml_type == GGML_Q8_0:
        vals = f16(0)[..., None] * blk[..., 2:].view(np.int8).astype(f32)
    elif ggml_type in (GGML_Q4_0, GGML_IQ4_NL):
        qs = blk[..., 2:]
        nib = np.concatenate([qs & 0xF, qs >> 4], axis=-1)
        q = nib.astype(f32) - f32(8) if ggml_type == GGML_Q4_0 else IQ4NL_TABLE[nib]
        vals = f16(0)[..., None] * q
    elif ggml_type == GGML_Q4_K:
        d, dmin, sc, qs = f16(0), f16(2), blk[..., 4:16].astype(np.int32), blk[..., 16:]
        scale = np.empty(blk.shape[:2] + (8,), np.int32)
        mn = np.empty_like(scale)
        for j in range(8):
            if j < 4:
                scale[..., j], mn[..., j] = sc[..., j] & 63, sc[..., j + 4] & 63
            else:
                scale[..., j] = (sc[..., j + 4] & 0xF) | ((sc[..., j - 4] >> 6) << 4)
                mn[..., j] = (sc[..., j + 4] >> 4) | ((sc[..., j] >> 6) << 4)
        dd = d[..., None] * scale.astype(f32)
        mm = dmin[..., None] * mn.astype(f32)
        q = qs.reshape(blk.shape[:2] + (4, 32))
        nib = np.stack([q & 0xF, q >> 4], axis=3).reshape(blk.shape[:2] + (8, 32)).astype(f32)     # sub-block j = 2 * chunk + half
        vals = (dd[..., None] * nib - mm[..., None]).reshape(blk.shape[:2] + (256,))
    else:
        ql = blk[..., 0:128].reshape(blk.shape[:2] + (2, 64)).astype(np.int32)
        qh = blk[..., 128:192].reshape(blk.shape[:2] + (2, 32)).astype(np.int32)
        sc = blk[..., 192:208].view(np.int8).reshape(blk.shape[:2] + (2, 8)).astype(f32)
        d = f16(208)
        lo, hi = ql[..., :32], ql[..., 32:]
        q = np.stack([(lo & 0xF) | ((qh & 3) << 4), (hi & 0xF) | (((qh >> 2) & 3) << 4),
                      (lo >> 4) | (((qh >> 4) & 3) << 4), (hi >> 4) | (((qh >> 6) & 3) << 4)], axis=3) - 32     # [N, nb, 2, 4, 32]
        ds = d[..., None, None] * sc                                                                           # [N, nb, 2, 8]
        scale = np.repeat(ds.reshape(blk.shape[:2] + (2, 4, 2)), 16, axis=-1)                                    # index 2 * quarter + l // 16
        vals = (scale * q.astype(f32)).reshape(blk.shape[:2] + (256,))
    return np.ascontiguousarray(vals.reshape(N, -1).astype(f32))


def ggml_quantize_rows(w: np.ndarray, ggml_type: int) -> np.ndarray:
    """Test data: float rows [N, K] -> native Q4_0 / Q8_0 blocks [N, bytesPerRow] (round-to-nearest block
    quantisation; only the layout matters to the tests, which compare against orc.qdense_ggml on the same bytes)."""
    w = np.asarray(w, np.float32)
    N, K = w.shape
    assert K % 32 == 0
    blocks = w.reshape(N, K // 32, 32)
    amax = np.abs(blocks).max(axis=2)
    out = np.zeros((N, K // 32, GGML_BLOCK_BYTES[ggml_type]), np.uint8)
    if ggml_type == GGML_Q8_0:
        d = (amax / 127.0).astype(np.float16)
        q = np.where(d[..., None] > 0, np.rint(blocks / np.maximum(d.astype(np.float32), 1e-30)[..., None]), 0).clip(-127, 127).astype(np.int8)
        out[..., 2:] = q.view(np.uint8)
    else:
        d = (amax / 7.0).astype(np.float16)
        q = (np.where(d[..., None] > 0, np.rint(blocks / np.maximum(d.astype(np.float32), 1e-30)[..., None]), 0).clip(-8, 7) + 8).astype(np.uint8)
        out[..., 2:] = q[..., :16] | (q[..., 16:] << 4)
    out[..., 0:2] = d.view(np.uint16)[..., None].view(np.uint8).reshape(N, K // 32, 2)
    return np.ascontiguousarray(out.reshape(N, -1))


def ggml_dequant_rows(data: np.ndarray, ggml_type: int) -> np.ndarray:
    data = np.ascontiguousarray(data, np.uint8)
    N, bpr = data.shape
    K = bpr // GGML_BLOCK_BYTES[ggml_type] * GGML_BLOCK_VALUES[ggml_type]
    out = np.empty((N, K), np.float32)
    fn = lib().orc_ggml_dequant_row
    fn.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_int]
    for n in range(N):
        fn(data[n].ctypes.data, out[n].ctypes.data, K, ggml_type)
    return out


def qdense_ggml(x, w_blocks, bias=None, ggml_type: int = GGML_Q8_0, activation: int = ACT_NONE) -> np.ndarray:
    """Reference FusedQuantizedDense, GGML scheme (quantizeddense_ggml.go:55-131)."""
    x = _c(x, np.float32)
    w_blocks = np.ascontiguousarray(w_blocks, np.uint8)
    N, bpr = w_blocks.shape
    K = bpr // GGML_BLOCK_BYTES[ggml_type] * GGML_BLOCK_VALUES[ggml_type]
    assert x.shape[-1] == K
    M = x.size // K if K else 0
    b = None if bias is None else _c(bias, np.float32)
    out = np.empty(x.shape[:-1] + (N,), np.float32)
    fn = lib().orc_qdense_ggml
    fn.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_int, C.c_int]
    fn(_p(x), _p(w_blocks), _p(b), _p(out), M, K, N, ggml_type, activation)
    return out


def embedding_lookup(table, indices, ggml_type: int) -> np.ndarray:
    """Reference QuantizedEmbeddingLookup (quantizeddense.go:250-321, 455-499): indices [..., 1] of any integer
    dtype -> float32 [..., K]; an index outside the table raises, as the reference returns an error."""
    table = np.ascontiguousarray(table, np.uint8)
    idx = np.ascontiguousarray(indices).astype(np.int64)
    assert idx.ndim >= 1 and idx.shape[-1] == 1
    vocab, bpr = table.shape
    K = bpr // GGML_BLOCK_BYTES[ggml_type] * GGML_BLOCK_VALUES[ggml_type]
    out = np.empty(idx.shape[:-1] + (K,), np.float32)
    fn = lib().orc_embedding_lookup
    fn.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_int]
    fn.restype = C.c_int64
    bad = fn(_p(table), _p(idx), _p(out), vocab, idx.size, K, ggml_type)
    if bad >= 0:
        raise IndexError(f"QuantizedEmbeddingLookup: index {int(idx.reshape(-1)[bad])} out of range [0, {vocab})")
    return out


# ---------------------------------------------------------------- decoder block (composition of the ops above)
def _bf(a: np.ndarray) -> np.ndarray:
    """Round float32 values to bfloat16 and back (what a bfloat16 graph stores between ops)."""
    return bf16_to_f32(bf16_from_f32(np.ascontiguousarray(a, np.float32)))


def rms_norm(x: np.ndarray, gamma: np.ndarray, eps: float) -> np.ndarray:
    x64 = np.asarray(x, np.float64)
    return (x64 / np.sqrt((x64 ** 2).mean(-1, keepdims=True) + eps) * np.asarray(gamma, np.float64)).astype(np.float32)


def decoder_block(x, weights, heads: int, kv_heads: int, head_dim: int, eps: float, cache_k=None, cache_v=None,
                  rows=None, threads: int = 1):
    """The Llama-style block of the fifth benchmark configuration from the reference's ops: RMS norm, int8 per-channel
    quantized dense (quantizeddense.go:616-650) for q / k / v / o / gate / up / down, fused SDPA (sdpa.go:373-636, BSHD,
    grouped KV heads), SwiGLU, residuals; every op's result is rounded to bfloat16, as a bfloat16 graph stores it.
    x: [B, S, H] float32 values.  Prefill (no cache): causal attention over the S tokens; with `rows` = list of (b, s)
    only those tokens' outputs are computed beyond the key / value projections (which all tokens need).  Decode:
    attention over cache_k / cache_v [B, Skv, kv_heads, head_dim].  Returns y (for `rows` when given), k, v."""
    B, S, H = x.shape
    qd = lambda a, name, act=ACT_NONE: _bf(qdense_linear(np.ascontiguousarray(a, np.float32).reshape(-1, a.shape[-1]), weights[name],
                                                         np.repeat(weights[name + "_scale"], weights[name].shape[0], axis=0), None, None, 1, act,
                                                         threads=threads, fast=True))
    g1, g2 = bf16_to_f32(weights["g1"]), bf16_to_f32(weights["g2"])
    h = _bf(rms_norm(x, g1, eps))
    k = qd(h, "wk").reshape(B, S, kv_heads, head_dim)
    v = qd(h, "wv").reshape(B, S, kv_heads, head_dim)
    if cache_k is not None:
        q = qd(h, "wq").reshape(B, S, heads, head_dim)
        att = _bf(sdpa(q, cache_k, cache_v, layout="BSHD", causal=False, fast=True))
        sel_x, sel_att = x.reshape(B * S, H), att.reshape(B * S, heads * head_dim)
    elif rows is None:
        q = qd(h, "wq").reshape(B, S, heads, head_dim)
        att = _bf(sdpa(q, k, v, layout="BSHD", causal=True, fast=True))
        sel_x, sel_att = x.reshape(B * S, H), att.reshape(B * S, heads * head_dim)
    else:
        sel_x = np.stack([x[b, s] for b, s in rows])
        hq = np.stack([h[b, s] for b, s in rows])
        q = qd(hq, "wq").reshape(len(rows), heads, head_dim)
        att = np.empty((len(rows), heads, head_dim), np.float32)
        for i, (b, s) in enumerate(rows):       # a token attends to the tokens up to itself: one query row per call
            att[i] = sdpa(q[i][None, None], k[b:b + 1, :s + 1], v[b:b + 1, :s + 1], layout="BSHD", causal=False, fast=True)[0, 0]
        sel_att = _bf(att).reshape(len(rows), heads * head_dim)
    o = qd(sel_att, "wo")
    x1 = _bf(sel_x + o)
    h2 = _bf(rms_norm(x1, g2, eps))
    gate = qd(h2, "wg", ACT_SILU)
    up = qd(h2, "wu")
    d = qd(_bf(gate * up), "wd")
    y = _bf(x1 + d)
    if rows is None:
        y = y.reshape(B, S, H)
    return y, k, v
