"""Immediate-mode helpers: run one op of the hot path on host arrays through the C ABI.

Each call uploads its numpy inputs, launches the planned kernel and downloads the
result — convenient for tests and small jobs.  Long-running callers keep buffers
resident and launch plans themselves (see compute_b200.device.Plan).
Half-precision arrays are uint16 bit patterns plus an explicit dtype code.
"""
from __future__ import annotations

from typing import Optional

import numpy as np

from . import device as dv
from ._lib import BackendError, ERR_INVALID_ARG


def _run(plan: dv.Plan, host_inputs, out_shape, out_np_dtype, dev: int = 0) -> np.ndarray:
    bufs = [dv.DeviceMem.from_numpy(a, dev) for a in host_inputs]
    out_nbytes = int(np.prod(out_shape)) * np.dtype(out_np_dtype).itemsize
    out = dv.DeviceMem(out_nbytes, dev)
    ws = plan.new_workspace()
    try:
        plan.launch([b.ptr for b in bufs], [out.ptr], ws.ptr if ws else None)
        dv.check(dv._lib.load().cb_stream_sync(dev, None))
        plan.check_status(ws.ptr if ws else None)
        return out.download(out_shape, out_np_dtype)
    finally:
        for b in bufs:
            b.free()
        out.free()
        if ws:
            ws.free()


def quantized_dense(x: np.ndarray, w: np.ndarray, scales: np.ndarray, zero_points: Optional[np.ndarray] = None,
                    bias: Optional[np.ndarray] = None, *, x_dtype: int = dv.F32, scale_layout: int = dv.SCALE_REF,
                    block_size: int = 1, activation: int = dv.ACT_NONE, variant: int = dv.QDENSE_AUTO,
                    dev: int = 0, return_plan: bool = False, scheme: int = dv.QUANT_LINEAR,
                    packed: Optional[tuple] = None):
    """y = act(x @ dequant(w) + bias).  x: [..., K] f32 (or bf16 bits with x_dtype=BF16);
    w: [K, N] int8/uint8; scales per `scale_layout`; bias [N] f32.  Packed 4-bit weights:
    `packed=(dv.I4 or dv.U4, N)` and `w` the uint8 bytes of the K*N elements, two per byte, low
    nibble first.  `scheme=dv.QUANT_NF4`: the low nibble of every element indexes the NF4 table."""
    x = np.ascontiguousarray(x, dv.NP_CARRIER[x_dtype])
    w = np.ascontiguousarray(w)
    if x.ndim < 1:
        raise BackendError(ERR_INVALID_ARG, f"FusedQuantizedDense: x must have rank >= 1, got {x.ndim}")
    K = x.shape[-1]
    if packed is not None:
        w_code, N = packed
        if w_code not in (dv.I4, dv.U4) or w.dtype != np.uint8 or w.size != (K * N + 1) // 2:
            raise BackendError(ERR_INVALID_ARG, f"FusedQuantizedDense: packed weights must be {(K * N + 1) // 2} uint8 bytes, got {w.dtype} {w.shape}")
    else:
        if w.dtype not in (np.int8, np.uint8) or w.ndim != 2:
            raise BackendError(ERR_INVALID_ARG, f"FusedQuantizedDense: weights must be [K, N] int8/uint8, got {w.dtype} {w.shape}")
        if w.shape[0] != K:
            raise BackendError(ERR_INVALID_ARG, f"FusedQuantizedDense: weights must be [{K}, N], got {list(w.shape)}")
        N = w.shape[1]
        w_code = dv.U8 if w.dtype == np.uint8 else dv.I8
    M = x.size // K if K else 0
    scales = np.ascontiguousarray(scales, np.float32)
    want = {dv.SCALE_REF: (K, -(-N // max(block_size, 1))), dv.SCALE_CHANNEL: (N,),
            dv.SCALE_KGROUP: (-(-K // max(block_size, 1)), N)}[scale_layout]
    if scales.shape != want:
        raise BackendError(ERR_INVALID_ARG, f"FusedQuantizedDense: scales must be {list(want)}, got {list(scales.shape)}")
    ins = [x, w, scales]
    if zero_points is not None:
        zp = np.ascontiguousarray(zero_points, np.float32)
        if zp.shape != want:
            raise BackendError(ERR_INVALID_ARG, f"FusedQuantizedDense: zero points must be {list(want)}")
        ins.append(zp)
    if bias is not None:
        b = np.ascontiguousarray(bias, np.float32)
        if b.shape != (N,):
            raise BackendError(ERR_INVALID_ARG, f"FusedQuantizedDense: bias must be [{N}], got {list(b.shape)}")
        ins.append(b)
    plan = dv.Plan.qdense(M, K, N, x_dtype, w_code, scale_layout, block_size,
                          zero_points is not None, bias is not None, activation, variant, dev, scheme=scheme)
    out = _run(plan, ins, x.shape[:-1] + (N,), dv.NP_CARRIER[x_dtype], dev)
    return (out, plan) if return_plan else out


def dot_normalised(lhs: np.ndarray, rhs: np.ndarray, *, in_dtype: int, out_dtype: int = dv.INVALID,
                   rhs_transposed: bool = False, variant: int = dv.DOT_AUTO, dev: int = 0, return_plan: bool = False,
                   bias: Optional[np.ndarray] = None, activation: int = dv.ACT_NONE):
    """out[B,M,N] = lhs[B,M,K] x rhs[B,K,N] (or rhs[B,N,K] when rhs_transposed); with `bias` [N] (of the input
    dtype) and / or `activation` the plan is FusedDense: act(dot + bias)."""
    lhs = np.ascontiguousarray(lhs, dv.NP_CARRIER[in_dtype])
    rhs = np.ascontiguousarray(rhs, dv.NP_CARRIER[in_dtype])
    B, M, K = lhs.shape
    N = rhs.shape[1] if rhs_transposed else rhs.shape[2]
    od = out_dtype or in_dtype
    plan = dv.Plan.dot(B, M, N, K, in_dtype, out_dtype, rhs_transposed, variant, dev, has_bias=bias is not None, activation=activation)
    ins = [lhs, rhs]
    if bias is not None:
        ins.append(np.ascontiguousarray(bias, dv.NP_CARRIER[in_dtype]).reshape(N))
    out = _run(plan, ins, (B, M, N), dv.NP_CARRIER[od], dev)
    return (out, plan) if return_plan else out


def sdpa(q: np.ndarray, k: np.ndarray, v: np.ndarray, *, dtype: int = dv.F32, layout: int = dv.LAYOUT_BHSD,
         scale: float = 0.0, causal: bool = False, mask: Optional[np.ndarray] = None,
         q_len: Optional[np.ndarray] = None, kv_len: Optional[np.ndarray] = None,
         bias: Optional[np.ndarray] = None, variant: int = dv.SDPA_AUTO, dev: int = 0, return_plan: bool = False):
    """Fused scaled-dot-product attention; inputs in the reference's node-input order."""
    carrier = dv.NP_CARRIER[dtype]
    q, k, v = (np.ascontiguousarray(a, carrier) for a in (q, k, v))
    if q.ndim != 4 or k.ndim != 4:
        raise BackendError(ERR_INVALID_ARG, f"FusedScaledDotProductAttention: query and key must have rank 4, got {q.ndim}, {k.ndim}")
    if layout == dv.LAYOUT_BSHD:
        B, S, Hq, D = q.shape
        Skv, Hkv = k.shape[1], k.shape[2]
    else:
        B, Hq, S, D = q.shape
        Hkv, Skv = k.shape[1], k.shape[2]
    ins = [q, k, v]
    mask_kind, mask_dims = dv.MASK_NONE, ()
    if mask is not None:
        mask = np.asarray(mask)
        if mask.dtype == np.bool_:
            mask_kind = dv.MASK_BOOL
            ins.append(np.ascontiguousarray(mask, np.uint8))
        else:
            mask_kind = dv.MASK_ADDITIVE
            ins.append(np.ascontiguousarray(mask, carrier))
        mask_dims = mask.shape
    if (q_len is None) != (kv_len is None):
        raise BackendError(ERR_INVALID_ARG, "FusedScaledDotProductAttention: QuerySeqLen and KeyValueSeqLen must both be set or both nil")
    if q_len is not None:
        for name, a in (("QuerySeqLen", q_len), ("KeyValueSeqLen", kv_len)):
            a = np.asarray(a)
            if a.dtype != np.int32 or a.shape != (B,):
                raise BackendError(ERR_INVALID_ARG, f"FusedScaledDotProductAttention: {name} must be int32 with length batch ({B}), got {a.dtype} {a.shape}")
            ins.append(np.ascontiguousarray(a))
    bias_dims = ()
    if bias is not None:
        bias = np.ascontiguousarray(bias, carrier)
        bias_dims = bias.shape
        ins.append(bias)
    plan = dv.Plan.sdpa(B, Hq, Hkv, S, Skv, D, dtype, layout, scale, causal, mask_kind, mask_dims,
                        q_len is not None, bias_dims, variant, dev)
    out = _run(plan, ins, q.shape, carrier, dev)
    return (out, plan) if return_plan else out


def softmax(x: np.ndarray, axis: int, *, dtype: int = dv.F32, dev: int = 0) -> np.ndarray:
    """FusedSoftmax along one non-negative axis; x in the numpy carrier of `dtype`."""
    x = np.ascontiguousarray(x, dv.NP_CARRIER[dtype])
    if axis < 0 or axis >= x.ndim:
        raise BackendError(ERR_INVALID_ARG, f"FusedSoftmax: axis {axis} out of range for rank {x.ndim}")
    outer = int(np.prod(x.shape[:axis], dtype=np.int64))
    inner = int(np.prod(x.shape[axis + 1:], dtype=np.int64))
    return _run(dv.Plan.softmax(dtype, outer, x.shape[axis], inner, dev), [x], x.shape, dv.NP_CARRIER[dtype], dev)


def gelu(x: np.ndarray, exact: bool = True, *, dtype: int = dv.F32, dev: int = 0) -> np.ndarray:
    """FusedGelu (erf form, or the tanh approximation)."""
    x = np.ascontiguousarray(x, dv.NP_CARRIER[dtype])
    return _run(dv.Plan.gelu(dtype, x.size, exact, dev), [x], x.shape, dv.NP_CARRIER[dtype], dev)


def layer_norm_rows(x: np.ndarray, epsilon: float, gamma: Optional[np.ndarray] = None, beta: Optional[np.ndarray] = None, *,
                    dtype: int = dv.F32, dev: int = 0) -> np.ndarray:
    """FusedLayerNorm over the last axis of a 2-D x (other axis sets are transposed by the graph layer)."""
    x = np.ascontiguousarray(x, dv.NP_CARRIER[dtype])
    rows, L = x.shape
    ins = [x] + [np.ascontiguousarray(a, dv.NP_CARRIER[dtype]).reshape(L) for a in (gamma, beta) if a is not None]
    plan = dv.Plan.layernorm(dtype, rows, L, epsilon, gamma is not None, beta is not None, dev)
    return _run(plan, ins, x.shape, dv.NP_CARRIER[dtype], dev)
