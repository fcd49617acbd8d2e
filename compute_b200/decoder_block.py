"""A Llama-style decoder block written against the Backend interface (the fifth benchmark configuration): RMS norm
in its decomposed form, int8 per-output-channel FusedQuantizedDense for every projection, fused scaled-dot-product
attention with grouped KV heads (no rotary embedding), SwiGLU, residual additions — what a model layer built on
gomlx/compute's Function API emits (fused_ops.go:349-378, :413-435; standard_ops.go Mul / Add / ReduceSum / Rsqrt).
Builder.Compile turns the two RMS norms into row kernels and groups the independent projections (q / k / v, gate / up)
into single launches when the batch is decode-shaped.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Tuple

import numpy as np

from . import backend as be, device as dv


@dataclass(frozen=True)
class BlockConfig:
    hidden: int = 4096
    heads: int = 32
    kv_heads: int = 8
    head_dim: int = 128
    mlp: int = 14336
    eps: float = 1e-5

    @property
    def q_dim(self) -> int:
        return self.heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.kv_heads * self.head_dim


PROJECTIONS = ("wq", "wk", "wv", "wo", "wg", "wu", "wd")


def projection_shapes(cfg: BlockConfig) -> Dict[str, Tuple[int, int]]:
    return {"wq": (cfg.hidden, cfg.q_dim), "wk": (cfg.hidden, cfg.kv_dim), "wv": (cfg.hidden, cfg.kv_dim),
            "wo": (cfg.q_dim, cfg.hidden), "wg": (cfg.hidden, cfg.mlp), "wu": (cfg.hidden, cfg.mlp), "wd": (cfg.mlp, cfg.hidden)}


def bf16_bits(a: np.ndarray) -> np.ndarray:
    b = np.ascontiguousarray(a, np.float32).view(np.uint32)
    return ((b + 0x7FFF + ((b >> 16) & 1)) >> 16).astype(np.uint16)


def make_block_weights(cfg: BlockConfig, seed: int = 0) -> Dict[str, np.ndarray]:
    """Random-init weights ~ N(0, 0.02) quantised to int8 with one scale per output channel (max |w| / 127), and the
    two RMS-norm gains as bfloat16 bit patterns."""
    rng = np.random.default_rng(seed)
    out: Dict[str, np.ndarray] = {}
    for name, (k, n) in projection_shapes(cfg).items():
        # int8 values drawn directly: round(N(0, 0.02) / s) with s = 4 sigma / 127 is N(0, 127/4) clipped
        w = np.clip(np.rint(rng.standard_normal((k, n), dtype=np.float32) * np.float32(127.0 / 4.0)), -127, 127).astype(np.int8)
        out[name] = w
        out[name + "_scale"] = np.full((1, n), 0.02 * 4.0 / 127.0, np.float32) * rng.uniform(0.9, 1.1, size=(1, n)).astype(np.float32)
    out["g1"] = bf16_bits(1.0 + 0.1 * rng.standard_normal(cfg.hidden).astype(np.float32))
    out["g2"] = bf16_bits(1.0 + 0.1 * rng.standard_normal(cfg.hidden).astype(np.float32))
    return out


def _rms_norm(f: be.Function, x: be.Value, gamma: be.Value, cfg: BlockConfig, lead: List[int]) -> be.Value:
    """x * Reshape(Rsqrt(ReduceSum(x*x, -1) * (1/H) + eps)) * gamma — the decomposed form (the interface has no fused one)."""
    H = cfg.hidden
    c = lambda v: f.Constant(bf16_bits(np.float32([v])), dtype=dv.BF16)
    ss = f.ReduceSum(f.Mul(x, x), -1)
    r = f.Rsqrt(f.Add(f.Mul(ss, c(1.0 / H)), c(cfg.eps)))
    xn = f.Mul(x, f.Reshape(r, *(lead + [1])))
    return f.Mul(xn, f.Reshape(gamma, *([1] * len(lead) + [H])))


def _qd(f: be.Function, x: be.Value, w: be.Value, s: be.Value, k: int, act: int = dv.ACT_NONE) -> be.Value:
    # one scale per output channel: blocks along the input-features axis spanning all of K
    return f.FusedQuantizedDense(x, w, None, be.Quantization(be.QUANT_LINEAR, s, None, BlockAxis=0, BlockSize=k), act)


def build_block(f: be.Function, cfg: BlockConfig, batch: int, seq: int, kv_len: int = 0):
    """Adds the block to `f`.  Prefill (kv_len == 0): causal attention over the `seq` tokens themselves.  Decode
    (kv_len > 0, seq == 1): attention of the new token over a key / value cache of kv_len positions given as
    parameters [batch, kv_len, kv_heads, head_dim]; the new token's key and value projections are returned for the
    caller to store.  Returns (parameter names in Execute order, outputs)."""
    H, D = cfg.hidden, cfg.head_dim
    shapes = projection_shapes(cfg)
    names = ["x"]
    x = f.Parameter("x", be.make_shape(dv.BF16, batch, seq, H))
    p: Dict[str, be.Value] = {}
    for n in PROJECTIONS:
        k, nn = shapes[n]
        p[n] = f.Parameter(n, be.make_shape(dv.I8, k, nn))
        p[n + "_scale"] = f.Parameter(n + "_scale", be.make_shape(dv.F32, 1, nn))
        names += [n, n + "_scale"]
    for n in ("g1", "g2"):
        p[n] = f.Parameter(n, be.make_shape(dv.BF16, H))
        names.append(n)
    cache_k = cache_v = None
    if kv_len:
        cache_k = f.Parameter("cache_k", be.make_shape(dv.BF16, batch, kv_len, cfg.kv_heads, D))
        cache_v = f.Parameter("cache_v", be.make_shape(dv.BF16, batch, kv_len, cfg.kv_heads, D))
        names += ["cache_k", "cache_v"]
    h = _rms_norm(f, x, p["g1"], cfg, [batch, seq])
    q = _qd(f, h, p["wq"], p["wq_scale"], H)
    k = _qd(f, h, p["wk"], p["wk_scale"], H)
    v = _qd(f, h, p["wv"], p["wv_scale"], H)
    q4 = f.Reshape(q, batch, seq, cfg.heads, D)
    if kv_len:
        att, _ = f.FusedScaledDotProductAttention(q4, cache_k, cache_v, be.LAYOUT_BSHD, be.ScaledDotProductAttentionConfig(Causal=False))
    else:
        att, _ = f.FusedScaledDotProductAttention(q4, f.Reshape(k, batch, seq, cfg.kv_heads, D), f.Reshape(v, batch, seq, cfg.kv_heads, D),
                                                  be.LAYOUT_BSHD, be.ScaledDotProductAttentionConfig(Causal=True))
    o = _qd(f, f.Reshape(att, batch, seq, cfg.q_dim), p["wo"], p["wo_scale"], cfg.q_dim)
    x1 = f.Add(x, o)
    h2 = _rms_norm(f, x1, p["g2"], cfg, [batch, seq])
    gate = _qd(f, h2, p["wg"], p["wg_scale"], H, dv.ACT_SILU)
    up = _qd(f, h2, p["wu"], p["wu_scale"], H)
    d = _qd(f, f.Mul(gate, up), p["wd"], p["wd_scale"], cfg.mlp)
    y = f.Add(x1, d)
    outs = [y, k, v] if kv_len else [y]
    return names, outs


def compile_block(backend: be.Backend, cfg: BlockConfig, batch: int, seq: int, kv_len: int = 0):
    builder = backend.Builder("decoder-block-" + ("decode" if kv_len else "prefill"))
    f = builder.Main()
    names, outs = build_block(f, cfg, batch, seq, kv_len)
    f.Return(outs)
    return builder.Compile(), names


def parameter_shape(name: str, cfg: BlockConfig, batch: int, seq: int, kv_len: int) -> be.Shape:
    shapes = projection_shapes(cfg)
    if name == "x":
        return be.make_shape(dv.BF16, batch, seq, cfg.hidden)
    if name in ("g1", "g2"):
        return be.make_shape(dv.BF16, cfg.hidden)
    if name in ("cache_k", "cache_v"):
        return be.make_shape(dv.BF16, batch, kv_len, cfg.kv_heads, cfg.head_dim)
    if name.endswith("_scale"):
        return be.make_shape(dv.F32, 1, shapes[name[:-6]][1])
    return be.make_shape(dv.I8, *shapes[name])
