"""The Llama-style decoder block of the fifth benchmark configuration as ONE compiled Executable, against the oracle's
composition of the reference ops (every op's result rounded to bfloat16 on both sides).  bfloat16 tolerance 2e-2
(max-abs normalised), as for the single ops."""
import numpy as np
import pytest

from compute_b200 import backend as be, decoder_block as blk, device as dv
from oracle import oracle as orc
from tests.helpers import max_abs_normalised

pytestmark = pytest.mark.gpu
BF16_TOL = 2e-2


@pytest.fixture(scope="module")
def backend():
    b = be.New("")
    yield b
    b.Finalize()


def run_block(backend, cfg, weights, x_bits, cache=None):
    B, S, _ = x_bits.shape
    kv_len = cache[0].shape[1] if cache else 0
    exe, names = blk.compile_block(backend, cfg, B, S, kv_len)
    host = dict(weights)
    host["x"] = x_bits
    if cache:
        host["cache_k"], host["cache_v"] = cache
    bufs = [backend.BufferFromFlatData(0, host[n], blk.parameter_shape(n, cfg, B, S, kv_len)) for n in names]
    outs = exe.Execute(bufs, None, 0)
    res = [o.ToNumpy() for o in outs]
    kernels = exe.KernelNames()
    for b in bufs + outs:
        b.Finalize()
    exe.Finalize()
    return res, kernels


def test_small_block_prefill_and_decode(backend):
    cfg = blk.BlockConfig(hidden=512, heads=4, kv_heads=2, head_dim=128, mlp=1792)
    w = blk.make_block_weights(cfg, 3)
    rng = np.random.default_rng(1)
    # prefill: 2 sequences of 128 tokens
    xb = orc.bf16_from_f32(rng.standard_normal((2, 128, cfg.hidden), dtype=np.float32))
    (y,), kernels = run_block(backend, cfg, w, xb)
    assert sum(k.startswith("rms_norm_") for k in kernels) == 2 and not any(k.startswith("reduce_") for k in kernels), kernels
    assert any(k.startswith("sdpa_flash") for k in kernels), kernels
    want, _, _ = orc.decoder_block(orc.bf16_to_f32(xb), w, cfg.heads, cfg.kv_heads, cfg.head_dim, cfg.eps, threads=orc.max_threads())
    assert max_abs_normalised(orc.bf16_to_f32(y), want) < BF16_TOL
    # decode: 16 sequences, one new token each, attention over a cache of 256 positions
    xd = orc.bf16_from_f32(rng.standard_normal((16, 1, cfg.hidden), dtype=np.float32))
    ck = orc.bf16_from_f32(rng.standard_normal((16, 256, cfg.kv_heads, cfg.head_dim), dtype=np.float32))
    cv = orc.bf16_from_f32(rng.standard_normal((16, 256, cfg.kv_heads, cfg.head_dim), dtype=np.float32))
    (y, k, v), kernels = run_block(backend, cfg, w, xd, (ck, cv))
    # q / k / v and gate / up are single grouped launches; o and down run alone
    assert sum(k_.startswith("qdense_decode_tc_") for k_ in kernels) == 4, kernels
    assert any(k_.endswith("_x3") for k_ in kernels) and any(k_.endswith("_x2") for k_ in kernels), kernels
    want, kw, vw = orc.decoder_block(orc.bf16_to_f32(xd), w, cfg.heads, cfg.kv_heads, cfg.head_dim, cfg.eps,
                                     cache_k=orc.bf16_to_f32(ck), cache_v=orc.bf16_to_f32(cv), threads=orc.max_threads())
    assert max_abs_normalised(orc.bf16_to_f32(y), want) < BF16_TOL
    assert max_abs_normalised(orc.bf16_to_f32(k).reshape(kw.shape), kw) < BF16_TOL
    assert max_abs_normalised(orc.bf16_to_f32(v).reshape(vw.shape), vw) < BF16_TOL


def test_full_size_decode_block(backend):
    """Hidden 4096, 32 / 8 heads of 128, MLP 14336; 16 sequences x 1 token over a cache of 2048 positions."""
    cfg = blk.BlockConfig()
    w = blk.make_block_weights(cfg, 5)
    rng = np.random.default_rng(2)
    xd = orc.bf16_from_f32(rng.standard_normal((16, 1, cfg.hidden), dtype=np.float32))
    ck = orc.bf16_from_f32(rng.standard_normal((16, 2048, cfg.kv_heads, cfg.head_dim), dtype=np.float32))
    cv = orc.bf16_from_f32(rng.standard_normal((16, 2048, cfg.kv_heads, cfg.head_dim), dtype=np.float32))
    (y, k, v), kernels = run_block(backend, cfg, w, xd, (ck, cv))
    want, kw, vw = orc.decoder_block(orc.bf16_to_f32(xd), w, cfg.heads, cfg.kv_heads, cfg.head_dim, cfg.eps,
                                     cache_k=orc.bf16_to_f32(ck), cache_v=orc.bf16_to_f32(cv), threads=orc.max_threads())
    assert max_abs_normalised(orc.bf16_to_f32(y), want) < BF16_TOL
    assert max_abs_normalised(orc.bf16_to_f32(k).reshape(kw.shape), kw) < BF16_TOL


def test_full_size_prefill_block_sampled_tokens(backend):
    """4 sequences x 512 tokens at full size; the oracle computes the key / value projections of every token and the
    rest of the block for a sample of tokens (first, last, tile edges of the attention kernel)."""
    cfg = blk.BlockConfig()
    w = blk.make_block_weights(cfg, 6)
    rng = np.random.default_rng(3)
    xb = orc.bf16_from_f32(rng.standard_normal((4, 512, cfg.hidden), dtype=np.float32))
    (y,), kernels = run_block(backend, cfg, w, xb)
    assert any(k.startswith("sdpa_flash") for k in kernels) and any(k.startswith("qdense_prefill") for k in kernels), kernels
    rows = [(0, 0), (0, 127), (1, 128), (2, 300), (3, 511)]
    want, _, _ = orc.decoder_block(orc.bf16_to_f32(xb), w, cfg.heads, cfg.kv_heads, cfg.head_dim, cfg.eps, rows=rows, threads=orc.max_threads())
    got = np.stack([orc.bf16_to_f32(y)[b, s] for b, s in rows])
    assert max_abs_normalised(got, want) < BF16_TOL
