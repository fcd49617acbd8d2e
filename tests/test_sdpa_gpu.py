"""GPU parity of FusedScaledDotProductAttention: the reference's known-answer cases and
seeded comparisons against the CPU oracle, through the C ABI."""
import numpy as np
import pytest

from compute_b200 import BackendError, ErrNotImplemented, device as dv, ops
from oracle import oracle as orc
from tests.helpers import DT, as_f64, load_golden, max_abs_normalised, tensor

pytestmark = pytest.mark.gpu
G = load_golden("backendtest_sdpa.json")
LAYOUT = {"BHSD": dv.LAYOUT_BHSD, "BSHD": dv.LAYOUT_BSHD}


@pytest.mark.parametrize("variant", [dv.SDPA_GENERIC, dv.SDPA_AUTO])
@pytest.mark.parametrize("case", G["cases"], ids=[c["name"] for c in G["cases"]])
def test_sdpa_known_answers(case, variant):
    code = DT[case["dtype"]]
    t = lambda key: tensor(case[key], case["dtype"])
    mask = tensor(case["mask"], "bool") if "mask" in case else None
    bias = t("bias") if "bias" in case else None
    ql = np.array(case["q_len"], np.int32) if "q_len" in case else None
    kl = np.array(case["kv_len"], np.int32) if "kv_len" in case else None
    got = ops.sdpa(t("q"), t("k"), t("v"), dtype=code, layout=LAYOUT[case["layout"]], scale=case["scale"],
                   causal=case["causal"], mask=mask, q_len=ql, kv_len=kl, bias=bias, variant=variant)
    want = np.array(case["want"]["data"], np.float64).reshape(case["want"]["shape"])
    assert np.max(np.abs(as_f64(got, code) - want)) <= case["tol"]


@pytest.mark.parametrize("case", G["error_cases"], ids=[c["name"] for c in G["error_cases"]])
def test_sdpa_rejected_requests(case):
    q, k, v = (tensor(case[n], "f32") for n in ("q", "k", "v"))
    kwargs = dict(scale=1.0)
    if "bias" in case:
        kwargs["bias"] = tensor(case["bias"], "f32")
    if "q_len" in case:
        dt = np.int64 if case.get("seq_len_dtype") == "i64" else np.int32
        kwargs["q_len"] = np.array(case["q_len"], dt)
        kwargs["kv_len"] = np.array(case["kv_len"], dt)
    if case["error"] == "not_implemented":
        with pytest.raises(ErrNotImplemented):
            dv.Plan.sdpa(1, 1, 1, 2, 2, 1, dv.F8E4M3FN, causal=True, scale=1.0)
    else:
        with pytest.raises(BackendError) as e:
            ops.sdpa(q, k, v, **kwargs)
        assert not isinstance(e.value, ErrNotImplemented)


def random_case(seed, B, Hq, Hkv, S, Skv, D):
    rng = np.random.default_rng(seed)
    return (rng.standard_normal((B, Hq, S, D), dtype=np.float32),
            rng.standard_normal((B, Hkv, Skv, D), dtype=np.float32),
            rng.standard_normal((B, Hkv, Skv, D), dtype=np.float32), rng)


@pytest.mark.parametrize("layout", ["BHSD", "BSHD"])
@pytest.mark.parametrize("variant", [dv.SDPA_GENERIC, dv.SDPA_AUTO])
def test_sdpa_matches_oracle_f32(layout, variant):
    B, Hq, Hkv, S, Skv, D = 2, 6, 2, 37, 53, 24
    q, k, v, rng = random_case(3, B, Hq, Hkv, S, Skv, D)
    bias = rng.standard_normal((B, Hq, S, Skv), dtype=np.float32)
    bmask = rng.random((S, Skv)) > 0.3
    bmask[5, :] = False                      # an all-masked row must give zeros
    amask = np.where(rng.random((B, 1, S, Skv)) > 0.2, 0.0, -1e9).astype(np.float32)
    ql = np.array([S, 20], np.int32)
    kl = np.array([Skv - 3, 999], np.int32)
    tr = (lambda a: np.ascontiguousarray(a.transpose(0, 2, 1, 3))) if layout == "BSHD" else (lambda a: a)
    for kw in (dict(causal=True), dict(bias=bias), dict(mask=bmask, causal=True), dict(mask=amask, bias=bias),
               dict(q_len=ql, kv_len=kl, causal=True), dict(scale=0.37)):
        okw = dict(kw)
        gkw = dict(kw)
        for name in ("bias", "mask"):
            if name in kw and kw[name].ndim == 4:
                gkw[name] = tr(kw[name])
                okw[name] = tr(kw[name])
        want = orc.sdpa(tr(q), tr(k), tr(v), layout=layout, **okw)
        got = ops.sdpa(tr(q), tr(k), tr(v), dtype=dv.F32, layout=LAYOUT[layout], variant=variant, **gkw)
        assert max_abs_normalised(got, want) < 1e-4, kw.keys()
        if "mask" in kw and kw["mask"].dtype == np.bool_:
            row = got[:, :, 5, :] if layout == "BHSD" else got[:, 5, :, :]
            assert np.all(row == 0)


@pytest.mark.parametrize("dtype", ["bf16", "f16", "f64"])
def test_sdpa_other_dtypes(dtype):
    B, Hq, Hkv, S, Skv, D = 1, 4, 4, 19, 19, 16
    q, k, v, _ = random_case(5, B, Hq, Hkv, S, Skv, D)
    code = DT[dtype]
    if dtype == "f64":
        got = ops.sdpa(q.astype(np.float64), k.astype(np.float64), v.astype(np.float64), dtype=dv.F64, causal=True)
        want = orc.sdpa(q, k, v, causal=True)
        assert max_abs_normalised(got, want) < 1e-5
        return
    qh, kh, vh = (orc.from_f32(a, code) for a in (q, k, v))
    want = orc.sdpa(orc.to_f32(qh, code), orc.to_f32(kh, code), orc.to_f32(vh, code), causal=True)
    got = ops.sdpa(qh, kh, vh, dtype=code, causal=True)
    assert max_abs_normalised(orc.to_f32(got, code), want) < 2e-2


def test_sdpa_config4_slice():
    """B=8, 32 query / 8 kv heads, head_dim 128, seq 2048, bf16, causal: two (batch, kv head) groups of the
    full configuration against the oracle, the rest through a checksum identity (with V = ones every output
    element is exactly 1).  A sampled group is all four query heads of its KV head over all 2048 query
    positions: both head pairs that the causal kernel gives to one CTA (heads 4h, 4h+1 and 4h+2, 4h+3), and
    every 128-row query tile from the first (one key tile) to the last (sixteen).  The second group is the
    last batch entry and last KV head: the work items the persistent grid reaches last."""
    B, Hq, Hkv, S, D = 8, 32, 8, 2048, 128
    rng = np.random.default_rng(0x5EED0004)
    q = orc.bf16_from_f32(rng.standard_normal((B, Hq, S, D), dtype=np.float32))
    k = orc.bf16_from_f32(rng.standard_normal((B, Hkv, S, D), dtype=np.float32))
    v = orc.bf16_from_f32(rng.standard_normal((B, Hkv, S, D), dtype=np.float32))
    got = ops.sdpa(q, k, v, dtype=dv.BF16, causal=True)
    for b, h in ((3, 5), (B - 1, Hkv - 1)):
        qs = orc.bf16_to_f32(q[b:b + 1, 4 * h:4 * h + 4])
        want = orc.sdpa(qs, orc.bf16_to_f32(k[b:b + 1, h:h + 1]), orc.bf16_to_f32(v[b:b + 1, h:h + 1]), causal=True, fast=True)
        assert max_abs_normalised(orc.bf16_to_f32(got[b:b + 1, 4 * h:4 * h + 4]), want) < 2e-2
    ones = orc.bf16_from_f32(np.ones((B, Hkv, S, D), np.float32))
    got1 = orc.bf16_to_f32(ops.sdpa(q, k, ones, dtype=dv.BF16, causal=True))
    assert np.max(np.abs(got1 - 1.0)) < 2e-2


# ------------------------------------------------------------- tensor-core kernel on ragged shapes
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("B,Hq,Hkv,S,Skv,layout,dtype", [
    (2, 4, 2, 300, 300, "BHSD", "bf16"),      # even GQA group: causal CTAs pair two heads; rows and keys end inside a tile
    (1, 6, 2, 257, 257, "BHSD", "bf16"),      # group of three: one head per CTA
    (1, 2, 2, 128, 128, "BSHD", "f16"),       # no grouping, exactly one tile
    (1, 4, 1, 129, 200, "BHSD", "bf16"),      # more keys than queries
    (2, 8, 4, 384, 384, "BSHD", "bf16"),      # an odd number of 128-row tiles
])
def test_sdpa_flash_ragged_shapes(B, Hq, Hkv, S, Skv, layout, dtype, causal):
    D = 128
    code = DT[dtype]
    rng = np.random.default_rng(S + Hq)
    shp = (lambda h, s: (B, h, s, D)) if layout == "BHSD" else (lambda h, s: (B, s, h, D))
    q, k, v = (orc.from_f32(rng.standard_normal(shp(h, s), dtype=np.float32), code) for h, s in ((Hq, S), (Hkv, Skv), (Hkv, Skv)))
    got, plan = ops.sdpa(q, k, v, dtype=code, layout=dv.LAYOUT_BHSD if layout == "BHSD" else dv.LAYOUT_BSHD, causal=causal,
                         variant=dv.SDPA_FLASH, return_plan=True)
    assert plan.kernel_name.startswith("sdpa_flash_")
    want = orc.sdpa(orc.to_f32(q, code), orc.to_f32(k, code), orc.to_f32(v, code), layout=layout, causal=causal)
    assert max_abs_normalised(orc.to_f32(got, code), want) < 2e-2


@pytest.mark.parametrize("B,Hq,Hkv,S,D,layout,dtype,causal", [
    (6, 8, 2, 512, 128, "BSHD", "bf16", True),       # a padded prefill batch: every sequence with its own length
    (5, 4, 4, 300, 128, "BHSD", "f16", False),       # ragged S, no grouping, not causal
])
def test_sdpa_flash_kernel_with_sequence_lengths(B, Hq, Hkv, S, D, layout, dtype, causal):
    """QuerySeqLen / KeyValueSeqLen on the tensor-core kernel: lengths inside a key block, at a block boundary, the
    whole sequence, one key, none (zero rows); padded query positions are zero rows (sdpa.go:389-411, 471-474)."""
    rng = np.random.default_rng(B * 31 + S)
    code = DT[dtype]
    shape = (lambda h, s: (B, s, h, D)) if layout == "BSHD" else (lambda h, s: (B, h, s, D))
    q, k, v = (orc.from_f32(rng.standard_normal(shape(h, S), dtype=np.float32), code) for h in (Hq, Hkv, Hkv))
    lens = rng.integers(1, S + 1, size=B).astype(np.int32)
    lens[0], lens[1], lens[2], lens[3] = S, 1, 0, 128
    q_len = lens.copy()
    q_len[4] = max(1, int(lens[4]) // 2)              # fewer query positions than keys
    got, plan = ops.sdpa(q, k, v, dtype=code, layout=LAYOUT[layout], causal=causal, q_len=q_len, kv_len=lens, return_plan=True)
    assert plan.kernel_name.startswith("sdpa_flash_"), plan.kernel_name
    want = orc.sdpa(orc.to_f32(q, code), orc.to_f32(k, code), orc.to_f32(v, code), q_len=q_len, kv_len=lens, layout=layout, causal=causal)
    gotf = orc.to_f32(got, code)
    assert max_abs_normalised(gotf, want) < 2e-2
    assert np.all(gotf[want == 0.0] == 0.0)


# ------------------------------------------------------------- tiled CUDA-core kernel: float32, head_dim 32 / 64, masks, bias
TILE_CASES = [
    # B, Hq, Hkv, S, Skv, D, layout, dtype, causal, mask, bias, lens
    (4, 12, 12, 128, 128, 64, "BHSD", "f32", False, "pad", None, False),     # an encoder layer: padding mask [B, 1, S, Skv]
    (2, 8, 2, 100, 130, 64, "BSHD", "f32", True, None, None, False),         # ragged tiles, grouped heads, causal
    (2, 4, 4, 96, 200, 32, "BHSD", "f32", False, "full", "full", True),      # boolean mask, bias and lengths together
    (3, 6, 3, 64, 64, 128, "BSHD", "bf16", False, "additive", None, False),  # additive mask [S, Skv], bfloat16, head_dim 128
    (2, 4, 2, 40, 512, 64, "BHSD", "f16", True, None, "head", True),         # bias [1, H, S, Skv], float16, lengths
    (1, 2, 2, 33, 129, 64, "BHSD", "f32", False, "rows", None, False),       # some rows with every key masked: zero rows
]


@pytest.mark.parametrize("B,Hq,Hkv,S,Skv,D,layout,dtype,causal,mask_kind,bias_kind,lens", TILE_CASES)
def test_sdpa_tiled_kernel(B, Hq, Hkv, S, Skv, D, layout, dtype, causal, mask_kind, bias_kind, lens):
    rng = np.random.default_rng(B * 100 + S + Skv)
    code = DT[dtype]
    shape = (lambda h, s: (B, s, h, D)) if layout == "BSHD" else (lambda h, s: (B, h, s, D))
    q, k, v = (orc.from_f32(rng.standard_normal(shape(h, s), dtype=np.float32), code) for h, s in ((Hq, S), (Hkv, Skv), (Hkv, Skv)))
    mask = bias = q_len = kv_len = None
    if mask_kind == "pad":
        valid = rng.integers(Skv // 2, Skv + 1, size=B)
        # the reference's masks are whole [S, Skv] planes, broadcast over batch and heads only (sdpa.go:309-329)
        mask = np.ascontiguousarray(np.broadcast_to((np.arange(Skv)[None, :] < valid[:, None]).reshape(B, 1, 1, Skv), (B, 1, S, Skv)))
    elif mask_kind == "full":
        mask = rng.random((B, Hq, S, Skv)) < 0.8
        if layout == "BSHD":
            mask = np.ascontiguousarray(mask.transpose(0, 2, 1, 3))
    elif mask_kind == "additive":
        mask = orc.to_f32(orc.from_f32((rng.standard_normal((S, Skv)) * 2).astype(np.float32), code), code)
    elif mask_kind == "rows":
        mask = rng.random((S, Skv)) < 0.7
        mask[5] = False
        mask[32] = False
    if bias_kind == "full":
        bias = rng.standard_normal((B, Hq, S, Skv)).astype(np.float32)
        if layout == "BSHD":
            bias = np.ascontiguousarray(bias.transpose(0, 2, 1, 3))
    elif bias_kind == "head":
        bias = rng.standard_normal((1, Hq, S, Skv)).astype(np.float32)
    if bias is not None:
        bias = orc.to_f32(orc.from_f32(bias, code), code)
    if lens:
        kv_len = rng.integers(1, Skv + 1, size=B).astype(np.int32)
        q_len = rng.integers(1, S + 1, size=B).astype(np.int32)
        kv_len[0] = 0
    dev_mask = mask if mask is None or mask.dtype == np.bool_ else orc.from_f32(mask, code)
    dev_bias = None if bias is None else orc.from_f32(bias, code)
    got, plan = ops.sdpa(q, k, v, dtype=code, layout=LAYOUT[layout], causal=causal, mask=dev_mask, bias=dev_bias, q_len=q_len, kv_len=kv_len,
                         return_plan=True)
    assert plan.kernel_name == f"sdpa_tile_{ {'f32': 'Float32', 'bf16': 'BFloat16', 'f16': 'Float16'}[dtype] }", plan.kernel_name
    want = orc.sdpa(orc.to_f32(q, code), orc.to_f32(k, code), orc.to_f32(v, code), mask=mask, bias=bias, q_len=q_len, kv_len=kv_len,
                    layout=layout, causal=causal)
    gotf = orc.to_f32(got, code)
    assert max_abs_normalised(gotf, want) < (2e-5 if dtype == "f32" else 2e-2)
    assert np.all(gotf[want == 0.0] == 0.0)
    # the row kernel (the reference's order of summation) on the same case
    gen = ops.sdpa(q, k, v, dtype=code, layout=LAYOUT[layout], causal=causal, mask=dev_mask, bias=dev_bias, q_len=q_len, kv_len=kv_len,
                   variant=dv.SDPA_GENERIC)
    assert max_abs_normalised(gotf, orc.to_f32(gen, code)) < (2e-5 if dtype == "f32" else 2.0 ** -7)


@pytest.mark.parametrize("seed", range(16))
def test_sdpa_tiled_kernel_random_sweep(seed):
    """Seeded random shapes, head counts, layouts, dtypes, head dimensions and option combinations on the tiled kernel."""
    rng = np.random.default_rng(9000 + seed)
    dtype = ["f32", "f32", "bf16", "f16"][seed % 4]
    code = DT[dtype]
    D = [32, 64, 128][rng.integers(0, 3)]
    Hkv = int(rng.integers(1, 4))
    Hq = Hkv * int(rng.integers(1, 4))
    B = int(rng.integers(1, 4))
    S = int(rng.integers(16, 150))
    Skv = int(rng.integers(max(16, -(-4096 // S)), 300))
    layout = ["BHSD", "BSHD"][seed % 2]
    causal = bool(rng.integers(0, 2))
    shape = (lambda h, s: (B, s, h, D)) if layout == "BSHD" else (lambda h, s: (B, h, s, D))
    q, k, v = (orc.from_f32(rng.standard_normal(shape(h, s), dtype=np.float32), code) for h, s in ((Hq, S), (Hkv, Skv), (Hkv, Skv)))
    mask = bias = q_len = kv_len = None
    mk = int(rng.integers(0, 4))
    if mk == 1:
        mask = rng.random((S, Skv)) < 0.85
    elif mk == 2:
        mask = rng.random((B, S, Skv)) < 0.85                     # rank 3 is [batch, seq, kv]
    elif mk == 3:
        mask = orc.to_f32(orc.from_f32(rng.standard_normal((B, Hq, S, Skv)).astype(np.float32), code), code)
        if layout == "BSHD":
            mask = np.ascontiguousarray(mask.transpose(0, 2, 1, 3))
    if rng.integers(0, 2):
        bias = orc.to_f32(orc.from_f32(rng.standard_normal((S, Skv)).astype(np.float32), code), code)
    if rng.integers(0, 2):
        q_len = rng.integers(0, S + 1, size=B).astype(np.int32)
        kv_len = rng.integers(0, Skv + 1, size=B).astype(np.int32)
    dev_mask = mask if mask is None or mask.dtype == np.bool_ else orc.from_f32(mask, code)
    dev_bias = None if bias is None else orc.from_f32(bias, code)
    got, plan = ops.sdpa(q, k, v, dtype=code, layout=LAYOUT[layout], causal=causal, mask=dev_mask, bias=dev_bias, q_len=q_len, kv_len=kv_len,
                         return_plan=True)
    assert plan.kernel_name.startswith("sdpa_tile_"), (plan.kernel_name, B, Hq, Hkv, S, Skv, D)
    want = orc.sdpa(orc.to_f32(q, code), orc.to_f32(k, code), orc.to_f32(v, code), mask=mask, bias=bias, q_len=q_len, kv_len=kv_len,
                    layout=layout, causal=causal)
    gotf = orc.to_f32(got, code)
    assert max_abs_normalised(gotf, want) < (2e-5 if dtype == "f32" else 2e-2), (B, Hq, Hkv, S, Skv, D, layout, causal, mk)
    assert np.all(gotf[want == 0.0] == 0.0)


# ------------------------------------------------------------- decode shapes: a few query tokens over a long cache
DECODE_CASES = [
    # B, Hq, Hkv, S, Skv, D, layout, dtype, causal
    (16, 32, 8, 1, 2048, 128, "BSHD", "bf16", False),      # the decode step of the fifth benchmark configuration
    (2, 8, 8, 1, 300, 64, "BHSD", "f16", False),           # no grouping, head_dim 64, a cache that is no multiple of anything
    (3, 8, 2, 2, 1000, 128, "BHSD", "bf16", False),        # two query tokens, group of 4: 8 rows per KV head
    (2, 4, 2, 2, 257, 128, "BSHD", "bf16", True),          # causal as the reference defines it: row s sees the keys 0..s
    (1, 16, 4, 1, 8192, 128, "BHSD", "bf16", False),       # one sequence: the cache is split many ways
    (2, 32, 2, 1, 1024, 128, "BSHD", "bf16", False),       # a group of 16 query heads: both halves of the 16-row tile
    (2, 8, 2, 3, 515, 64, "BHSD", "f16", True),            # 12 rows (3 tokens x group of 4), causal, head_dim 64
]


@pytest.mark.parametrize("B,Hq,Hkv,S,Skv,D,layout,dtype,causal", DECODE_CASES)
def test_sdpa_decode_kernel(B, Hq, Hkv, S, Skv, D, layout, dtype, causal):
    rng = np.random.default_rng(B * 1000 + Skv)
    code = DT[dtype]
    shape = (lambda h, s: (B, s, h, D)) if layout == "BSHD" else (lambda h, s: (B, h, s, D))
    q, k, v = (orc.from_f32(rng.standard_normal(shape(h, s), dtype=np.float32), code) for h, s in ((Hq, S), (Hkv, Skv), (Hkv, Skv)))
    got, plan = ops.sdpa(q, k, v, dtype=code, layout=LAYOUT[layout], causal=causal, return_plan=True)
    assert plan.kernel_name.startswith("sdpa_decode_"), plan.kernel_name
    want = orc.sdpa(orc.to_f32(q, code), orc.to_f32(k, code), orc.to_f32(v, code), layout=layout, causal=causal)
    assert max_abs_normalised(orc.to_f32(got, code), want) < 2e-2
    # the generic kernel (the reference's per-row algorithm) agrees more tightly than the tolerance
    gen = ops.sdpa(q, k, v, dtype=code, layout=LAYOUT[layout], causal=causal, variant=dv.SDPA_GENERIC)
    assert max_abs_normalised(orc.to_f32(got, code), orc.to_f32(gen, code)) < 2.0 ** -7


@pytest.mark.parametrize("B,Hq,Hkv,S,Skv,D,layout,dtype,causal", [
    (16, 32, 8, 1, 2048, 128, "BSHD", "bf16", False),      # the benchmark's decode step with a different cache length per sequence
    (5, 8, 2, 3, 1000, 64, "BHSD", "f16", True),           # three query tokens of which some are padding, causal
])
def test_sdpa_decode_kernel_with_sequence_lengths(B, Hq, Hkv, S, Skv, D, layout, dtype, causal):
    """KeyValueSeqLen cuts each sequence's cache (a length inside a split, at a split boundary, the whole cache, one key,
    none: that row is all zeros), QuerySeqLen zeroes the padded query positions (sdpa.go:389-411)."""
    rng = np.random.default_rng(B * 77 + Skv)
    code = DT[dtype]
    shape = (lambda h, s: (B, s, h, D)) if layout == "BSHD" else (lambda h, s: (B, h, s, D))
    q, k, v = (orc.from_f32(rng.standard_normal(shape(h, s), dtype=np.float32), code) for h, s in ((Hq, S), (Hkv, Skv), (Hkv, Skv)))
    kv_len = rng.integers(1, Skv + 1, size=B).astype(np.int32)
    kv_len[0], kv_len[1], kv_len[2] = Skv, 1, 0
    if B > 3:
        kv_len[3] = 512
    q_len = rng.integers(0, S + 1, size=B).astype(np.int32)
    q_len[0] = S
    got, plan = ops.sdpa(q, k, v, dtype=code, layout=LAYOUT[layout], causal=causal, q_len=q_len, kv_len=kv_len, return_plan=True)
    assert plan.kernel_name.startswith("sdpa_decode_"), plan.kernel_name
    want = orc.sdpa(orc.to_f32(q, code), orc.to_f32(k, code), orc.to_f32(v, code), q_len=q_len, kv_len=kv_len, layout=layout, causal=causal)
    gotf = orc.to_f32(got, code)
    assert max_abs_normalised(gotf, want) < 2e-2
    # rows the reference leaves at zero are zero here too, bit for bit
    assert np.array_equal(gotf == 0.0, want == 0.0) or np.all(gotf[want == 0.0] == 0.0)
    gen = ops.sdpa(q, k, v, dtype=code, layout=LAYOUT[layout], causal=causal, q_len=q_len, kv_len=kv_len, variant=dv.SDPA_GENERIC)
    assert max_abs_normalised(gotf, orc.to_f32(gen, code)) < 2.0 ** -7


def test_sdpa_decode_kernel_is_refused_where_it_does_not_apply():
    with pytest.raises(ErrNotImplemented):      # float32 stays on the generic kernel
        dv.Plan.sdpa(2, 8, 2, 1, 1024, 128, dv.F32, variant=dv.SDPA_DECODE)
    with pytest.raises(ErrNotImplemented):      # more query rows per KV head than a CTA carries
        dv.Plan.sdpa(2, 64, 2, 1, 1024, 128, dv.BF16, variant=dv.SDPA_DECODE)
    assert dv.Plan.sdpa(2, 8, 2, 1, 64, 128, dv.BF16).kernel_name.startswith("sdpa_generic")      # a short cache
