"""CPU checks of the drop-in boundary: the shared library loads, exports every symbol the
header declares, and plans (shape/dtype kernel selection) can be built without a GPU."""
import os
import re

import pytest

import compute_b200 as cb
from compute_b200 import _lib, device as dv

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_symbols(name="cudabackend.h", prefix="cb_"):
    text = open(os.path.join(ROOT, "include", name)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(" + prefix + r"[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = cb.load_library()
    names = header_symbols()
    assert len(names) >= 30
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/cudabackend.h but not exported"
        assert n in _lib.SIGNATURES, f"{n} has no ctypes signature"
    assert set(_lib.SIGNATURES) <= set(names)
    from compute_b200 import backend as be
    gnames = header_symbols("cudabackend_graph.h", "cbg_")
    assert len(gnames) >= 40
    for n in gnames:
        assert hasattr(lib, n), f"{n} declared in include/cudabackend_graph.h but not exported"
        assert n in be._GRAPH_SIGNATURES, f"{n} has no ctypes signature"


def test_plans_select_kernels_by_shape_and_dtype():
    p = dv.Plan.qdense(1, 4096, 14336, dv.BF16, dv.I8, dv.SCALE_KGROUP, 128, activation=dv.ACT_SILU)
    assert p.kernel_name == "qdense_decode_tc_bf16_n16_i8" and p.workspace_bytes > 0
    # beyond five rows bfloat16 activations travel as two int8 digit planes (16 rows each at M = 16), float32 as three
    assert dv.Plan.qdense(8, 4096, 14336, dv.BF16, dv.I8, dv.SCALE_KGROUP, 128).kernel_name.endswith("_n16p2_i8")
    assert dv.Plan.qdense(16, 4096, 14336, dv.BF16, dv.I8, dv.SCALE_KGROUP, 128).kernel_name.endswith("_n32p2_i8")
    assert dv.Plan.qdense(16, 4096, 14336, dv.F32, dv.I8, dv.SCALE_KGROUP, 128).kernel_name.endswith("_n48_i8")
    # a group of independent projections is one launch: 8 x 112 column tiles on 128 CTAs, 7 whole tiles each (c, c + 128, ...)
    g = dv.Plan.qdense_group(16, 4096, [(14336, False, dv.ACT_SILU)] * 8, dv.BF16, dv.I8, dv.SCALE_KGROUP, 128)
    assert g.kernel_name == "qdense_decode_tc_bf16_n32p2_i8_x8" and g.blocks == 128
    # an 8-way column shard of the same step: 8 x 14 tiles, one whole tile per CTA
    assert dv.Plan.qdense_group(16, 4096, [(1792, False, dv.ACT_SILU)] * 8, dv.BF16, dv.I8, dv.SCALE_KGROUP, 128).blocks == 112
    # few column tiles are shared by clusters of CTAs, each with an equal run of the tile's 128-row units: four CTAs per
    # tile (32 tiles), two (56 tiles), none when a tile has too few units to share (K = 512: four units)
    assert dv.Plan.qdense(16, 4096, 4096, dv.BF16, dv.I8, dv.SCALE_CHANNEL).blocks == 128
    assert dv.Plan.qdense(16, 4096, 7168, dv.BF16, dv.I8, dv.SCALE_CHANNEL).blocks == 112
    assert dv.Plan.qdense(16, 512, 2048, dv.BF16, dv.I8, dv.SCALE_CHANNEL).blocks in (16, 64)
    with pytest.raises(cb.ErrNotImplemented):      # members must suit the tensor-core decode kernel
        dv.Plan.qdense_group(16, 4096, [(14336, False, 0)], dv.BF16, dv.I8, dv.SCALE_KGROUP, 64)
    with pytest.raises(cb.BackendError):
        dv.Plan.qdense_group(16, 4096, [(128, False, 0)] * 17, dv.BF16, dv.I8, dv.SCALE_CHANNEL)
    # K groups finer than the 128-row tensor-core unit stay on the mma.sync decode kernel; M > 16 is prefill
    assert dv.Plan.qdense(16, 4096, 14336, dv.BF16, dv.I8, dv.SCALE_KGROUP, 64).kernel_name == "qdense_decode_bf16_m16_i8"
    assert dv.Plan.qdense(2048, 4096, 14336, dv.BF16, dv.I8, dv.SCALE_CHANNEL).kernel_name == "qdense_prefill_tcgen05_bf16_i8"
    assert dv.Plan.dot(1, 4096, 4096, 4096, dv.F32).kernel_name == "gemm_tcgen05_Float32_Float32_nn"
    # the reference's own scale layout and zero points go to the reference-order kernel
    assert dv.Plan.qdense(1, 4096, 14336, dv.F32, dv.I8, dv.SCALE_REF, 128).kernel_name == "qdense_w8_f32_i8"   # the reference's scale layout
    assert dv.Plan.qdense(4, 64, 64, dv.F32, dv.U8, dv.SCALE_CHANNEL, has_zero_point=True).kernel_name == "qdense_generic_f32_u8"
    assert dv.Plan.dot(1, 3, 5, 7, dv.F64).kernel_name.startswith("dot_generic_Float64")
    assert dv.Plan.sdpa(1, 4, 2, 5, 7, 8, dv.F32, causal=True).kernel_name.startswith("sdpa_")


def test_error_mapping():
    with pytest.raises(cb.ErrNotImplemented):
        dv.Plan.sdpa(1, 1, 1, 2, 2, 8, dv.F8E4M3FN)
    with pytest.raises(cb.BackendError) as e:
        dv.Plan.sdpa(1, 3, 2, 2, 2, 8, dv.F32)
    assert "divisible" in str(e.value) and not isinstance(e.value, cb.ErrNotImplemented)
    with pytest.raises(cb.BackendError):
        dv.Plan.sdpa(1, 1, 1, 2, 2, 1, dv.F32, bias_dims=(2,))
    with pytest.raises(cb.BackendError):
        dv.Plan.sdpa(1, 1, 1, 2, 2, 1, dv.F32, bias_dims=(2, 3))
    with pytest.raises(cb.ErrNotImplemented):
        dv.Plan.dot(1, 2, 2, 2, dv.BOOL)
