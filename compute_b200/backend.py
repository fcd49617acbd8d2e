"""Host-side mirror of gomlx/compute's Backend / Builder / Function / Executable / Buffer
interface (compute.go, builder.go, function.go, executable.go, buffer.go of the
reference) for the accelerated path.  Method names and argument meaning follow
the reference so that tests read like its own; the work happens in
libcudabackend (include/cudabackend_graph.h).  Ops outside the path raise
ErrNotImplemented, as a Go backend embedding notimplemented.Function would.

Host data are numpy arrays; bfloat16 / float16 travel as uint16 bit patterns
with an explicit dtype (compute_b200.device.BF16 / F16).
"""
from __future__ import annotations

import ctypes as C
import re
from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import numpy as np

from . import _lib, device as dv
from ._lib import BackendError, ErrNotImplemented, check

# compute.OpType values used by Capabilities (optype.go)
OP_PARAMETER, OP_CONSTANT, OP_DOT_GENERAL = 1, 2, 32
OP_FUSED_SOFTMAX, OP_FUSED_LAYER_NORM, OP_FUSED_GELU, OP_FUSED_DENSE = 116, 117, 118, 119
OP_FUSED_SDPA, OP_FUSED_ATTENTION_QKV_PROJECTION, OP_FUSED_QUANTIZED_DENSE = 120, 122, 123
OP_QUANTIZED_EMBEDDING_LOOKUP = 124
OP_ALL_REDUCE, OP_ALL_GATHER = 112, 114
REDUCE_OP_SUM, REDUCE_OP_PRODUCT, REDUCE_OP_MAX, REDUCE_OP_MIN = 1, 2, 3, 4      # compute.ReduceOpType (standard_ops.go:65-84)
OP_NAMES = {1: "Parameter", 2: "Constant", 32: "DotGeneral", 112: "AllReduce", 114: "AllGather", 116: "FusedSoftmax", 117: "FusedLayerNorm", 118: "FusedGelu",
            119: "FusedDense", 120: "FusedScaledDotProductAttention", 122: "FusedAttentionQKVProjection", 123: "FusedQuantizedDense"}

# compute.QuantizationScheme (fused_ops.go:81-98)
QUANT_LINEAR, QUANT_NF4, QUANT_GGML = 0, 1, 2
# compute.AttentionAxesLayout (fused_ops.go:6-16)
LAYOUT_BHSD, LAYOUT_BSHD = 0, 1


class _SdpaOptions(C.Structure):
    _fields_ = [("quantized_matmuls", C.c_int), ("query_seq_len", C.c_void_p), ("key_value_seq_len", C.c_void_p),
                ("bias", C.c_void_p), ("scale", C.c_double), ("causal", C.c_int), ("mask", C.c_void_p)]


_GRAPH_SIGNATURES = {
    "cbg_backend_new": ([C.c_char_p, C.POINTER(C.c_void_p)], C.c_int),
    "cbg_backend_name": ([C.c_void_p], C.c_char_p),
    "cbg_backend_description": ([C.c_void_p], C.c_char_p),
    "cbg_backend_num_devices": ([C.c_void_p], C.c_int),
    "cbg_backend_device_description": ([C.c_void_p, C.c_int, C.c_char_p, C.c_size_t], C.c_int),
    "cbg_backend_capabilities": ([C.c_void_p, C.POINTER(C.c_int32), C.POINTER(C.c_int), C.POINTER(C.c_int32), C.POINTER(C.c_int)], C.c_int),
    "cbg_backend_finalize": ([C.c_void_p], C.c_int),
    "cbg_backend_is_finalized": ([C.c_void_p], C.c_int),
    "cbg_backend_free": ([C.c_void_p], C.c_int),
    "cbg_buffer_from_flat": ([C.c_void_p, C.c_int, C.c_void_p, C.c_int32, C.c_int, C.POINTER(C.c_int64), C.POINTER(C.c_void_p)], C.c_int),
    "cbg_buffer_shape": ([C.c_void_p, C.POINTER(C.c_int32), C.POINTER(C.c_int), C.POINTER(C.c_int64)], C.c_int),
    "cbg_buffer_device_num": ([C.c_void_p, C.POINTER(C.c_int)], C.c_int),
    "cbg_buffer_to_flat": ([C.c_void_p, C.c_void_p, C.c_size_t], C.c_int),
    "cbg_buffer_copy_to_device": ([C.c_void_p, C.c_int, C.POINTER(C.c_void_p)], C.c_int),
    "cbg_buffer_device_ptr": ([C.c_void_p, C.POINTER(C.c_void_p)], C.c_int),
    "cbg_buffer_finalize": ([C.c_void_p], C.c_int),
    "cbg_builder_new": ([C.c_void_p, C.c_char_p, C.POINTER(C.c_void_p)], C.c_int),
    "cbg_builder_main": ([C.c_void_p, C.POINTER(C.c_void_p)], C.c_int),
    "cbg_builder_distributed_spmd": ([C.c_void_p, C.c_int], C.c_int),
    "cbg_builder_device_assignment": ([C.c_void_p, C.POINTER(C.c_int), C.c_int], C.c_int),
    "cbg_builder_compile": ([C.c_void_p, C.POINTER(C.c_void_p)], C.c_int),
    "cbg_builder_free": ([C.c_void_p], C.c_int),
    "cbg_fn_parameter": ([C.c_void_p, C.c_char_p, C.c_int32, C.c_int, C.POINTER(C.c_int64), C.POINTER(C.c_void_p)], C.c_int),
    "cbg_fn_constant": ([C.c_void_p, C.c_void_p, C.c_int32, C.c_int, C.POINTER(C.c_int64), C.POINTER(C.c_void_p)], C.c_int),
    "cbg_fn_shape": ([C.c_void_p, C.POINTER(C.c_int32), C.POINTER(C.c_int), C.POINTER(C.c_int64)], C.c_int),
    "cbg_fn_return": ([C.c_void_p, C.POINTER(C.c_void_p), C.c_int], C.c_int),
    "cbg_fn_dot_general": ([C.c_void_p, C.c_void_p, C.POINTER(C.c_int), C.c_int, C.POINTER(C.c_int), C.c_int, C.c_void_p,
                            C.POINTER(C.c_int), C.POINTER(C.c_int), C.c_int32, C.c_int32, C.POINTER(C.c_void_p)], C.c_int),
    "cbg_fn_reshape": ([C.c_void_p, C.c_void_p, C.c_int, C.POINTER(C.c_int64), C.POINTER(C.c_void_p)], C.c_int),
    "cbg_fn_slice": ([C.c_void_p, C.c_void_p, C.POINTER(C.c_int64), C.POINTER(C.c_int64), C.POINTER(C.c_int64), C.POINTER(C.c_void_p)], C.c_int),
    "cbg_fn_iota": ([C.c_void_p, C.c_int32, C.c_int, C.POINTER(C.c_int64), C.c_int, C.POINTER(C.c_void_p)], C.c_int),
    "cbg_fn_convert_dtype": ([C.c_void_p, C.c_void_p, C.c_int32, C.POINTER(C.c_void_p)], C.c_int),
    "cbg_fn_transpose": ([C.c_void_p, C.c_void_p, C.POINTER(C.c_int), C.POINTER(C.c_void_p)], C.c_int),
    "cbg_fn_fused_softmax": ([C.c_void_p, C.c_void_p, C.c_int, C.POINTER(C.c_void_p)], C.c_int),
    "cbg_fn_fused_gelu": ([C.c_void_p, C.c_void_p, C.c_int, C.POINTER(C.c_void_p)], C.c_int),
    "cbg_fn_fused_layer_norm": ([C.c_void_p, C.c_void_p, C.POINTER(C.c_int), C.c_int, C.c_double, C.c_void_p, C.c_void_p, C.POINTER(C.c_void_p)], C.c_int),
    "cbg_fn_fused_attention_qkv_projection": ([C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64,
                                               C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.POINTER(C.c_void_p)], C.c_int),
    "cbg_fn_fused_dense": ([C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.POINTER(C.c_void_p)], C.c_int),
    "cbg_fn_fused_quantized_dense": ([C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p,
                                      C.c_int, C.c_int64, C.c_int, C.POINTER(C.c_void_p)], C.c_int),
    "cbg_fn_quantized_embedding_lookup": ([C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.POINTER(C.c_void_p)], C.c_int),
    "cbg_fn_fused_quantized_dense_ggml": ([C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.POINTER(C.c_void_p)], C.c_int),
    "cbg_fn_fused_sdpa": ([C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.POINTER(_SdpaOptions), C.POINTER(C.c_void_p)], C.c_int),
    "cbg_fn_not_implemented": ([C.c_void_p, C.c_char_p], C.c_int),
    "cbg_fn_add": ([C.c_void_p, C.c_void_p, C.c_void_p, C.POINTER(C.c_void_p)], C.c_int),
    "cbg_fn_sub": ([C.c_void_p, C.c_void_p, C.c_void_p, C.POINTER(C.c_void_p)], C.c_int),
    "cbg_fn_mul": ([C.c_void_p, C.c_void_p, C.c_void_p, C.POINTER(C.c_void_p)], C.c_int),
    "cbg_fn_div": ([C.c_void_p, C.c_void_p, C.c_void_p, C.POINTER(C.c_void_p)], C.c_int),
    "cbg_fn_max": ([C.c_void_p, C.c_void_p, C.c_void_p, C.POINTER(C.c_void_p)], C.c_int),
    "cbg_fn_min": ([C.c_void_p, C.c_void_p, C.c_void_p, C.POINTER(C.c_void_p)], C.c_int),
    "cbg_fn_neg": ([C.c_void_p, C.c_void_p, C.POINTER(C.c_void_p)], C.c_int),
    "cbg_fn_rsqrt": ([C.c_void_p, C.c_void_p, C.POINTER(C.c_void_p)], C.c_int),
    "cbg_fn_sqrt": ([C.c_void_p, C.c_void_p, C.POINTER(C.c_void_p)], C.c_int),
    "cbg_fn_exp": ([C.c_void_p, C.c_void_p, C.POINTER(C.c_void_p)], C.c_int),
    "cbg_fn_logistic": ([C.c_void_p, C.c_void_p, C.POINTER(C.c_void_p)], C.c_int),
    "cbg_fn_tanh": ([C.c_void_p, C.c_void_p, C.POINTER(C.c_void_p)], C.c_int),
    "cbg_fn_reduce_sum": ([C.c_void_p, C.c_void_p, C.POINTER(C.c_int), C.c_int, C.POINTER(C.c_void_p)], C.c_int),
    "cbg_fn_reduce_max": ([C.c_void_p, C.c_void_p, C.POINTER(C.c_int), C.c_int, C.POINTER(C.c_void_p)], C.c_int),
    "cbg_fn_broadcast_in_dim": ([C.c_void_p, C.c_void_p, C.c_int32, C.c_int, C.POINTER(C.c_int64), C.POINTER(C.c_int), C.POINTER(C.c_void_p)], C.c_int),
    "cbg_fn_all_reduce": ([C.c_void_p, C.POINTER(C.c_void_p), C.c_int, C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_int), C.c_int, C.POINTER(C.c_void_p)], C.c_int),
    "cbg_fn_all_gather": ([C.c_void_p, C.POINTER(C.c_void_p), C.c_int, C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_int), C.c_int, C.POINTER(C.c_void_p)], C.c_int),
    "cbg_fn_parameter_sharded": ([C.c_void_p, C.c_char_p, C.c_int32, C.c_int, C.POINTER(C.c_int64), C.POINTER(C.c_char_p), C.POINTER(C.c_int), C.c_int,
                                 C.POINTER(C.c_char_p), C.c_int, C.POINTER(C.c_void_p)], C.c_int),
    "cbg_exec_input_sharding": ([C.c_void_p, C.c_int, C.c_char_p, C.c_size_t], C.c_int),
    "cbg_exec_num_inputs": ([C.c_void_p], C.c_int),
    "cbg_exec_num_outputs": ([C.c_void_p], C.c_int),
    "cbg_exec_input_info": ([C.c_void_p, C.c_int, C.c_char_p, C.c_size_t, C.POINTER(C.c_int32), C.POINTER(C.c_int), C.POINTER(C.c_int64)], C.c_int),
    "cbg_exec_output_info": ([C.c_void_p, C.c_int, C.POINTER(C.c_int32), C.POINTER(C.c_int), C.POINTER(C.c_int64)], C.c_int),
    "cbg_exec_kernel_names": ([C.c_void_p, C.c_char_p, C.c_size_t], C.c_int),
    "cbg_exec_last_trace": ([C.c_void_p, C.c_char_p, C.c_size_t], C.c_int),
    "cbg_exec_graph_replays": ([C.c_void_p], C.c_int),
    "cbg_exec_execute": ([C.c_void_p, C.POINTER(C.c_void_p), C.c_int, C.POINTER(C.c_uint8), C.c_int, C.POINTER(C.c_void_p), C.c_int], C.c_int),
    "cbg_exec_finalize": ([C.c_void_p], C.c_int),
}
_glib = None


def _g():
    global _glib
    if _glib is None:
        lib = _lib.load()
        for name, (args, res) in _GRAPH_SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes = args
            fn.restype = res
        _glib = lib
    return _glib


def _i64(vals):
    vals = list(vals)
    return (C.c_int64 * max(len(vals), 1))(*vals)


def _ints(vals):
    vals = list(vals or [])
    return (C.c_int * max(len(vals), 1))(*vals)


@dataclass(frozen=True)
class Shape:
    """shapes.Shape: dtype + dimensions."""
    dtype: int
    dimensions: Tuple[int, ...] = ()

    def rank(self) -> int:
        return len(self.dimensions)

    def size(self) -> int:
        return int(np.prod(self.dimensions, dtype=np.int64)) if self.dimensions else 1

    def _c_dims(self):
        """(element count, dimensions as a C int64 array), built once per Shape: BufferFromFlatData is on the per-step
        path of a decode loop and a Shape is immutable in use."""
        c = self.__dict__.get("_c_cache")
        if c is None or c[2] != self.dimensions:
            c = (self.size(), _i64(self.dimensions), self.dimensions)
            self.__dict__["_c_cache"] = c
        return c


def make_shape(dtype: int, *dims: int) -> Shape:
    return Shape(dtype, tuple(int(d) for d in dims))


def _read_shape(fn, handle) -> Shape:
    dt, rk, dims = C.c_int32(0), C.c_int(0), (C.c_int64 * 8)()
    check(fn(handle, C.byref(dt), C.byref(rk), dims))
    return Shape(dt.value, tuple(dims[i] for i in range(rk.value)))


@dataclass
class Capabilities:
    """compute.Capabilities (capabilities.go:12-39)."""
    Operations: dict = field(default_factory=dict)
    DTypes: dict = field(default_factory=dict)
    Functions: bool = False
    DynamicAxes: bool = False
    PreferConstantsForVariables: bool = False


@dataclass
class DotGeneralConfig:
    """compute.DotGeneralConfig (standard_ops.go:91-111); 0 = InvalidDType = unset."""
    AccumulatorDType: int = 0
    OutputDType: int = 0


# compute.DenseLayout (fused_ops.go:50-58)
DENSE_LAYOUT_INPUT_OUTPUTS, DENSE_LAYOUT_OUTPUTS_INPUT = 0, 1


@dataclass
class DenseConfig:
    """compute.DenseConfig (fused_ops.go:72-78)."""
    Activation: int = dv.ACT_NONE
    WeightLayout: int = DENSE_LAYOUT_INPUT_OUTPUTS


@dataclass
class Quantization:
    """compute.Quantization (fused_ops.go:204-234).  BlockAxis=1 is the reference layout
    (Scale [K, ceil(N/BlockSize)]); BlockAxis=0 is this backend's extension
    (Scale [ceil(K/BlockSize), N]; BlockSize=K gives per-output-channel scales)."""
    Scheme: int = QUANT_LINEAR
    Scale: Optional["Value"] = None
    ZeroPoint: Optional["Value"] = None
    BlockAxis: int = 1
    BlockSize: int = 1
    GGMLType: int = 0


@dataclass
class ScaledDotProductAttentionConfig:
    """compute.ScaledDotProductAttentionConfig (fused_ops.go:245-277)."""
    QuantizedMatmuls: bool = False
    QuerySeqLen: Optional["Value"] = None
    KeyValueSeqLen: Optional["Value"] = None
    Bias: Optional["Value"] = None
    Scale: float = 0.0
    Causal: bool = False
    Mask: Optional["Value"] = None


@dataclass
class DeviceMesh:
    """distributed.DeviceMesh (distributed/devicemesh.go:23-110): named axes over the devices of a computation."""
    AxesNames: Tuple[str, ...]
    AxesSizes: Tuple[int, ...]

    def NumDevices(self) -> int:
        return int(np.prod(self.AxesSizes, dtype=np.int64)) if self.AxesSizes else 1

    def ComputeReplicaGroups(self, axes: Sequence[str]) -> List[List[int]]:
        """Groups of device indices that differ only along `axes` (distributed/devicemesh.go:224-293): the devices are
        numbered row-major over the mesh; every group walks the listed axes (in mesh order) with the others fixed."""
        for a in axes:
            if a not in self.AxesNames:
                raise BackendError(_lib.ERR_INVALID_ARG, f"mesh axis {a!r} not found in the mesh axes {list(self.AxesNames)}")
        if len(set(axes)) != len(axes):
            raise BackendError(_lib.ERR_INVALID_ARG, f"mesh axes {list(axes)} are repeated")
        ids = np.arange(self.NumDevices()).reshape(self.AxesSizes)
        red = [i for i, n in enumerate(self.AxesNames) if n in axes]
        keep = [i for i in range(len(self.AxesNames)) if i not in red]
        moved = np.transpose(ids, keep + red).reshape(-1, int(np.prod([self.AxesSizes[i] for i in red], dtype=np.int64)) if red else 1)
        return [list(map(int, row)) for row in moved]


@dataclass
class ShardingSpec:
    """distributed.ShardingSpec (distributed/shardingspec.go:43-110): per tensor axis the mesh axes it is sharded over
    (an empty tuple = replicated; missing trailing axes are replicated)."""
    Mesh: DeviceMesh
    Axes: Tuple[Tuple[str, ...], ...] = ()


class Value:
    """compute.Value: an opaque node of a function under construction."""

    def __init__(self, handle, fn: "Function"):
        self.handle = handle
        self.fn = fn


class Buffer:
    """compute.Buffer (buffer.go:12-42)."""

    def __init__(self, handle, backend: "Backend"):
        self.handle = handle
        self._backend = backend

    def Backend(self) -> "Backend":
        return self._backend

    def Shape(self) -> Shape:
        return _read_shape(_g().cbg_buffer_shape, self.handle)

    def DeviceNum(self) -> int:
        d = C.c_int(0)
        check(_g().cbg_buffer_device_num(self.handle, C.byref(d)))
        return d.value

    def ToFlatData(self, flat: np.ndarray) -> None:
        """Copies the buffer into `flat` (exact size), like Buffer.ToFlatData."""
        if not flat.flags.c_contiguous:
            raise BackendError(_lib.ERR_INVALID_ARG, "Buffer.ToFlatData: flat must be contiguous")
        check(_g().cbg_buffer_to_flat(self.handle, flat.__array_interface__["data"][0], flat.nbytes))

    def ToNumpy(self) -> np.ndarray:
        s = self.Shape()
        out = np.empty(s.dimensions, dv.NP_CARRIER[s.dtype])
        self.ToFlatData(out)
        return out

    def CopyToDevice(self, device_num: int) -> "Buffer":
        h = C.c_void_p()
        check(_g().cbg_buffer_copy_to_device(self.handle, device_num, C.byref(h)))
        return Buffer(h, self._backend)

    def DevicePtr(self) -> int:
        p = C.c_void_p()
        check(_g().cbg_buffer_device_ptr(self.handle, C.byref(p)))
        return p.value

    def Data(self):
        raise BackendError(_lib.ERR_INVALID_ARG, "Buffer.Data: the cuda backend has no shared (host-visible) buffers")

    def Finalize(self) -> None:
        if self.handle:
            _g().cbg_buffer_finalize(self.handle)
            self.handle = None


class Function:
    """compute.Function (function.go:23-134): graph building.  Only the ops of the
    accelerated path exist; the rest raise ErrNotImplemented."""

    def __init__(self, handle, builder: "Builder"):
        self.handle = handle
        self._builder = builder

    def Builder(self) -> "Builder":
        return self._builder

    def Name(self) -> str:
        return "main"

    def _v(self, h) -> Value:
        return Value(h, self)

    def Parameter(self, name: str, shape: Shape, sharding: Optional[ShardingSpec] = None) -> Value:
        h = C.c_void_p()
        if sharding is None:
            check(_g().cbg_fn_parameter(self.handle, name.encode(), shape.dtype, shape.rank(), _i64(shape.dimensions), C.byref(h)))
            return self._v(h)
        mesh = sharding.Mesh
        names = (C.c_char_p * max(len(mesh.AxesNames), 1))(*[n.encode() for n in mesh.AxesNames])
        specs = (C.c_char_p * max(len(sharding.Axes), 1))(*[",".join(a).encode() for a in sharding.Axes])
        check(_g().cbg_fn_parameter_sharded(self.handle, name.encode(), shape.dtype, shape.rank(), _i64(shape.dimensions), names,
                                            _ints(mesh.AxesSizes), len(mesh.AxesNames), specs, len(sharding.Axes), C.byref(h)))
        return self._v(h)

    def Constant(self, flat, *dims: int, dtype: Optional[int] = None) -> Value:
        a = np.ascontiguousarray(flat)
        if dtype is None:
            rev = {np.dtype(v): k for k, v in dv.NP_CARRIER.items() if k not in (dv.F16, dv.BF16, dv.U16)}
            rev[np.dtype(np.uint16)] = dv.U16
            dtype = rev[a.dtype]
        h = C.c_void_p()
        n = int(np.prod(dims, dtype=np.int64)) if dims else 1
        if dtype in (dv.I4, dv.U4):
            n = (n + 1) // 2
        if a.size != n:
            raise BackendError(_lib.ERR_INVALID_ARG, f"Constant: flat has {a.size} elements, dimensions {list(dims)} need {n}")
        check(_g().cbg_fn_constant(self.handle, a.ctypes.data, dtype, len(dims), _i64(dims), C.byref(h)))
        return self._v(h)

    def Shape(self, value: Value) -> Shape:
        return _read_shape(_g().cbg_fn_shape, value.handle)

    def Return(self, outputs: Sequence[Value], shardings=None) -> None:
        arr = (C.c_void_p * max(len(outputs), 1))(*[o.handle for o in outputs])
        check(_g().cbg_fn_return(self.handle, arr, len(outputs)))

    # ---- StandardOps on the path
    def DotGeneral(self, lhs: Value, lhsContractingAxes, lhsBatchAxes, rhs: Value, rhsContractingAxes, rhsBatchAxes,
                   config: Optional[DotGeneralConfig] = None) -> Value:
        config = config or DotGeneralConfig()
        lc, lb = list(lhsContractingAxes or []), list(lhsBatchAxes or [])
        rc, rb = list(rhsContractingAxes or []), list(rhsBatchAxes or [])
        if len(lc) != len(rc):
            raise BackendError(_lib.ERR_INVALID_ARG, f"DotGeneral number of contracting axes for lhs ({len(lc)}) doesn't match rhs ({len(rc)})")
        if len(lb) != len(rb):
            raise BackendError(_lib.ERR_INVALID_ARG, f"DotGeneral number of batch axes for lhs ({len(lb)}) doesn't match rhs ({len(rb)})")
        h = C.c_void_p()
        check(_g().cbg_fn_dot_general(self.handle, lhs.handle, _ints(lc), len(lc), _ints(lb), len(lb), rhs.handle,
                                      _ints(rc), _ints(rb), config.AccumulatorDType, config.OutputDType, C.byref(h)))
        return self._v(h)

    def Reshape(self, x: Value, *dims: int) -> Value:
        h = C.c_void_p()
        check(_g().cbg_fn_reshape(self.handle, x.handle, len(dims), _i64(dims), C.byref(h)))
        return self._v(h)

    def Slice(self, x: Value, starts, limits, strides=None) -> Value:
        h = C.c_void_p()
        check(_g().cbg_fn_slice(self.handle, x.handle, _i64(starts), _i64(limits),
                                _i64(strides) if strides is not None else None, C.byref(h)))
        return self._v(h)

    def Iota(self, shape: Shape, iotaAxis: int) -> Value:
        h = C.c_void_p()
        check(_g().cbg_fn_iota(self.handle, shape.dtype, shape.rank(), _i64(shape.dimensions), iotaAxis, C.byref(h)))
        return self._v(h)

    def ConvertDType(self, x: Value, dtype: int) -> Value:
        h = C.c_void_p()
        check(_g().cbg_fn_convert_dtype(self.handle, x.handle, dtype, C.byref(h)))
        return self._v(h)

    def Transpose(self, x: Value, *permutation: int) -> Value:
        h = C.c_void_p()
        check(_g().cbg_fn_transpose(self.handle, x.handle, _ints(permutation), C.byref(h)))
        return self._v(h)

    # ---- element-wise / reduce ops a decoder block needs (float dtypes; not advertised in Capabilities)
    def _binary(self, name: str, lhs: Value, rhs: Value) -> Value:
        h = C.c_void_p()
        check(getattr(_g(), "cbg_fn_" + name)(self.handle, lhs.handle, rhs.handle, C.byref(h)))
        return self._v(h)

    def _unary(self, name: str, x: Value) -> Value:
        h = C.c_void_p()
        check(getattr(_g(), "cbg_fn_" + name)(self.handle, x.handle, C.byref(h)))
        return self._v(h)

    def Add(self, lhs: Value, rhs: Value) -> Value: return self._binary("add", lhs, rhs)
    def Sub(self, lhs: Value, rhs: Value) -> Value: return self._binary("sub", lhs, rhs)
    def Mul(self, lhs: Value, rhs: Value) -> Value: return self._binary("mul", lhs, rhs)
    def Div(self, lhs: Value, rhs: Value) -> Value: return self._binary("div", lhs, rhs)
    def Max(self, lhs: Value, rhs: Value) -> Value: return self._binary("max", lhs, rhs)
    def Min(self, lhs: Value, rhs: Value) -> Value: return self._binary("min", lhs, rhs)
    def Neg(self, x: Value) -> Value: return self._unary("neg", x)
    def Rsqrt(self, x: Value) -> Value: return self._unary("rsqrt", x)
    def Sqrt(self, x: Value) -> Value: return self._unary("sqrt", x)
    def Exp(self, x: Value) -> Value: return self._unary("exp", x)
    def Logistic(self, x: Value) -> Value: return self._unary("logistic", x)
    def Tanh(self, x: Value) -> Value: return self._unary("tanh", x)

    def ReduceSum(self, x: Value, *axes: int) -> Value:
        h = C.c_void_p()
        check(_g().cbg_fn_reduce_sum(self.handle, x.handle, _ints(axes), len(axes), C.byref(h)))
        return self._v(h)

    def ReduceMax(self, x: Value, *axes: int) -> Value:
        h = C.c_void_p()
        check(_g().cbg_fn_reduce_max(self.handle, x.handle, _ints(axes), len(axes), C.byref(h)))
        return self._v(h)

    def BroadcastInDim(self, x: Value, outputShape: Shape, broadcastAxes: Sequence[int]) -> Value:
        h = C.c_void_p()
        check(_g().cbg_fn_broadcast_in_dim(self.handle, x.handle, outputShape.dtype, outputShape.rank(), _i64(outputShape.dimensions),
                                           _ints(broadcastAxes), C.byref(h)))
        return self._v(h)

    # ---- CollectiveOps (collectiveops.go:10-39)
    @staticmethod
    def _groups(replicaGroups):
        groups = [list(g) for g in (replicaGroups or [])]
        flat = [r for g in groups for r in g]
        return _ints(flat), _ints([len(g) for g in groups]), len(groups)

    def AllReduce(self, operands: Sequence[Value], reductionType: int, replicaGroups=None) -> List[Value]:
        ops = (C.c_void_p * max(len(operands), 1))(*[o.handle for o in operands])
        outs = (C.c_void_p * max(len(operands), 1))()
        flat, sizes, n = self._groups(replicaGroups)
        check(_g().cbg_fn_all_reduce(self.handle, ops, len(operands), reductionType, flat, sizes, n, outs))
        return [self._v(C.c_void_p(outs[i])) for i in range(len(operands))]

    def AllGather(self, operands: Sequence[Value], gatherAxis: int, replicaGroups=None) -> List[Value]:
        """The extension the interface sketches (collectiveops.go:31-32)."""
        ops = (C.c_void_p * max(len(operands), 1))(*[o.handle for o in operands])
        outs = (C.c_void_p * max(len(operands), 1))()
        flat, sizes, n = self._groups(replicaGroups)
        check(_g().cbg_fn_all_gather(self.handle, ops, len(operands), gatherAxis, flat, sizes, n, outs))
        return [self._v(C.c_void_p(outs[i])) for i in range(len(operands))]

    # ---- FusedOps on the path
    def FusedSoftmax(self, x: Value, axis: int) -> Value:
        h = C.c_void_p()
        check(_g().cbg_fn_fused_softmax(self.handle, x.handle, axis, C.byref(h)))
        return self._v(h)

    def FusedGelu(self, x: Value, exact: bool) -> Value:
        h = C.c_void_p()
        check(_g().cbg_fn_fused_gelu(self.handle, x.handle, int(exact), C.byref(h)))
        return self._v(h)

    def FusedLayerNorm(self, x: Value, axes: Sequence[int], epsilon: float, gamma: Optional[Value] = None,
                       beta: Optional[Value] = None) -> Value:
        h = C.c_void_p()
        check(_g().cbg_fn_fused_layer_norm(self.handle, x.handle, _ints(axes), len(axes), float(epsilon),
                                           gamma.handle if gamma is not None else None,
                                           beta.handle if beta is not None else None, C.byref(h)))
        return self._v(h)

    def FusedAttentionQKVProjection(self, x: Value, wQKV: Value, biasQ: Optional[Value], biasK: Optional[Value],
                                    biasV: Optional[Value], queryDim: int, keyValueDim: int):
        """Returns (query, key, value)."""
        hv = lambda v: v.handle if v is not None else None
        q, k, v = C.c_void_p(), C.c_void_p(), C.c_void_p()
        check(_g().cbg_fn_fused_attention_qkv_projection(self.handle, x.handle, wQKV.handle, hv(biasQ), hv(biasK), hv(biasV),
                                                         queryDim, keyValueDim, C.byref(q), C.byref(k), C.byref(v)))
        return self._v(q), self._v(k), self._v(v)

    def FusedDense(self, x: Value, weight: Value, bias: Optional[Value], options: Optional[DenseConfig] = None) -> Value:
        o = options or DenseConfig()
        h = C.c_void_p()
        check(_g().cbg_fn_fused_dense(self.handle, x.handle, weight.handle, bias.handle if bias is not None else None,
                                      o.Activation, o.WeightLayout, C.byref(h)))
        return self._v(h)

    def FusedQuantizedDense(self, x: Value, weights: Value, bias: Optional[Value], weightsQuantization: Quantization,
                            activation: int = dv.ACT_NONE) -> Value:
        q = weightsQuantization
        if q is None:
            raise BackendError(_lib.ERR_INVALID_ARG, "FusedQuantizedDense: weightsQuantization must not be nil")
        h = C.c_void_p()
        if q.Scheme == QUANT_GGML:
            if q.ZeroPoint is not None:
                raise BackendError(_lib.ERR_INVALID_ARG, "FusedQuantizedDense(GGML): ZeroPoint must be nil for GGML scheme")
            check(_g().cbg_fn_fused_quantized_dense_ggml(self.handle, x.handle, weights.handle,
                                                         bias.handle if bias is not None else None, q.GGMLType, activation, C.byref(h)))
            return self._v(h)
        check(_g().cbg_fn_fused_quantized_dense(
            self.handle, x.handle, weights.handle, bias.handle if bias is not None else None, q.Scheme,
            q.Scale.handle if q.Scale is not None else None, q.ZeroPoint.handle if q.ZeroPoint is not None else None,
            q.BlockAxis, q.BlockSize, activation, C.byref(h)))
        return self._v(h)

    def QuantizedEmbeddingLookup(self, data: Value, indices: Value, dataQuantization: Quantization) -> Value:
        """FusedOps.QuantizedEmbeddingLookup (fused_ops.go:394-411): data [vocabSize, bytesPerRow] Uint8 GGML blocks,
        indices integer [batch..., 1] -> Float32 [batch..., K]."""
        q = dataQuantization
        if q is None:
            raise BackendError(_lib.ERR_INVALID_ARG, "QuantizedEmbeddingLookup: dataQuantization must not be nil")
        h = C.c_void_p()
        check(_g().cbg_fn_quantized_embedding_lookup(self.handle, data.handle, indices.handle, q.Scheme, q.GGMLType, C.byref(h)))
        return self._v(h)

    def FusedScaledDotProductAttention(self, query: Value, key: Value, value: Value, axesLayout: int = LAYOUT_BHSD,
                                       options: Optional[ScaledDotProductAttentionConfig] = None):
        """Returns (output, statesForVJP); statesForVJP is empty (no fused backward)."""
        o = None
        if options is not None:
            hv = lambda v: v.handle if v is not None else None
            o = _SdpaOptions(int(options.QuantizedMatmuls), hv(options.QuerySeqLen), hv(options.KeyValueSeqLen),
                             hv(options.Bias), float(options.Scale), int(options.Causal), hv(options.Mask))
        h = C.c_void_p()
        check(_g().cbg_fn_fused_sdpa(self.handle, query.handle, key.handle, value.handle, axesLayout,
                                     C.byref(o) if o is not None else None, C.byref(h)))
        return self._v(h), []

    def FusedScaledDotProductAttentionVJP(self, *args, **kwargs):
        return self._not_implemented("FusedScaledDotProductAttentionVJP")

    # ---- everything else: notimplemented
    def _not_implemented(self, op: str):
        check(_g().cbg_fn_not_implemented(self.handle, op.encode()))

    def __getattr__(self, name: str):
        # Any other op of the interface (Neg, Add, FusedSoftmax, AllReduce, While, ...).
        if name and name[0].isupper():
            def stub(*args, **kwargs):
                return self._not_implemented(name)
            return stub
        raise AttributeError(name)


class Executable:
    """compute.Executable (executable.go:10-37)."""

    def __init__(self, handle, backend: "Backend"):
        self.handle = handle
        self._backend = backend

    def Inputs(self) -> Tuple[List[str], List[Shape]]:
        names, shapes = [], []
        for i in range(_g().cbg_exec_num_inputs(self.handle)):
            nm = C.create_string_buffer(256)
            dt, rk, dims = C.c_int32(0), C.c_int(0), (C.c_int64 * 8)()
            check(_g().cbg_exec_input_info(self.handle, i, nm, 256, C.byref(dt), C.byref(rk), dims))
            names.append(nm.value.decode())
            shapes.append(Shape(dt.value, tuple(dims[j] for j in range(rk.value))))
        return names, shapes

    def Outputs(self) -> List[Shape]:
        out = []
        for i in range(_g().cbg_exec_num_outputs(self.handle)):
            dt, rk, dims = C.c_int32(0), C.c_int(0), (C.c_int64 * 8)()
            check(_g().cbg_exec_output_info(self.handle, i, C.byref(dt), C.byref(rk), dims))
            out.append(Shape(dt.value, tuple(dims[j] for j in range(rk.value))))
        return out

    def InputSharding(self, i: int) -> str:
        buf = C.create_string_buffer(512)
        check(_g().cbg_exec_input_sharding(self.handle, i, buf, 512))
        return buf.value.decode()

    def KernelNames(self) -> List[str]:
        buf = C.create_string_buffer(4096)
        check(_g().cbg_exec_kernel_names(self.handle, buf, 4096))
        return [s for s in buf.value.decode().split("\n") if s]

    def GraphReplays(self) -> int:
        """How many Execute calls so far were replays of a captured CUDA graph."""
        return int(_g().cbg_exec_graph_replays(self.handle))

    def LastTrace(self) -> List[dict]:
        """The per-launch device times of the latest Execute when the backend was created with the
        "trace" option (or CUDABACKEND_TRACE=1): one dict per launch (device, node, kernel, out, us)."""
        buf = C.create_string_buffer(1 << 16)
        check(_g().cbg_exec_last_trace(self.handle, buf, 1 << 16))
        rows = []
        pat = re.compile(r"cudabackend trace: exec=(\S+) device=(\d+) node=(\d+) kernel=(\S+) out=(.*) us=([0-9.]+)$")
        for line in buf.value.decode().split("\n"):
            m = pat.match(line)
            if m:
                rows.append({"exec": m.group(1), "device": int(m.group(2)), "node": int(m.group(3)), "kernel": m.group(4),
                             "out": m.group(5), "us": float(m.group(6))})
        return rows

    def Execute(self, inputs: Sequence[Buffer], donate: Optional[Sequence[bool]] = None, defaultDevice: int = 0) -> List[Buffer]:
        n_in = len(inputs)
        ins = (C.c_void_p * max(n_in, 1))(*[b.handle if b is not None else None for b in inputs])
        don = None
        if donate is not None:
            if len(donate) != n_in:
                raise BackendError(_lib.ERR_INVALID_ARG, f"Execute: donate has {len(donate)} entries for {n_in} inputs")
            don = (C.c_uint8 * max(n_in, 1))(*[1 if d else 0 for d in donate])
        n_out_max = self.__dict__.get("_n_out_max")
        if n_out_max is None:          # fixed for the life of the executable
            n_out_max = self._n_out_max = max(_g().cbg_exec_num_outputs(self.handle) * max(self._backend.NumDevices(), 1), 1)
        outs = (C.c_void_p * n_out_max)()
        check(_g().cbg_exec_execute(self.handle, ins, n_in, don, defaultDevice, outs, n_out_max))
        if donate is not None:
            for b, d in zip(inputs, donate):
                if d:
                    b._donated = True
        return [Buffer(C.c_void_p(outs[i]), self._backend) for i in range(n_out_max) if outs[i]]

    def Finalize(self) -> None:
        if self.handle:
            _g().cbg_exec_finalize(self.handle)
            self.handle = None


class Builder:
    """compute.Builder (builder.go:29-82)."""

    def __init__(self, handle, backend: "Backend", name: str):
        self.handle = handle
        self._backend = backend
        self._name = name
        self._main = None

    def Name(self) -> str:
        return self._name

    def Main(self) -> Function:
        if self._main is None:
            h = C.c_void_p()
            check(_g().cbg_builder_main(self.handle, C.byref(h)))
            self._main = Function(h, self)
        return self._main

    def NewFunction(self, name: str):
        raise ErrNotImplemented(_lib.ERR_NOT_IMPLEMENTED, "NewFunction: functions/closures are not implemented by the cuda backend")

    def OpShape(self, value: Value) -> Shape:
        return _read_shape(_g().cbg_fn_shape, value.handle)

    def DistributedSPMD(self, numDevices: int) -> None:
        check(_g().cbg_builder_distributed_spmd(self.handle, numDevices))

    def DistributedAutoSharding(self, *meshes) -> None:
        raise ErrNotImplemented(_lib.ERR_NOT_IMPLEMENTED, "DistributedAutoSharding is not implemented by the cuda backend")

    def DeviceAssignment(self, *devices: int) -> None:
        check(_g().cbg_builder_device_assignment(self.handle, _ints(devices), len(devices)))

    def Compile(self) -> Executable:
        h = C.c_void_p()
        check(_g().cbg_builder_compile(self.handle, C.byref(h)))
        return Executable(h, self._backend)

    def __del__(self):
        try:
            if self.handle:
                _g().cbg_builder_free(self.handle)
                self.handle = None
        except Exception:
            pass


class Backend:
    """compute.Backend (compute.go:68-102) + DataInterface (buffer.go:46-61)."""

    def __init__(self, config: str = ""):
        h = C.c_void_p()
        check(_g().cbg_backend_new(config.encode(), C.byref(h)))
        self.handle = h

    def Name(self) -> str:
        return _g().cbg_backend_name(self.handle).decode()

    def String(self) -> str:
        return self.Name()

    def Description(self) -> str:
        return _g().cbg_backend_description(self.handle).decode()

    def NumDevices(self) -> int:
        return _g().cbg_backend_num_devices(self.handle)

    def DeviceDescription(self, deviceNum: int) -> str:
        buf = C.create_string_buffer(256)
        check(_g().cbg_backend_device_description(self.handle, deviceNum, buf, 256))
        return buf.value.decode()

    def Capabilities(self) -> Capabilities:
        ops, dts = (C.c_int32 * 32)(), (C.c_int32 * 32)()
        no, nd = C.c_int(32), C.c_int(32)
        check(_g().cbg_backend_capabilities(self.handle, ops, C.byref(no), dts, C.byref(nd)))
        return Capabilities(Operations={ops[i]: True for i in range(no.value)},
                            DTypes={dts[i]: True for i in range(nd.value)})

    def Builder(self, name: str) -> Builder:
        h = C.c_void_p()
        check(_g().cbg_builder_new(self.handle, name.encode(), C.byref(h)))
        return Builder(h, self, name)

    # ---- DataInterface
    def BufferFromFlatData(self, deviceNum: int, flat: np.ndarray, shape: Shape) -> Buffer:
        if shape.dtype in (dv.I4, dv.U4):        # packed sub-byte dtypes come as bytes, two elements each (buffer.go:47-49)
            a = np.ascontiguousarray(flat, np.uint8)
            if a.size != (shape.size() + 1) // 2:
                raise BackendError(_lib.ERR_INVALID_ARG, f"BufferFromFlatData: flat has {a.size} bytes, packed shape needs {(shape.size() + 1) // 2}")
        else:
            carrier = dv.NP_CARRIER.get(shape.dtype)
            a = flat if (isinstance(flat, np.ndarray) and flat.dtype == carrier and flat.flags.c_contiguous) else np.ascontiguousarray(flat, carrier)
            if a.size != shape._c_dims()[0]:
                raise BackendError(_lib.ERR_INVALID_ARG, f"BufferFromFlatData: flat has {a.size} elements, shape needs {shape.size()}")
        h = C.c_void_p()
        check(_g().cbg_buffer_from_flat(self.handle, deviceNum, a.__array_interface__["data"][0], shape.dtype, len(shape.dimensions),
                                        shape._c_dims()[1], C.byref(h)))
        return Buffer(h, self)

    def HasSharedBuffers(self) -> bool:
        return False

    def NewSharedBuffer(self, deviceNum: int, shape: Shape):
        raise BackendError(_lib.ERR_INVALID_ARG, "NewSharedBuffer: the cuda backend has no shared buffers")

    def Finalize(self) -> None:
        if self.handle:
            check(_g().cbg_backend_finalize(self.handle))

    def IsFinalized(self) -> bool:
        return bool(_g().cbg_backend_is_finalized(self.handle))


def New(config: str = "") -> Backend:
    """compute.NewWithConfig("cuda:<config>")."""
    return Backend(config)


def exec_graph(backend: Backend, inputs: Sequence[Tuple[np.ndarray, int]], build_fn, default_device: int = 0):
    """The reference's testutil.Exec helper (support/testutil/exec.go:14-76): one parameter per
    input (array, dtype), build, compile, execute, and return the outputs as numpy arrays."""
    builder = backend.Builder("test")
    fn = builder.Main()
    params, bufs = [], []
    for i, (arr, dtype) in enumerate(inputs):
        arr = np.asarray(arr)
        shape = make_shape(dtype, *arr.shape)
        params.append(fn.Parameter(f"x{i}", shape))
        bufs.append(backend.BufferFromFlatData(default_device, arr, shape))
    outs = build_fn(fn, params)
    if isinstance(outs, Value):
        outs = [outs]
    fn.Return(list(outs))
    exe = builder.Compile()
    try:
        results = exe.Execute(bufs, None, default_device)
        arrays = [r.ToNumpy() for r in results]
        shapes = [r.Shape() for r in results]
        for r in results:
            r.Finalize()
    finally:
        for b in bufs:
            b.Finalize()
        exe.Finalize()
    return arrays, shapes
