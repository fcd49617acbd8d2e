"""Thin object layer over the C ABI: device memory, streams, events and plans."""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import numpy as np

from . import _lib
from ._lib import DotDesc, QDenseDesc, QDenseMember, SdpaDesc, check

# dtype codes of gomlx/compute dtypes/dtype_enum.go (also cb_dtype in cudabackend.h)
INVALID, BOOL, I8, I16, I32, I64, U8, U16, U32, U64, F16, F32, F64, BF16 = range(14)
F8E5M2, F8E4M3FN = 19, 20
I4, U4 = 21, 22          # packed two per byte, low nibble first: quantized dense weights only
DTYPE_SIZE = {BOOL: 1, I8: 1, U8: 1, I16: 2, U16: 2, F16: 2, BF16: 2, I32: 4, U32: 4, F32: 4,
              I64: 8, U64: 8, F64: 8, F8E5M2: 1, F8E4M3FN: 1}
# numpy carrier of each dtype; half types travel as uint16 bit patterns
NP_CARRIER = {BOOL: np.bool_, I8: np.int8, U8: np.uint8, I16: np.int16, U16: np.uint16,
              F16: np.uint16, BF16: np.uint16, I32: np.int32, U32: np.uint32, F32: np.float32,
              I64: np.int64, U64: np.uint64, F64: np.float64}

ACT_NONE, ACT_GELU, ACT_RELU, ACT_SILU, ACT_HARDSWISH, ACT_TANH = range(6)
SCALE_REF, SCALE_CHANNEL, SCALE_KGROUP = range(3)
QDENSE_AUTO, QDENSE_GENERIC, QDENSE_DECODE_MMA, QDENSE_PREFILL, QDENSE_DECODE_TC = range(5)
QUANT_LINEAR, QUANT_NF4, QUANT_GGML = 0, 1, 2
GGML_Q4_0, GGML_Q8_0, GGML_IQ4_NL, GGML_Q4_K, GGML_Q6_K = 0, 1, 2, 5, 7       # compute.GGMLQuantType (fused_ops.go:132-145)
DOT_AUTO, DOT_GENERIC, DOT_TCGEN05, DOT_TCGEN05_EXACT = range(4)
SDPA_AUTO, SDPA_GENERIC, SDPA_FLASH, SDPA_DECODE, SDPA_TILE = range(5)
LAYOUT_BHSD, LAYOUT_BSHD = 0, 1
MASK_NONE, MASK_BOOL, MASK_ADDITIVE = range(3)


def init() -> int:
    """Number of visible CUDA devices; raises BackendError when there is none."""
    n = C.c_int(0)
    check(_lib.load().cb_init(C.byref(n)))
    return n.value


def device_description(dev: int = 0) -> str:
    buf = C.create_string_buffer(256)
    check(_lib.load().cb_device_desc(dev, buf, 256))
    return buf.value.decode()


def sm_count(dev: int = 0) -> int:
    n = C.c_int(0)
    check(_lib.load().cb_device_sm_count(dev, C.byref(n)))
    return n.value


class Stream:
    def __init__(self, dev: int = 0):
        self.dev = dev
        h = C.c_void_p()
        check(_lib.load().cb_stream_create(dev, C.byref(h)))
        self.handle = h

    def sync(self) -> None:
        check(_lib.load().cb_stream_sync(self.dev, self.handle))

    def wait_event(self, event: "Event") -> None:
        """Work submitted to this stream from now on starts after `event` has completed."""
        check(_lib.load().cb_stream_wait_event(self.dev, self.handle, event.handle))

    def close(self) -> None:
        if self.handle:
            _lib.load().cb_stream_destroy(self.dev, self.handle)
            self.handle = None


class Event:
    def __init__(self, dev: int = 0):
        self.dev = dev
        h = C.c_void_p()
        check(_lib.load().cb_event_create(dev, C.byref(h)))
        self.handle = h

    def record(self, stream: Optional[Stream]) -> None:
        check(_lib.load().cb_event_record(self.dev, self.handle, stream.handle if stream else None))

    def elapsed_ms(self, stop: "Event") -> float:
        ms = C.c_float(0)
        check(_lib.load().cb_event_elapsed_ms(self.handle, stop.handle, C.byref(ms)))
        return ms.value

    def close(self) -> None:
        if self.handle:
            _lib.load().cb_event_destroy(self.dev, self.handle)
            self.handle = None


IPC_HANDLE_BYTES = 64


def ipc_export(mem: "DeviceMem") -> bytes:
    """A handle other processes on this machine can open to reach `mem` (its base pointer)."""
    buf = C.create_string_buffer(IPC_HANDLE_BYTES)
    check(_lib.load().cb_ipc_export(mem.dev, mem.ptr, buf))
    return buf.raw


def ipc_open(dev: int, handle: bytes) -> int:
    """Maps another process's allocation; returns a device pointer valid in this process."""
    p = C.c_void_p()
    check(_lib.load().cb_ipc_open(dev, handle, C.byref(p)))
    return p.value


def ipc_close(dev: int, ptr: int) -> None:
    check(_lib.load().cb_ipc_close(dev, ptr))


def peer_signal(dev: int, flag_arrays: Sequence[int], slot: int, stream=None) -> None:
    """After the work already in `stream`: adds 1 to word `slot` of every rank's flag array."""
    arr = (C.c_void_p * len(flag_arrays))(*flag_arrays)
    check(_lib.load().cb_peer_signal(dev, arr, len(flag_arrays), slot, stream.handle if stream else None))


def peer_wait(dev: int, flags: int, n_flags: int, target: int, status_word: int, stream=None) -> None:
    """Enqueues a bounded wait until flags[0..n_flags) have all reached `target`."""
    check(_lib.load().cb_peer_wait(dev, flags, n_flags, target & 0xFFFFFFFF, status_word, stream.handle if stream else None))


class PeerBarrier:
    """cb_peer_signal_wait with its argument array built once: one call per step signals this rank's slices and waits
    for everyone's."""

    def __init__(self, dev: int, flag_arrays: Sequence[int], rank: int, local_flags: int, status_word: int):
        self.dev, self.rank, self.n = dev, rank, len(flag_arrays)
        self._arr = (C.c_void_p * self.n)(*flag_arrays)
        self.local, self.status = local_flags, status_word

    def signal_wait(self, target: int, stream=None) -> None:
        check(_lib.load().cb_peer_signal_wait(self.dev, self._arr, self.n, self.rank, self.local, target & 0xFFFFFFFF, self.status,
                                              stream.handle if stream else None))


REDUCE_SUM, REDUCE_PRODUCT, REDUCE_MAX, REDUCE_MIN = range(4)
BIN_ADD, BIN_SUB, BIN_MUL, BIN_DIV, BIN_MAX, BIN_MIN = range(6)
UN_NEG, UN_RSQRT, UN_SQRT, UN_EXP, UN_LOGISTIC, UN_TANH = range(6)
COMM_ID_BYTES = 128


class Comm:
    """One rank of a communicator (one process per GPU).  `unique_id()` is called on one rank and its
    128 bytes are handed to the others by the host program; then every rank constructs its Comm."""

    @staticmethod
    def unique_id() -> bytes:
        buf = C.create_string_buffer(COMM_ID_BYTES)
        check(_lib.load().cb_comm_unique_id(buf))
        return buf.raw

    def __init__(self, dev: int, nranks: int, rank: int, uid: bytes, timeout_s: float = 0.0):
        """`timeout_s` > 0 makes a non-blocking communicator: the initialisation and every enqueue
        are bounded by it, and when it passes the communicator is aborted and BackendError(ERR_TIMEOUT)
        raised.  0 keeps the blocking kind (cheaper per call), watched through `sync`.
        dev < 0: the current device."""
        assert len(uid) == COMM_ID_BYTES
        self.dev, self.nranks, self.rank = dev, nranks, rank
        h = C.c_void_p()
        check(_lib.load().cb_comm_init_rank_timeout(dev, nranks, rank, uid, float(timeout_s), C.byref(h)))
        self.handle = h

    def check(self) -> None:
        """One poll of the communicator's asynchronous state; raises once NCCL has reported an error."""
        check(_lib.load().cb_comm_check(self.handle))

    def sync(self, stream=None, timeout_s: float = 0.0) -> None:
        """Waits for `stream` while watching the communicator; aborts it and raises ERR_TIMEOUT when the limit passes."""
        check(_lib.load().cb_comm_sync(self.handle, stream.handle if stream else None, float(timeout_s)))

    def allgather(self, send: int, recv: int, bytes_per_rank: int, stream=None) -> None:
        check(_lib.load().cb_comm_allgather(self.handle, send, recv, bytes_per_rank, stream.handle if stream else None))

    def allreduce(self, send: int, recv: int, count: int, dtype: int, op: int = REDUCE_SUM, stream=None) -> None:
        check(_lib.load().cb_comm_allreduce(self.handle, send, recv, count, dtype, op, stream.handle if stream else None))

    def close(self) -> None:
        if self.handle:
            _lib.load().cb_comm_destroy(self.handle)
            self.handle = None


class DeviceMem:
    """A device allocation owned by this object."""

    def __init__(self, nbytes: int, dev: int = 0):
        self.dev = dev
        self.nbytes = int(nbytes)
        p = C.c_void_p()
        check(_lib.load().cb_alloc(dev, self.nbytes, C.byref(p)))
        self.ptr = p.value

    @classmethod
    def from_numpy(cls, a: np.ndarray, dev: int = 0, stream: Optional[Stream] = None) -> "DeviceMem":
        a = np.ascontiguousarray(a)
        m = cls(a.nbytes, dev)
        m.upload(a, stream)
        return m

    def upload(self, a: np.ndarray, stream: Optional[Stream] = None) -> None:
        a = np.ascontiguousarray(a)
        assert a.nbytes <= self.nbytes
        check(_lib.load().cb_h2d(self.dev, self.ptr, a.ctypes.data, a.nbytes, stream.handle if stream else None))

    def download(self, shape, np_dtype, stream: Optional[Stream] = None) -> np.ndarray:
        out = np.empty(shape, np_dtype)
        assert out.nbytes <= self.nbytes
        check(_lib.load().cb_d2h(self.dev, out.ctypes.data, self.ptr, out.nbytes, stream.handle if stream else None))
        return out

    def zero(self, stream: Optional[Stream] = None) -> None:
        check(_lib.load().cb_memset(self.dev, self.ptr, 0, self.nbytes, stream.handle if stream else None))

    def free(self) -> None:
        if self.ptr:
            _lib.load().cb_free(self.dev, self.ptr)
            self.ptr = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class PinnedHost:
    """Page-locked host buffer exposed as a numpy array (for timed H2D / D2H copies)."""

    def __init__(self, shape, np_dtype):
        self.shape = tuple(shape)
        self.dtype = np.dtype(np_dtype)
        n = int(np.prod(self.shape)) * self.dtype.itemsize
        p = C.c_void_p()
        check(_lib.load().cb_host_alloc(max(n, 1), C.byref(p)))
        self.ptr = p.value
        self.nbytes = n
        buf = (C.c_uint8 * max(n, 1)).from_address(self.ptr)
        self.array = np.frombuffer(buf, dtype=self.dtype, count=int(np.prod(self.shape))).reshape(self.shape)

    def free(self) -> None:
        if self.ptr:
            self.array = None
            _lib.load().cb_host_free(self.ptr)
            self.ptr = None


class Plan:
    """An immutable launch plan: kernel variant, grid and workspace size, chosen by shape and dtype."""

    def __init__(self, handle: C.c_void_p, dev: int):
        self.handle = handle
        self.dev = dev
        lib = _lib.load()
        n = C.c_size_t(0)
        check(lib.cb_plan_workspace_bytes(handle, C.byref(n)))
        self.workspace_bytes = n.value
        self.kernel_name = lib.cb_plan_kernel_name(handle).decode()
        b, t, s = C.c_int(0), C.c_int(0), C.c_int(0)
        check(lib.cb_plan_grid(handle, C.byref(b), C.byref(t), C.byref(s)))
        self.blocks, self.threads, self.dyn_smem = b.value, t.value, s.value

    # --- constructors ------------------------------------------------------
    @classmethod
    def qdense(cls, M, K, N, x_dtype=F32, w_dtype=I8, scale_layout=SCALE_REF, block_size=1,
               has_zero_point=False, has_bias=False, activation=ACT_NONE, variant=QDENSE_AUTO, dev=0,
               gather_ranks=0, gather_rank=0, scheme=QUANT_LINEAR, ggml_type=0) -> "Plan":
        d = QDenseDesc(M, K, N, x_dtype, w_dtype, scale_layout, block_size, int(has_zero_point),
                       int(has_bias), activation, variant, gather_ranks, gather_rank, scheme, ggml_type)
        h = C.c_void_p()
        check(_lib.load().cb_plan_qdense(dev, C.byref(d), C.byref(h)))
        return cls(h, dev)

    @classmethod
    def qdense_group(cls, M, K, members, x_dtype=F32, w_dtype=I8, scale_layout=SCALE_CHANNEL, block_size=0, dev=0,
                     gather_ranks=0, gather_rank=0) -> "Plan":
        """Several independent decode-shaped projections sharing M and K as one launch.  `members` is a
        sequence of (N, has_bias, activation); launch inputs are x, w, scales, bias? per member in order."""
        d = QDenseDesc(M, K, 0, x_dtype, w_dtype, scale_layout, block_size, 0, 0, ACT_NONE, QDENSE_DECODE_TC,
                       gather_ranks, gather_rank, QUANT_LINEAR, 0)
        arr = (QDenseMember * max(len(members), 1))(*[QDenseMember(int(n), int(b), int(a)) for n, b, a in members])
        h = C.c_void_p()
        check(_lib.load().cb_plan_qdense_group(dev, C.byref(d), arr, len(members), C.byref(h)))
        return cls(h, dev)

    @classmethod
    def dot(cls, B, M, N, K, in_dtype=F32, out_dtype=INVALID, rhs_transposed=False, variant=DOT_AUTO, dev=0,
            has_bias=False, activation=ACT_NONE) -> "Plan":
        d = DotDesc(B, M, N, K, int(rhs_transposed), in_dtype, out_dtype, variant, int(has_bias), activation)
        h = C.c_void_p()
        check(_lib.load().cb_plan_dot(dev, C.byref(d), C.byref(h)))
        return cls(h, dev)

    @classmethod
    def embedding_lookup(cls, vocab, bytes_per_row, n_indices, index_dtype, ggml_type, dev=0) -> "Plan":
        """QuantizedEmbeddingLookup: launch inputs table, indices; output float32 [n_indices, K]."""
        h = C.c_void_p()
        check(_lib.load().cb_plan_embedding_lookup(dev, vocab, bytes_per_row, n_indices, index_dtype, ggml_type, C.byref(h)))
        return cls(h, dev)

    @classmethod
    def gelu(cls, dtype, n, exact=True, dev=0) -> "Plan":
        h = C.c_void_p()
        check(_lib.load().cb_plan_gelu(dev, dtype, n, int(exact), C.byref(h)))
        return cls(h, dev)

    @classmethod
    def softmax(cls, dtype, outer, axis_size, inner=1, dev=0) -> "Plan":
        h = C.c_void_p()
        check(_lib.load().cb_plan_softmax(dev, dtype, outer, axis_size, inner, C.byref(h)))
        return cls(h, dev)

    @classmethod
    def layernorm(cls, dtype, rows, norm_size, epsilon=1e-5, has_gamma=False, has_beta=False, dev=0) -> "Plan":
        h = C.c_void_p()
        check(_lib.load().cb_plan_layernorm(dev, dtype, rows, norm_size, float(epsilon), int(has_gamma), int(has_beta), C.byref(h)))
        return cls(h, dev)

    @classmethod
    def binary(cls, op, dtype, lhs_dims, rhs_dims, dev=0) -> "Plan":
        """Element-wise binary op; both shapes given with the same rank, dimensions equal or 1 (broadcast)."""
        r = len(lhs_dims)
        h = C.c_void_p()
        check(_lib.load().cb_plan_binary(dev, op, dtype, r, (C.c_int64 * max(r, 1))(*lhs_dims), (C.c_int64 * max(r, 1))(*rhs_dims), C.byref(h)))
        return cls(h, dev)

    @classmethod
    def unary(cls, op, dtype, n, dev=0) -> "Plan":
        h = C.c_void_p()
        check(_lib.load().cb_plan_unary(dev, op, dtype, n, C.byref(h)))
        return cls(h, dev)

    @classmethod
    def reduce(cls, op, dtype, dims, reduced_axes, dev=0) -> "Plan":
        r = len(dims)
        flags = [1 if a in set(reduced_axes) else 0 for a in range(r)]
        h = C.c_void_p()
        check(_lib.load().cb_plan_reduce(dev, op, dtype, r, (C.c_int64 * max(r, 1))(*dims), (C.c_int32 * max(r, 1))(*flags), C.byref(h)))
        return cls(h, dev)

    @classmethod
    def broadcast_in_dim(cls, dtype, dims, out_dims, broadcast_axes, dev=0) -> "Plan":
        r, ro = len(dims), len(out_dims)
        h = C.c_void_p()
        check(_lib.load().cb_plan_broadcast_in_dim(dev, dtype, r, (C.c_int64 * max(r, 1))(*dims), ro, (C.c_int64 * max(ro, 1))(*out_dims),
                                                   (C.c_int32 * max(r, 1))(*broadcast_axes), C.byref(h)))
        return cls(h, dev)

    @classmethod
    def rms_norm(cls, dtype, rows, row_size, epsilon=1e-5, has_gamma=True, dev=0) -> "Plan":
        h = C.c_void_p()
        check(_lib.load().cb_plan_rms_norm(dev, dtype, rows, row_size, float(epsilon), int(has_gamma), C.byref(h)))
        return cls(h, dev)

    @classmethod
    def sdpa(cls, B, Hq, Hkv, S, Skv, D, dtype=F32, layout=LAYOUT_BHSD, scale=0.0, causal=False,
             mask_kind=MASK_NONE, mask_dims: Sequence[int] = (), has_seq_lens=False,
             bias_dims: Sequence[int] = (), variant=SDPA_AUTO, dev=0) -> "Plan":
        d = SdpaDesc()
        d.B, d.Hq, d.Hkv, d.S, d.Skv, d.D = B, Hq, Hkv, S, Skv, D
        d.layout, d.dtype, d.scale, d.causal = layout, dtype, float(scale), int(causal)
        d.mask_kind, d.mask_rank = mask_kind, len(mask_dims)
        for i, v in enumerate(list(mask_dims)[:4]):
            d.mask_dims[i] = v
        d.has_seq_lens = int(has_seq_lens)
        d.bias_rank = len(bias_dims)
        for i, v in enumerate(list(bias_dims)[:4]):
            d.bias_dims[i] = v
        d.variant = variant
        if len(mask_dims) > 4 or len(bias_dims) > 4:
            raise _lib.BackendError(_lib.ERR_INVALID_ARG, "mask/bias must have rank 2, 3, or 4")
        h = C.c_void_p()
        check(_lib.load().cb_plan_sdpa(dev, C.byref(d), C.byref(h)))
        return cls(h, dev)

    @classmethod
    def copy(cls, dtype, n, dev=0) -> "Plan":
        h = C.c_void_p()
        check(_lib.load().cb_plan_copy(dev, dtype, n, C.byref(h)))
        return cls(h, dev)

    @classmethod
    def convert(cls, from_dtype, to_dtype, n, dev=0) -> "Plan":
        h = C.c_void_p()
        check(_lib.load().cb_plan_convert(dev, from_dtype, to_dtype, n, C.byref(h)))
        return cls(h, dev)

    @classmethod
    def iota(cls, dtype, dims, axis, dev=0) -> "Plan":
        arr = (C.c_int64 * max(len(dims), 1))(*dims)
        h = C.c_void_p()
        check(_lib.load().cb_plan_iota(dev, dtype, len(dims), arr, axis, C.byref(h)))
        return cls(h, dev)

    @classmethod
    def slice(cls, dtype, dims, starts, limits, strides=None, dev=0) -> "Plan":
        r = len(dims)
        mk = lambda v: (C.c_int64 * max(r, 1))(*v)
        h = C.c_void_p()
        check(_lib.load().cb_plan_slice(dev, dtype, r, mk(dims), mk(starts), mk(limits),
                                        mk(strides if strides is not None else [1] * r), C.byref(h)))
        return cls(h, dev)

    @classmethod
    def transpose(cls, dtype, dims, perm, dev=0) -> "Plan":
        r = len(dims)
        h = C.c_void_p()
        check(_lib.load().cb_plan_transpose(dev, dtype, r, (C.c_int64 * max(r, 1))(*dims),
                                            (C.c_int32 * max(r, 1))(*perm), C.byref(h)))
        return cls(h, dev)

    # --- execution -----------------------------------------------------------
    def new_workspace(self) -> Optional[DeviceMem]:
        """Allocates and prepares a workspace for this plan (None when it needs none)."""
        if self.workspace_bytes == 0:
            return None
        ws = DeviceMem(self.workspace_bytes, self.dev)
        check(_lib.load().cb_plan_prepare_workspace(self.handle, ws.ptr, None))
        check(_lib.load().cb_stream_sync(self.dev, None))
        return ws

    def launch(self, inputs: Sequence[int], outputs: Sequence[int], workspace: Optional[int] = None,
               stream: Optional[Stream] = None) -> None:
        ins = (C.c_void_p * max(len(inputs), 1))(*inputs)
        outs = (C.c_void_p * max(len(outputs), 1))(*outputs)
        check(_lib.load().cb_launch(self.handle, ins, len(inputs), outs, len(outputs), workspace,
                                    stream.handle if stream else None))

    def check_status(self, workspace: Optional[int]) -> None:
        check(_lib.load().cb_plan_check_status(self.handle, workspace))

    def bind(self, inputs: Sequence[int], outputs: Sequence[int], workspace: Optional[int] = None) -> "Bound":
        """Fixes the buffers of this plan: later launches are only the kernel launches."""
        ins = (C.c_void_p * max(len(inputs), 1))(*inputs)
        outs = (C.c_void_p * max(len(outputs), 1))(*outputs)
        h = C.c_void_p()
        check(_lib.load().cb_plan_bind(self.handle, ins, len(inputs), outs, len(outputs), workspace, C.byref(h)))
        return Bound(h, self)

    def destroy(self) -> None:
        if self.handle:
            _lib.load().cb_plan_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass


class Bound:
    """A plan bound to its buffers (cb_plan_bind); keeps the plan alive."""

    def __init__(self, handle: C.c_void_p, plan: Plan):
        self.handle = handle
        self.plan = plan

    def launch(self, stream: Optional[Stream] = None) -> None:
        check(_lib.load().cb_bound_launch(self.handle, stream.handle if stream else None))

    def destroy(self) -> None:
        if self.handle:
            _lib.load().cb_bound_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass


class BoundSequence:
    """A step's launches, issued by one C call (cb_bound_launch_many)."""

    def __init__(self, bounds: Sequence[Bound]):
        self.bounds = list(bounds)
        self._arr = (C.c_void_p * max(len(self.bounds), 1))(*[b.handle for b in self.bounds])

    def launch(self, stream: Optional[Stream] = None) -> None:
        check(_lib.load().cb_bound_launch_many(self._arr, len(self.bounds), stream.handle if stream else None))
