"""ctypes binding of libq4b200.so and thin object wrappers.

Mirrors the reference's C conventions for this path (int status + caller-supplied
error buffer, opaque handles, the library owns device memory): a nonzero status
becomes a Q4Error carrying the library's message and the status code
(1 bad argument, 2 device failure, 3 load failure -- qwen38_m3_decode.h:20-25).
"""
from __future__ import annotations

import ctypes
import os
import re

import numpy as np

F16, F32, BF16, NONE = 0, 1, 2, -1
_HERE = os.path.dirname(os.path.abspath(__file__))
_HEADER = os.path.join(os.path.dirname(_HERE), "include", "q4b200.h")
_ERR = 512


class Q4Error(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"libq4b200 status {status}: {message}")
        self.status = status
        self.message = message


def library_path() -> str:
    return os.path.join(_HERE, "libq4b200.so")


def declared_symbols() -> list[str]:
    """Every function include/q4b200.h declares."""
    with open(_HEADER) as handle:
        text = handle.read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(q4b_[a-z0-9_]+)\s*\(", text)))


_lib = None
_vp, _cp, _sz = ctypes.c_void_p, ctypes.c_char_p, ctypes.c_size_t
_u32, _u64, _int = ctypes.c_uint32, ctypes.c_uint64, ctypes.c_int


def library() -> ctypes.CDLL:
    """Load libq4b200.so, building it first when nvcc is available.

    Raises instead of degrading: there is no other implementation to fall to."""
    global _lib
    if _lib is not None:
        return _lib
    path = os.environ.get("Q4B_LIBRARY") or library_path()  # another build of the same library
    from . import _build
    try:
        if path == library_path() and _build.stale():
            _build.build()
    except Exception as error:  # no nvcc on this machine: use the shipped binary
        if not os.path.exists(path):
            raise RuntimeError(f"libq4b200.so is missing and cannot be built: {error}") from error
    lib = ctypes.CDLL(path)
    err = [_cp, _sz]
    spec = {
        "q4b_context_open": (_vp, [_int] + err),
        "q4b_context_close": (None, [_vp]),
        "q4b_device_count": (_int, []),
        "q4b_context_stream": (_vp, [_vp]),
        "q4b_context_set_variant": (None, [_vp, _int]),
        "q4b_context_launch_count": (_u64, [_vp]),
        "q4b_alloc": (_int, [_vp, _sz, ctypes.POINTER(_vp)] + err),
        "q4b_free": (_int, [_vp, _vp]),
        "q4b_alloc_host": (_int, [_vp, _sz, ctypes.POINTER(_vp)] + err),
        "q4b_free_host": (_int, [_vp, _vp]),
        "q4b_copy_to_device": (_int, [_vp, _vp, _vp, _sz] + err),
        "q4b_copy_to_host": (_int, [_vp, _vp, _vp, _sz] + err),
        "q4b_weight_upload": (_int, [_vp, _vp, _vp, _u32, _u32, _u32, _u32, ctypes.POINTER(_vp)] + err),
        "q4b_weight_upload_planes": (_int, [_vp, _vp, _vp, _vp, _int, _u32, _u32, _u32, _u32,
                                            ctypes.POINTER(_vp)] + err),
        "q4b_weight_upload_q8": (_int, [_vp, _vp, _vp, _vp, _u32, _u32, _u32, _u32, ctypes.POINTER(_vp)] + err),
        "q4b_planes_narrowed": (_u64, [_vp, _vp, _int, _u64]),
        "q4b_weight_from_device": (_int, [_vp, _vp, _vp, _u32, _u32, _u32, _u32, ctypes.POINTER(_vp)] + err),
        "q4b_weight_synth": (_int, [_vp, _u64, _u32, _u32, _u32, _u32, _u32, ctypes.POINTER(_vp)] + err),
        "q4b_synth_x": (_int, [_vp, _u64, _u64, _vp, _u64, _u64] + err),
        "q4b_weight_free": (None, [_vp, _vp]),
        "q4b_weight_info": (_int, [_vp, ctypes.POINTER(_u32), ctypes.POINTER(_u32), ctypes.POINTER(_u64)]),
        "q4b_weight_unpack": (_int, [_vp, _vp, _vp, _vp, _vp] + err),
        "q4b_matmul": (_int, [_vp, _vp, _vp, _int, _u32, _vp, _int, _u32, _vp, _int, _u32] + err),
        "q4b_matmul_no_alloc": (_int, [_vp, _vp, _vp, _int, _u32, _vp, _int, _u32] + err),
        "q4b_weight_rows": (_int, [_vp, _u32, _u32, ctypes.POINTER(_vp)] + err),
        "q4b_matmul_rows": (_int, [_vp, _vp, _vp, _u32, _vp, _int, _u32, _vp, _int, _u32] + err),
        "q4b_matmul_group": (_int, [_vp, ctypes.POINTER(_vp), _int, _vp, _int, _u32, ctypes.POINTER(_vp),
                                    _int, ctypes.POINTER(_u32)] + err),
        "q4b_gate_up_silu": (_int, [_vp, _vp, _vp, _vp, _int, _u32, _vp, _int, _u32] + err),
        "q4b_matmul_host": (_int, [_vp, _vp, _vp, _int, _u32, _vp, _int, ctypes.POINTER(ctypes.c_double)] + err),
        "q4b_gate_up_silu_host": (_int, [_vp, _vp, _vp, _vp, _int, _u32, _vp, _int,
                                         ctypes.POINTER(ctypes.c_double)] + err),
        "q4b_context_push_outputs": (_int, [_vp, _u32, ctypes.POINTER(_vp), _int]),
        "q4b_barrier_create": (_int, [_vp, _u32, _u32, ctypes.POINTER(_vp)] + err),
        "q4b_barrier_counter": (_vp, [_vp]),
        "q4b_barrier_set_peer": (_int, [_vp, _u32, _vp]),
        "q4b_barrier_queue": (_int, [_vp, _vp] + err),
        "q4b_barrier_free": (None, [_vp, _vp]),
        "q4b_embedding_lookup": (_int, [_vp, _vp, _vp, _u32, _vp, _int] + err),
        "q4b_rmsnorm": (_int, [_vp, _vp, _int, _vp, _vp, _u32, _u32, ctypes.c_float] + err),
        "q4b_sequence_create": (_int, [_vp, _u32, _u32, _u32, ctypes.POINTER(_vp)] + err),
        "q4b_sequence_add_matmul": (_int, [_vp, ctypes.POINTER(_vp), _int, _vp, ctypes.POINTER(_vp),
                                           ctypes.POINTER(_u32), _int] + err),
        "q4b_sequence_add_gate_up": (_int, [_vp, _vp, _vp, _vp, _vp, _u32, _int] + err),
        "q4b_sequence_add_projection": (_int, [_vp, _vp, _vp, _int, _vp, _int, _u32, _vp, _int, _u32] + err),
        "q4b_sequence_set_peer_output": (_int, [_vp, _u32, _u32, _u32, _vp]),
        "q4b_sequence_set_job_blocks": (_int, [_vp, _u32, _u32]),
        "q4b_sequence_finalize": (_int, [_vp, _vp] + err),
        "q4b_sequence_done_counters": (_vp, [_vp]),
        "q4b_sequence_set_peer_counters": (_int, [_vp, _u32, _vp]),
        "q4b_sequence_launch": (_int, [_vp, _vp] + err),
        "q4b_sequence_profile": (_int, [_vp, _vp, ctypes.POINTER(_u64), _u32, ctypes.POINTER(_u32)] + err),
        "q4b_sequence_free": (None, [_vp, _vp]),
        "q4b_ipc_export": (_int, [_vp, _vp, _vp] + err),
        "q4b_ipc_open": (_int, [_vp, _vp, ctypes.POINTER(_vp)] + err),
        "q4b_ipc_close": (_int, [_vp, _vp]),
        "q4b_copy_2d": (_int, [_vp, _vp, _sz, _vp, _sz, _sz, _sz] + err),
        "q4b_comm_unique_id": (_int, [_vp] + err),
        "q4b_comm_create": (_int, [_vp, _u32, _u32, _vp, ctypes.POINTER(_vp)] + err),
        "q4b_comm_world": (_u32, [_vp]),
        "q4b_comm_rank": (_u32, [_vp]),
        "q4b_all_gather": (_int, [_vp, _vp, _vp, _vp, _sz] + err),
        "q4b_all_gather_columns": (_int, [_vp, _vp, _vp, _vp, _u32, _u32, _u32, _vp] + err),
        "q4b_comm_free": (None, [_vp, _vp]),
        "q4b_probe_read": (_int, [_vp, _int, _sz, _int, _u32, _u32, _int, ctypes.POINTER(ctypes.c_double)] + err),
        "q4b_push_rows": (_int, [_vp, _vp, ctypes.POINTER(_vp), _u32, _u32, _u32, _u32] + err),
        "q4b_probe_signal": (_int, [_vp, _vp, _vp, _u32, _u32, _u32, _int, _int, ctypes.POINTER(ctypes.c_double)] + err),
        "q4b_timer_start": (_int, [_vp] + err),
        "q4b_sync": (_int, [_vp, ctypes.POINTER(ctypes.c_double)] + err),
        "q4b_graph_begin": (_int, [_vp] + err),
        "q4b_graph_end": (_int, [_vp, ctypes.POINTER(_vp)] + err),
        "q4b_graph_launch": (_int, [_vp, _vp] + err),
        "q4b_graph_free": (None, [_vp]),
    }
    for name, (restype, argtypes) in spec.items():
        function = getattr(lib, name)
        function.restype = restype
        function.argtypes = argtypes
    _lib = lib
    return lib


def _np_dtype_code(array: np.ndarray) -> int:
    if array.dtype == np.float16:
        return F16
    if array.dtype == np.float32:
        return F32
    raise TypeError(f"activations must be float16 or float32, not {array.dtype}")


_NP_OF = {F16: np.float16, F32: np.float32}


class DeviceBuffer:
    """A plain device allocation owned by a context."""

    def __init__(self, context: "Q4Context", nbytes: int):
        self.context = context
        self.nbytes = int(nbytes)
        pointer = _vp()
        context._check(library().q4b_alloc(context.handle, self.nbytes, ctypes.byref(pointer),
                                           context._err, _ERR))
        self.ptr = pointer.value

    def upload(self, array: np.ndarray) -> "DeviceBuffer":
        array = np.ascontiguousarray(array)
        assert array.nbytes <= self.nbytes
        self.context._check(library().q4b_copy_to_device(self.context.handle, self.ptr, array.ctypes.data,
                                                         array.nbytes, self.context._err, _ERR))
        self.context.sync()  # the NumPy temporary may die after this call
        return self

    def download(self, dtype, shape) -> np.ndarray:
        out = np.empty(shape, dtype=dtype)
        assert out.nbytes <= self.nbytes
        self.context._check(library().q4b_copy_to_host(self.context.handle, out.ctypes.data, self.ptr,
                                                       out.nbytes, self.context._err, _ERR))
        self.context.sync()
        return out

    def free(self):
        if self.ptr:
            library().q4b_free(self.context.handle, self.ptr)
            self.ptr = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class Q4Weight:
    """One Q4 matrix (or the N-slice of one) resident in HBM as a tile stream."""

    def __init__(self, context: "Q4Context", handle: int):
        self.context = context
        self.handle = handle
        rows, groups, nbytes = _u32(), _u32(), _u64()
        library().q4b_weight_info(handle, ctypes.byref(rows), ctypes.byref(groups), ctypes.byref(nbytes))
        self.rows, self.groups, self.device_bytes = rows.value, groups.value, nbytes.value
        self.columns = self.groups * 64

    def unpack(self, codes=True, w32=True, w16=True):
        """Device-side dequantisation of the whole shard -> host arrays."""
        shape = (self.rows, self.columns)
        c = np.empty(shape, np.uint8) if codes else None
        a = np.empty(shape, np.float32) if w32 else None
        b = np.empty(shape, np.uint16) if w16 else None
        p = lambda v: None if v is None else v.ctypes.data
        self.context._check(library().q4b_weight_unpack(self.context.handle, self.handle, p(c), p(a), p(b),
                                                        self.context._err, _ERR))
        return c, a, (None if b is None else b.view(np.float16))

    def rows_view(self, row_begin: int, row_count: int) -> "Q4Weight":
        """Rows [row_begin, +row_count) of this weight as a weight of their own, no copy (q4b_weight_rows)."""
        handle = _vp()
        self.context._check(library().q4b_weight_rows(self.handle, row_begin, row_count, ctypes.byref(handle),
                                                      self.context._err, _ERR))
        return Q4Weight(self.context, handle.value)

    def free(self):
        if self.handle:
            library().q4b_weight_free(self.context.handle, self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class Q4Graph:
    def __init__(self, context: "Q4Context", handle: int):
        self.context, self.handle = context, handle

    def launch(self):
        self.context._check(library().q4b_graph_launch(self.context.handle, self.handle,
                                                       self.context._err, _ERR))

    def free(self):
        if self.handle:
            library().q4b_graph_free(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class Q4Sequence:
    """A chain of projections executed by one persistent launch (q4b_sequence)."""

    def __init__(self, context: "Q4Context", m_rows: int, world: int = 1, rank: int = 0):
        self.context, self.m_rows, self.world, self.rank = context, m_rows, world, rank
        handle = _vp()
        context._check(library().q4b_sequence_create(context.handle, m_rows, world, rank, ctypes.byref(handle),
                                                     context._err, _ERR))
        self.handle = handle.value
        self.jobs = 0

    def add_matmul(self, weights, x_ptr: int, y_ptrs, ldys=None, y_dtype: int = F16) -> int:
        count = len(weights)
        handles = (_vp * count)(*[w.handle for w in weights])
        outputs = (_vp * count)(*y_ptrs)
        strides = (_u32 * count)(*(ldys if ldys is not None else [w.rows for w in weights]))
        self.context._check(library().q4b_sequence_add_matmul(self.handle, handles, count, x_ptr, outputs, strides,
                                                              y_dtype, self.context._err, _ERR))
        self.jobs += 1
        return self.jobs - 1

    def add_projection(self, weight, x_ptr: int, x_dtype: int, y_ptr: int, y_dtype: int = F16, ldy=None,
                       residual_ptr=None, residual_dtype: int = NONE, ld_residual: int = 0) -> int:
        """One matrix with fp16 or fp32 x and an optional residual."""
        self.context._check(library().q4b_sequence_add_projection(
            self.handle, weight.handle, x_ptr, x_dtype, y_ptr, y_dtype, weight.rows if ldy is None else ldy,
            residual_ptr, residual_dtype, ld_residual, self.context._err, _ERR))
        self.jobs += 1
        return self.jobs - 1

    def add_gate_up(self, gate, up, x_ptr: int, y_ptr: int, ldy=None, y_dtype: int = F16) -> int:
        self.context._check(library().q4b_sequence_add_gate_up(self.handle, gate.handle, up.handle, x_ptr, y_ptr,
                                                               gate.rows if ldy is None else ldy, y_dtype,
                                                               self.context._err, _ERR))
        self.jobs += 1
        return self.jobs - 1

    def set_peer_output(self, job: int, segment: int, peer_rank: int, peer_ptr: int):
        if library().q4b_sequence_set_peer_output(self.handle, job, segment, peer_rank, peer_ptr) != 0:
            raise Q4Error(1, "invalid peer output")

    def set_job_blocks(self, job: int, blocks_on_all_ranks: int):
        if library().q4b_sequence_set_job_blocks(self.handle, job, blocks_on_all_ranks) != 0:
            raise Q4Error(1, "invalid job block count")

    def finalize(self):
        self.context._check(library().q4b_sequence_finalize(self.context.handle, self.handle,
                                                            self.context._err, _ERR))

    @property
    def done_counters(self) -> int:
        return library().q4b_sequence_done_counters(self.handle)

    def set_peer_counters(self, peer_rank: int, pointer: int):
        if library().q4b_sequence_set_peer_counters(self.handle, peer_rank, pointer) != 0:
            raise Q4Error(1, "invalid peer counters")

    def launch(self):
        self.context._check(library().q4b_sequence_launch(self.context.handle, self.handle,
                                                          self.context._err, _ERR))

    PROFILE_PHASES = ("dependency", "entries", "weights", "tiles", "finish", "total")

    def profile(self):
        """First call: switches the phase clocks on, returns None.  Later calls: [thread blocks, 6] SM clock
        ticks added up by the launches since the previous call (q4b_sequence_profile)."""
        blocks = _u32(0)
        first = not getattr(self, "_profiling", False)
        if first:
            self.context._check(library().q4b_sequence_profile(self.context.handle, self.handle, None, 0,
                                                               ctypes.byref(blocks), self.context._err, _ERR))
            self._profiling = True
            self._profile_blocks = blocks.value
            return None
        out = np.zeros((self._profile_blocks, 6), dtype=np.uint64)
        self.context._check(library().q4b_sequence_profile(
            self.context.handle, self.handle, out.ctypes.data_as(ctypes.POINTER(_u64)), out.size,
            ctypes.byref(blocks), self.context._err, _ERR))
        return out

    def free(self):
        if self.handle:
            library().q4b_sequence_free(self.context.handle, self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class Q4Context:
    """One GPU, one stream (q4b_context)."""

    def __init__(self, device: int = 0):
        self._err = ctypes.create_string_buffer(_ERR)
        self.handle = library().q4b_context_open(device, self._err, _ERR)
        if not self.handle:
            raise Q4Error(2, self._err.value.decode(errors="replace"))
        self.device = device

    # -- plumbing ---------------------------------------------------------
    def _check(self, status: int):
        if status != 0:
            raise Q4Error(status, self._err.value.decode(errors="replace"))

    def close(self):
        if self.handle:
            library().q4b_context_close(self.handle)
            self.handle = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    @property
    def stream(self) -> int:
        return library().q4b_context_stream(self.handle)

    @property
    def launches(self) -> int:
        return int(library().q4b_context_launch_count(self.handle))

    def set_variant(self, variant: int):
        library().q4b_context_set_variant(self.handle, int(variant))

    def alloc(self, nbytes: int) -> DeviceBuffer:
        return DeviceBuffer(self, nbytes)

    def to_device(self, array: np.ndarray) -> DeviceBuffer:
        array = np.ascontiguousarray(array)
        return DeviceBuffer(self, max(array.nbytes, 16)).upload(array)

    def timer_start(self):
        self._check(library().q4b_timer_start(self.handle, self._err, _ERR))

    def sync(self, timed: bool = False) -> float:
        ms = ctypes.c_double(0.0)
        self._check(library().q4b_sync(self.handle, ctypes.byref(ms) if timed else None, self._err, _ERR))
        return ms.value

    # -- loader -----------------------------------------------------------
    def upload(self, quants: np.ndarray, meta: np.ndarray, rows: int, groups: int, row_begin: int = 0,
               row_count: int | None = None) -> Q4Weight:
        """Image segments (quants bytes, interleaved fp16 {scale,bias}) -> HBM."""
        quants = np.ascontiguousarray(quants)
        meta = np.ascontiguousarray(meta)
        handle = _vp()
        count = rows - row_begin if row_count is None else row_count
        self._check(library().q4b_weight_upload(self.handle, quants.ctypes.data, meta.ctypes.data, rows, groups,
                                                row_begin, count, ctypes.byref(handle), self._err, _ERR))
        return Q4Weight(self, handle.value)

    def upload_planes(self, quants, scales, biases, meta_dtype, rows, groups, row_begin=0, row_count=None):
        quants, scales, biases = (np.ascontiguousarray(a) for a in (quants, scales, biases))
        handle = _vp()
        count = rows - row_begin if row_count is None else row_count
        self._check(library().q4b_weight_upload_planes(self.handle, quants.ctypes.data, scales.ctypes.data,
                                                       biases.ctypes.data, meta_dtype, rows, groups, row_begin,
                                                       count, ctypes.byref(handle), self._err, _ERR))
        return Q4Weight(self, handle.value)

    def upload_q8(self, quants, scales_bf16, biases_bf16, rows, groups, row_begin=0, row_count=None):
        """Affine-Q8 planes (codes [rows, K] bytes, bf16 scales / biases [rows, K/64]) -> HBM (q4b_weight_upload_q8)."""
        quants, scales, biases = (np.ascontiguousarray(a) for a in (quants, scales_bf16, biases_bf16))
        handle = _vp()
        count = rows - row_begin if row_count is None else row_count
        self._check(library().q4b_weight_upload_q8(self.handle, quants.ctypes.data, scales.ctypes.data,
                                                   biases.ctypes.data, rows, groups, row_begin, count,
                                                   ctypes.byref(handle), self._err, _ERR))
        return Q4Weight(self, handle.value)

    def synth_weight(self, seed: int, projection: int, rows: int, groups: int, row_begin: int = 0,
                     row_count: int | None = None) -> Q4Weight:
        handle = _vp()
        count = rows - row_begin if row_count is None else row_count
        self._check(library().q4b_weight_synth(self.handle, seed, projection, rows, groups, row_begin, count,
                                               ctypes.byref(handle), self._err, _ERR))
        return Q4Weight(self, handle.value)

    def synth_x(self, seed: int, stream_id: int, m_rows: int, columns: int) -> DeviceBuffer:
        buffer = DeviceBuffer(self, m_rows * columns * 2)
        self._check(library().q4b_synth_x(self.handle, seed, stream_id, buffer.ptr, 0, m_rows * columns,
                                          self._err, _ERR))
        return buffer

    # -- compute on device pointers (asynchronous) --------------------------
    def matmul(self, weight: Q4Weight, x_ptr: int, x_dtype: int, m_rows: int, y_ptr: int, y_dtype: int = F16,
               ldy: int | None = None, residual_ptr: int | None = None, residual_dtype: int = NONE,
               ld_residual: int = 0):
        self._check(library().q4b_matmul(self.handle, weight.handle, x_ptr, x_dtype, m_rows, y_ptr, y_dtype,
                                         weight.rows if ldy is None else ldy, residual_ptr, residual_dtype,
                                         ld_residual, self._err, _ERR))

    def matmul_rows(self, weight: Q4Weight, row_ids_ptr: int, count: int, x_ptr: int, x_dtype: int, m_rows: int,
                    y_ptr: int, y_dtype: int = F32, ldy: int | None = None):
        """Listed rows of the matrix only (q4b_matmul_rows): y[m][slot] for row_ids[slot]."""
        self._check(library().q4b_matmul_rows(self.handle, weight.handle, row_ids_ptr, count, x_ptr, x_dtype, m_rows,
                                              y_ptr, y_dtype, count if ldy is None else ldy, self._err, _ERR))

    def matmul_no_alloc(self, weight: Q4Weight, x_ptr: int, x_dtype: int, m_rows: int, y_ptr: int,
                        y_dtype: int = F16, ldy: int | None = None):
        """q4b_matmul with the library's built-in scratch array: allocates nothing."""
        self._check(library().q4b_matmul_no_alloc(self.handle, weight.handle, x_ptr, x_dtype, m_rows, y_ptr,
                                                  y_dtype, weight.rows if ldy is None else ldy, self._err, _ERR))

    def matmul_group(self, weights, x_ptr: int, x_dtype: int, m_rows: int, y_ptrs, y_dtype: int = F16,
                     ldys=None):
        count = len(weights)
        handles = (_vp * count)(*[w.handle for w in weights])
        outputs = (_vp * count)(*y_ptrs)
        strides = (_u32 * count)(*(ldys if ldys is not None else [w.rows for w in weights]))
        self._check(library().q4b_matmul_group(self.handle, handles, count, x_ptr, x_dtype, m_rows, outputs,
                                               y_dtype, strides, self._err, _ERR))

    def push_outputs(self, world: int, peer_ptrs):
        """peer_ptrs[s][r]: where segment s of the NEXT matmul call lives on rank r (None: skip)."""
        count = len(peer_ptrs)
        flat = (_vp * (count * world))(*[peer_ptrs[s][r] for s in range(count) for r in range(world)])
        if library().q4b_context_push_outputs(self.handle, world, flat, count) != 0:
            raise Q4Error(1, "invalid pushed outputs")

    def embedding_lookup(self, embedding: Q4Weight, rows_ptr: int, count: int, out_ptr: int, out_dtype: int = F16):
        self._check(library().q4b_embedding_lookup(self.handle, embedding.handle, rows_ptr, count, out_ptr, out_dtype,
                                                   self._err, _ERR))

    def rmsnorm(self, input_ptr: int, input_dtype: int, weight_ptr: int, output_ptr: int, hidden: int,
                batch_rows: int, epsilon: float = 1e-6):
        """fp16 x of a layer's matmuls from its hidden state (q4b_rmsnorm)."""
        self._check(library().q4b_rmsnorm(self.handle, input_ptr, input_dtype, weight_ptr, output_ptr, hidden,
                                          batch_rows, epsilon, self._err, _ERR))

    def gate_up_silu(self, gate: Q4Weight, up: Q4Weight, x_ptr: int, x_dtype: int, m_rows: int, y_ptr: int,
                     y_dtype: int = F16, ldy: int | None = None):
        self._check(library().q4b_gate_up_silu(self.handle, gate.handle, up.handle, x_ptr, x_dtype, m_rows,
                                               y_ptr, y_dtype, gate.rows if ldy is None else ldy,
                                               self._err, _ERR))

    # -- operator-level calls on host arrays (synchronous) -------------------
    def matmul_host(self, weight: Q4Weight, x: np.ndarray, y_dtype: int = F16):
        """y = x @ W^T on host arrays; returns (y, device milliseconds)."""
        x = np.ascontiguousarray(x)
        m_rows = x.shape[0]
        y = np.empty((m_rows, weight.rows), dtype=_NP_OF[y_dtype])
        ms = ctypes.c_double(0.0)
        self._check(library().q4b_matmul_host(self.handle, weight.handle, x.ctypes.data, _np_dtype_code(x),
                                              m_rows, y.ctypes.data, y_dtype, ctypes.byref(ms),
                                              self._err, _ERR))
        return y, ms.value

    def gate_up_silu_host(self, gate: Q4Weight, up: Q4Weight, x: np.ndarray, y_dtype: int = F16):
        x = np.ascontiguousarray(x)
        m_rows = x.shape[0]
        y = np.empty((m_rows, gate.rows), dtype=_NP_OF[y_dtype])
        ms = ctypes.c_double(0.0)
        self._check(library().q4b_gate_up_silu_host(self.handle, gate.handle, up.handle, x.ctypes.data,
                                                    _np_dtype_code(x), m_rows, y.ctypes.data, y_dtype,
                                                    ctypes.byref(ms), self._err, _ERR))
        return y, ms.value

    # -- memory shared with peer processes -----------------------------------
    def ipc_export(self, device_ptr: int) -> bytes:
        handle = ctypes.create_string_buffer(64)
        self._check(library().q4b_ipc_export(self.handle, device_ptr, handle, self._err, _ERR))
        return handle.raw

    def ipc_open(self, handle: bytes) -> int:
        pointer = _vp()
        buffer = ctypes.create_string_buffer(handle, 64)
        self._check(library().q4b_ipc_open(self.handle, buffer, ctypes.byref(pointer), self._err, _ERR))
        return pointer.value

    def ipc_close(self, pointer: int):
        library().q4b_ipc_close(self.handle, pointer)

    def probe_read(self, mode: int = 0, nbytes: int = 2 << 30, ctas_per_sm: int = 2, stages: int = 4,
                   stage_bytes: int = 18432, iterations: int = 5) -> float:
        """HBM read bandwidth in GB/s (see q4b_probe_read)."""
        out = ctypes.c_double(0.0)
        self._check(library().q4b_probe_read(self.handle, mode, nbytes, ctas_per_sm, stages, stage_bytes,
                                             iterations, ctypes.byref(out), self._err, _ERR))
        return out.value

    def push_rows(self, local: int, peers: list[int], m_rows: int, row_bytes: int, ld_bytes: int):
        """Copy a block of this rank's output into the same place of every peer's (see q4b_push_rows)."""
        array = (_vp * len(peers))(*peers)
        self._check(library().q4b_push_rows(self.handle, local, array, len(peers), m_rows, row_bytes, ld_bytes,
                                            self._err, _ERR))

    def probe_signal(self, own: int, peer: int, payload_bytes: int, rounds: int, rounds_before: int,
                     initiator: bool, mode: int = 0) -> float:
        """Microseconds per round trip of the publish-and-wait exchange between two GPUs (see q4b_probe_signal)."""
        out = ctypes.c_double(0.0)
        self._check(library().q4b_probe_signal(self.handle, own, peer, payload_bytes, rounds, rounds_before,
                                               1 if initiator else 0, mode, ctypes.byref(out), self._err, _ERR))
        return out.value

    # -- graph replay -------------------------------------------------------
    def graph_begin(self):
        self._check(library().q4b_graph_begin(self.handle, self._err, _ERR))

    def graph_end(self) -> Q4Graph:
        handle = _vp()
        self._check(library().q4b_graph_end(self.handle, ctypes.byref(handle), self._err, _ERR))
        return Q4Graph(self, handle.value)


class Q4Barrier:
    """All ranks of a node: 'what I queued so far is stored' (q4b_barrier_*)."""

    def __init__(self, context: Q4Context, world: int, rank: int):
        self.context = context
        handle = _vp()
        context._check(library().q4b_barrier_create(context.handle, world, rank, ctypes.byref(handle),
                                                    context._err, _ERR))
        self.handle = handle

    @property
    def counter(self) -> int:
        return library().q4b_barrier_counter(self.handle)

    def set_peer(self, peer_rank: int, pointer: int):
        if library().q4b_barrier_set_peer(self.handle, peer_rank, pointer) != 0:
            raise Q4Error(1, "invalid peer counter")

    def queue(self):
        self.context._check(library().q4b_barrier_queue(self.context.handle, self.handle, self.context._err, _ERR))

    def free(self):
        if self.handle:
            library().q4b_barrier_free(self.context.handle, self.handle)
            self.handle = None



class Q4Comm:
    """NCCL communicator of the column-parallel ranks (q4b_comm_*).  `exchange(payload_bytes) -> list of every
    rank's payload` is any out-of-band all-gather of small byte strings the launcher has (a process group, a
    file, a socket): rank 0 makes the id, everybody gets it."""

    def __init__(self, context: Q4Context, world: int, rank: int, exchange):
        self.context, self.world, self.rank = context, world, rank
        unique = ctypes.create_string_buffer(128)
        if rank == 0:
            context._check(library().q4b_comm_unique_id(unique, context._err, _ERR))
        unique = ctypes.create_string_buffer(exchange(unique.raw)[0], 128)
        handle = _vp()
        context._check(library().q4b_comm_create(context.handle, world, rank, unique, ctypes.byref(handle),
                                                 context._err, _ERR))
        self.handle = handle

    def all_gather(self, slice_ptr: int, gathered_ptr: int, bytes_per_rank: int):
        self.context._check(library().q4b_all_gather(self.context.handle, self.handle, slice_ptr, gathered_ptr,
                                                     bytes_per_rank, self.context._err, _ERR))

    def all_gather_columns(self, slice_ptr: int, full_ptr: int, m_rows: int, slice_columns: int, element_bytes: int,
                           staging_ptr: int | None):
        self.context._check(library().q4b_all_gather_columns(self.context.handle, self.handle, slice_ptr, full_ptr,
                                                             m_rows, slice_columns, element_bytes, staging_ptr,
                                                             self.context._err, _ERR))

    def free(self):
        if self.handle:
            library().q4b_comm_free(self.context.handle, self.handle)
            self.handle = None
