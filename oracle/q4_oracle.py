"""ctypes/NumPy front end of the CPU oracle -- TEST INFRASTRUCTURE ONLY.

Loads ``oracle/libq4oracle.so`` (the C restatement of the reference's scalar
affine-Q4 formulas, built from ``oracle/q4_oracle.c``) and, when it exists,
``oracle/_ref/libq4ref.so`` (the reference's own packer code compiled from its
sources).  Only tests, the smoke check and the CPU-baseline leg of the benchmark
import this module; the CUDA library never does.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
F16, F32, BF16, NONE = 0, 1, 2, -1

_c_size = ctypes.c_size_t
_u8p = ctypes.POINTER(ctypes.c_uint8)
_u16p = ctypes.POINTER(ctypes.c_uint16)
_u32p = ctypes.POINTER(ctypes.c_uint32)
_f32p = ctypes.POINTER(ctypes.c_float)
_f64p = ctypes.POINTER(ctypes.c_double)


def build(force: bool = False) -> str:
    """Compile the C oracle in place (gcc only) and return the .so path."""
    target = os.path.join(_HERE, "libq4oracle.so")
    source = os.path.join(_HERE, "q4_oracle.c")
    stale = (not os.path.exists(target)
             or os.path.getmtime(target) < os.path.getmtime(source))
    if force or stale:
        subprocess.check_call(
            ["gcc", "-O3", "-std=c11", "-fopenmp", "-fPIC", "-shared", source,
             "-o", target, "-lm"], cwd=_HERE)
    return target


def reference_root() -> str | None:
    """A checkout of the reference project: REFERENCE in the environment, else a directory named `reference`
    beside this repository."""
    named = os.environ.get("REFERENCE", "")
    if named:
        return named if os.path.isdir(named) else None
    beside = os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")
    return beside if os.path.isdir(beside) else None


def build_ref() -> str | None:
    """Compile oracle/_ref from the reference tree when there is one; a prebuilt oracle/_ref is kept otherwise."""
    root = reference_root()
    if root is not None:
        subprocess.call(["make", "-s", "ref", f"REFERENCE={root}"], cwd=_HERE,
                        stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL)
    path = os.path.join(_HERE, "_ref", "libq4ref.so")
    return path if os.path.exists(path) else None


def _ptr(array, kind):
    return None if array is None else array.ctypes.data_as(kind)


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        handle = ctypes.CDLL(build())
        handle.q4o_hash.restype = ctypes.c_uint64
        handle.q4o_hash.argtypes = [ctypes.c_uint64] * 3
        handle.q4o_f32_to_f16.restype = ctypes.c_uint16
        handle.q4o_f32_to_f16.argtypes = [ctypes.c_float]
        handle.q4o_f64_to_f16.restype = ctypes.c_uint16
        handle.q4o_f64_to_f16.argtypes = [ctypes.c_double]
        handle.q4o_f16_to_f32.restype = ctypes.c_float
        handle.q4o_f16_to_f32.argtypes = [ctypes.c_uint16]
        handle.q4o_bf16_to_f16.restype = ctypes.c_uint16
        handle.q4o_bf16_to_f16.argtypes = [ctypes.c_uint16]
        handle.q4o_f32_to_bf16.restype = ctypes.c_uint16
        handle.q4o_f32_to_bf16.argtypes = [ctypes.c_float]
        handle.q4o_max_threads.restype = ctypes.c_int
        handle.q4o_synth_codes.argtypes = [ctypes.c_uint64, ctypes.c_uint64,
                                           _u32p, _c_size, _c_size]
        handle.q4o_synth_meta.argtypes = [ctypes.c_uint64, ctypes.c_uint64,
                                          _u16p, _c_size, _c_size]
        handle.q4o_synth_x.argtypes = [ctypes.c_uint64, ctypes.c_uint64, _u16p,
                                       _c_size, _c_size]
        handle.q4o_fill_weights_xorshift.argtypes = [_u8p, _u16p, _c_size,
                                                     ctypes.c_uint32]
        handle.q4o_activation_sincos.argtypes = [_u16p, _c_size]
        handle.q4o_h3_pattern.argtypes = [_u8p, _u16p, _c_size, _c_size, _u16p,
                                          _c_size, ctypes.c_uint32]
        handle.q4o_unpack_codes.argtypes = [_u8p, _c_size, _c_size, _u8p]
        handle.q4o_dequant_w32.argtypes = [_u8p, _u16p, _c_size, _c_size, _f32p]
        handle.q4o_dequant_w16.argtypes = [_u8p, _u16p, _c_size, _c_size, _u16p]
        handle.q4o_matmul.argtypes = [
            _u8p, _u16p, _c_size, _c_size, _c_size, ctypes.c_void_p,
            ctypes.c_int, _c_size, ctypes.c_void_p, ctypes.c_int, _c_size,
            _f32p, _f64p, _c_size, ctypes.c_int]
        handle.q4o_gate_up_silu.argtypes = [
            _u8p, _u16p, _u8p, _u16p, _c_size, _c_size, _c_size,
            ctypes.c_void_p, ctypes.c_int, _c_size, _f32p, _f64p, _c_size,
            ctypes.c_int]
        handle.q4o_matmul_bf16.argtypes = [
            _u8p, _u16p, _u16p, _c_size, _c_size, _c_size, _u16p, _c_size,
            _f32p, _c_size, ctypes.c_int]
        handle.q4o_round_f16.argtypes = [_f32p, _u16p, _c_size]
        handle.q4o_dequant_q8.argtypes = [_u8p, _u16p, _u16p, _c_size, _c_size, _f32p, _u16p]
        handle.q4o_matmul_q8.argtypes = [_u8p, _u16p, _u16p, _c_size, _c_size, _c_size, ctypes.c_void_p, ctypes.c_int,
                                         _c_size, _f32p, _f64p, _c_size, ctypes.c_int]
        handle.q4o_rms_norm.argtypes = [ctypes.c_void_p, ctypes.c_int, _f32p, _u16p, _c_size, _c_size,
                                        ctypes.c_float]
        _lib = handle
    return _lib


# stream ids of the seeded generator: one weight matrix = (codes, meta) pair
STREAM_X = 0


def stream_of(projection: int, part: int) -> int:
    """part 0 = codes, 1 = metadata; projection >= 0.  Stream 0 holds x."""
    return 1 + 2 * projection + part


def synth_weight(seed: int, projection: int, rows: int, groups: int):
    """Seeded Q4 matrix in the reference image layout.

    Returns (quants uint8 [rows, groups*32], meta uint16 [rows, groups, 2])."""
    words = np.empty(rows * groups * 8, dtype=np.uint32)
    lib().q4o_synth_codes(seed, stream_of(projection, 0), _ptr(words, _u32p), 0,
                          words.size)
    meta = np.empty(rows * groups * 2, dtype=np.uint16)
    lib().q4o_synth_meta(seed, stream_of(projection, 1), _ptr(meta, _u16p), 0,
                         rows * groups)
    return (words.view(np.uint8).reshape(rows, groups * 32),
            meta.reshape(rows, groups, 2))


def synth_weight_rows(seed: int, projection: int, groups: int, rows):
    """The given rows of the seeded matrix `synth_weight` would produce, without
    generating the rest (the generator is counter-based).  Returns (quants uint8
    [len(rows), groups*32], meta uint16 [len(rows), groups, 2])."""
    rows = [int(r) for r in rows]
    quants = np.empty((len(rows), groups * 8), dtype=np.uint32)
    meta = np.empty((len(rows), groups * 2), dtype=np.uint16)
    for i, row in enumerate(rows):
        lib().q4o_synth_codes(seed, stream_of(projection, 0), _ptr(quants[i], _u32p), row * groups * 8, groups * 8)
        lib().q4o_synth_meta(seed, stream_of(projection, 1), _ptr(meta[i], _u16p), row * groups, groups)
    return quants.view(np.uint8).reshape(len(rows), groups * 32), meta.reshape(len(rows), groups, 2)


def bf16_exact_meta(seed: int, projection: int, rows: int, groups: int):
    """Seeded metadata whose values are exact in BOTH bf16 and fp16.

    The reference packer reads BF16 planes and writes fp16 records; keeping 8
    significant bits makes that conversion lossless, so its BF16-source results
    and an fp16-image computation must agree bit for bit.  Returns (fp16 records
    [rows, groups, 2], bf16 scale plane, bf16 bias plane)."""
    _, meta = synth_weight(seed, projection, rows, groups)
    half = meta.copy()
    half &= np.uint16(0xFFF8)  # drop 3 of 10 mantissa bits
    scales = half[..., 0].view(np.float16).astype(np.float32)
    biases = half[..., 1].view(np.float16).astype(np.float32)
    assert np.all((scales.view(np.uint32) & 0xFFFF) == 0)
    assert np.all((biases.view(np.uint32) & 0xFFFF) == 0)
    to_bf16 = lambda a: (a.view(np.uint32) >> 16).astype(np.uint16)
    return half, to_bf16(scales), to_bf16(biases)


def synth_x(seed: int, stream: int, m_rows: int, columns: int) -> np.ndarray:
    """Seeded activations, fp16 bits viewed as float16 [m_rows, columns]."""
    bits = np.empty(m_rows * columns, dtype=np.uint16)
    lib().q4o_synth_x(seed, stream, _ptr(bits, _u16p), 0, bits.size)
    return bits.view(np.float16).reshape(m_rows, columns)


def fill_weights_xorshift(group_count: int, seed: int):
    quants = np.empty(group_count * 32, dtype=np.uint8)
    meta = np.empty(group_count * 2, dtype=np.uint16)
    lib().q4o_fill_weights_xorshift(_ptr(quants, _u8p), _ptr(meta, _u16p),
                                    group_count, seed)
    return quants, meta


def activation_sincos(count: int) -> np.ndarray:
    bits = np.empty(count, dtype=np.uint16)
    lib().q4o_activation_sincos(_ptr(bits, _u16p), count)
    return bits.view(np.float16)


def h3_pattern(rows: int, groups: int, x_count: int, input_seed: int):
    quants = np.empty(rows * groups * 32, dtype=np.uint8)
    meta = np.empty(rows * groups * 2, dtype=np.uint16)
    x = np.empty(x_count, dtype=np.uint16)
    lib().q4o_h3_pattern(_ptr(quants, _u8p), _ptr(meta, _u16p), rows, groups,
                         _ptr(x, _u16p), x_count, input_seed)
    return (quants.reshape(rows, groups * 32), meta.reshape(rows, groups, 2),
            x.view(np.float16))


def _flat(array, dtype):
    return np.ascontiguousarray(array).view(dtype).reshape(-1)


def unpack_codes(quants, rows, groups):
    q = _flat(quants, np.uint8)
    out = np.empty(rows * groups * 64, dtype=np.uint8)
    lib().q4o_unpack_codes(_ptr(q, _u8p), rows, groups, _ptr(out, _u8p))
    return out.reshape(rows, groups * 64)


def dequant_w32(quants, meta, rows, groups):
    q, m = _flat(quants, np.uint8), _flat(meta, np.uint16)
    out = np.empty(rows * groups * 64, dtype=np.float32)
    lib().q4o_dequant_w32(_ptr(q, _u8p), _ptr(m, _u16p), rows, groups,
                          _ptr(out, _f32p))
    return out.reshape(rows, groups * 64)


def dequant_w16(quants, meta, rows, groups):
    q, m = _flat(quants, np.uint8), _flat(meta, np.uint16)
    out = np.empty(rows * groups * 64, dtype=np.uint16)
    lib().q4o_dequant_w16(_ptr(q, _u8p), _ptr(m, _u16p), rows, groups,
                          _ptr(out, _u16p))
    return out.view(np.float16).reshape(rows, groups * 64)


def _dtype_code(array):
    if array.dtype == np.float16:
        return F16
    if array.dtype == np.float32:
        return F32
    raise TypeError(f"unsupported activation dtype {array.dtype}")


def matmul(quants, meta, groups, x, row_begin=0, row_count=None, residual=None,
           want32=True, want64=True, threads=0):
    """y[m, n] for rows row_begin..; returns (y32, y64), each [M, row_count]."""
    q, m = _flat(quants, np.uint8), _flat(meta, np.uint16)
    rows_total = q.size // (groups * 32)
    if row_count is None:
        row_count = rows_total - row_begin
    x = np.ascontiguousarray(x)
    m_rows = x.shape[0]
    assert x.shape[1] == groups * 64
    y32 = np.empty((m_rows, row_count), dtype=np.float32) if want32 else None
    y64 = np.empty((m_rows, row_count), dtype=np.float64) if want64 else None
    res_ptr, res_code, ld_res = None, NONE, 0
    if residual is not None:
        residual = np.ascontiguousarray(residual)
        res_ptr, res_code = residual.ctypes.data, _dtype_code(residual)
        ld_res = residual.shape[1]
    lib().q4o_matmul(_ptr(q, _u8p), _ptr(m, _u16p), groups, row_begin, row_count,
                     x.ctypes.data, _dtype_code(x), m_rows, res_ptr, res_code,
                     ld_res, _ptr(y32, _f32p), _ptr(y64, _f64p), row_count,
                     threads)
    return y32, y64


def gate_up_silu(gate_quants, gate_meta, up_quants, up_meta, groups, x,
                 row_begin=0, row_count=None, want32=True, want64=True,
                 threads=0):
    gq, gm = _flat(gate_quants, np.uint8), _flat(gate_meta, np.uint16)
    uq, um = _flat(up_quants, np.uint8), _flat(up_meta, np.uint16)
    rows_total = gq.size // (groups * 32)
    if row_count is None:
        row_count = rows_total - row_begin
    x = np.ascontiguousarray(x)
    m_rows = x.shape[0]
    y32 = np.empty((m_rows, row_count), dtype=np.float32) if want32 else None
    y64 = np.empty((m_rows, row_count), dtype=np.float64) if want64 else None
    lib().q4o_gate_up_silu(_ptr(gq, _u8p), _ptr(gm, _u16p), _ptr(uq, _u8p),
                           _ptr(um, _u16p), groups, row_begin, row_count,
                           x.ctypes.data, _dtype_code(x), m_rows,
                           _ptr(y32, _f32p), _ptr(y64, _f64p), row_count,
                           threads)
    return y32, y64


def matmul_bf16(quants, scales_bf16, biases_bf16, groups, x_bf16, row_begin=0,
                row_count=None, threads=0):
    q = _flat(quants, np.uint8)
    s, b = _flat(scales_bf16, np.uint16), _flat(biases_bf16, np.uint16)
    rows_total = q.size // (groups * 32)
    if row_count is None:
        row_count = rows_total - row_begin
    xb = np.ascontiguousarray(x_bf16).view(np.uint16)
    m_rows = xb.shape[0]
    y = np.empty((m_rows, row_count), dtype=np.float32)
    lib().q4o_matmul_bf16(_ptr(q, _u8p), _ptr(s, _u16p), _ptr(b, _u16p), groups,
                          row_begin, row_count, _ptr(xb.reshape(-1), _u16p),
                          m_rows, _ptr(y, _f32p), row_count, threads)
    return y


def rmsnorm(values: np.ndarray, weight: np.ndarray, epsilon: float = 1e-6) -> np.ndarray:
    """qwen38_rmsnorm_f16_to_f16 / _f32_to_f16 (qwen38_layer.metal:21-69), per row of
    `values` [batch, hidden] (float16 or float32): 256 strided partial sums of squares
    in index order, the halving tree over them, inv_rms = 1 / sqrt(sum / hidden +
    epsilon), out = half(x * inv_rms * weight).  Every operation is a separately
    rounded float32 operation; returns float16 [batch, hidden]."""
    x = np.ascontiguousarray(values).astype(np.float32)
    batch, hidden = x.shape
    chunks = -(-hidden // 256)
    squares = np.zeros((batch, chunks * 256), dtype=np.float32)
    squares[:, :hidden] = x * x
    squares = squares.reshape(batch, chunks, 256)
    partials = np.zeros((batch, 256), dtype=np.float32)
    for chunk in range(chunks):                      # thread t adds elements t, t + 256, ... in this order
        partials = partials + squares[:, chunk, :]
    stride = 128
    while stride:
        partials[:, :stride] = partials[:, :stride] + partials[:, stride:2 * stride]
        stride >>= 1
    mean = partials[:, 0] / np.float32(hidden) + np.float32(epsilon)
    inv_rms = np.float32(1.0) / np.sqrt(mean, dtype=np.float32)
    w = np.ascontiguousarray(weight, dtype=np.float32)
    return ((x * inv_rms[:, None]) * w[None, :]).astype(np.float16)


def rmsnorm_reference(values: np.ndarray, weight: np.ndarray, epsilon: float = 1e-6) -> np.ndarray:
    """The reference's own CPU check of the RMS norm, cpu_rms_half / cpu_rms_float
    (qwen38_m3_layer.m:395-420), restated in C (q4o_rms_norm): double sum of squares, float
    inverse, half(x * inv * weight).  The Metal kernel sums in float in another order, so the two agree
    to an fp16 ulp, not bit for bit; `rmsnorm` above follows the kernel's order."""
    x = np.ascontiguousarray(values)
    assert x.dtype in (np.float16, np.float32)
    batch, hidden = x.shape
    w = np.ascontiguousarray(weight, dtype=np.float32)
    out = np.empty((batch, hidden), dtype=np.uint16)
    lib().q4o_rms_norm(x.ctypes.data, 0 if x.dtype == np.float16 else 1, _ptr(w, _f32p), _ptr(out.reshape(-1), _u16p),
                       hidden, batch, epsilon)
    return out.view(np.float16)


def round_bf16(values: np.ndarray) -> np.ndarray:
    """float32 -> bf16 bits, round to nearest even: bfloat_bits of the H3 CPU check
    (benchmarks/minimax_h3_m3_real_gemm.c:18-23).  Finite inputs only."""
    bits = np.ascontiguousarray(values, dtype=np.float32).view(np.uint32).astype(np.uint64)
    rounding = np.uint64(0x7FFF) + ((bits >> np.uint64(16)) & np.uint64(1))
    return ((bits + rounding) >> np.uint64(16)).astype(np.uint16)


def bf16_to_f32(bits: np.ndarray) -> np.ndarray:
    """bf16 bits -> float32 (bfloat_value, benchmarks/minimax_h3_m3_real_gemm.c:11-16)."""
    return (np.ascontiguousarray(bits, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def dequant_wbf16(quants, scales_bf16, biases_bf16, rows, groups) -> np.ndarray:
    """The weights the H3 bf16 GEMM multiplies, as bf16 bits [rows, 64 * groups]:
    bf16(scale * float(q) + bias) with scale and bias widened from bf16, the
    product and the sum in fp32 (benchmarks/minimax_h3_m3_real_gemm.c:31-38;
    minimax_h3_attention.metal:542-551).  scale * q is exact in fp32."""
    codes = unpack_codes(quants, rows, groups).astype(np.float32).reshape(rows, groups, 64)
    scale = bf16_to_f32(np.asarray(scales_bf16).reshape(rows, groups, 1))
    bias = bf16_to_f32(np.asarray(biases_bf16).reshape(rows, groups, 1))
    product = scale * codes                   # float32, exact
    return round_bf16(product + bias).reshape(rows, groups * 64)


def synth_q8(seed: int, rows: int, groups: int):
    """Seeded affine-Q8 planes in the layout of minimax_h3_q8_gemm_bf16_meta: codes uint8 [rows, groups * 64]
    uniform in 0..255, bf16 scales uniform in [3e-5, 2.5e-4] and biases -128 * scale + N(0, 1e-3), so that the
    weights cover the same range as the Q4 distributions."""
    rng = np.random.default_rng(seed)
    quants = rng.integers(0, 256, size=(rows, groups * 64), dtype=np.uint8)
    scale = rng.uniform(3e-5, 2.5e-4, size=(rows, groups)).astype(np.float32)
    scales = round_bf16(scale)
    biases = round_bf16(-128.0 * bf16_to_f32(scales) + rng.standard_normal((rows, groups)).astype(np.float32) * 1e-3)
    return quants, scales, biases


def dequant_q8(quants, scales_bf16, biases_bf16, rows, groups):
    """(w32, w16) of the Q8 contract half(float(scale) * q + float(bias)); w16 as float16."""
    q = _flat(quants, np.uint8)
    s, b = _flat(scales_bf16, np.uint16), _flat(biases_bf16, np.uint16)
    w32 = np.empty(rows * groups * 64, dtype=np.float32)
    w16 = np.empty(rows * groups * 64, dtype=np.uint16)
    lib().q4o_dequant_q8(_ptr(q, _u8p), _ptr(s, _u16p), _ptr(b, _u16p), rows, groups, _ptr(w32, _f32p),
                         _ptr(w16, _u16p))
    return w32.reshape(rows, groups * 64), w16.view(np.float16).reshape(rows, groups * 64)


def matmul_q8(quants, scales_bf16, biases_bf16, groups, x, row_begin=0, row_count=None, threads=0):
    """[M, row_count] double sums of half(w) * x for the affine-Q8 matrix."""
    q = _flat(quants, np.uint8)
    s, b = _flat(scales_bf16, np.uint16), _flat(biases_bf16, np.uint16)
    rows_total = q.size // (groups * 64)
    if row_count is None:
        row_count = rows_total - row_begin
    x = np.ascontiguousarray(x)
    m_rows = x.shape[0]
    y64 = np.empty((m_rows, row_count), dtype=np.float64)
    lib().q4o_matmul_q8(_ptr(q, _u8p), _ptr(s, _u16p), _ptr(b, _u16p), groups, row_begin, row_count,
                        x.ctypes.data, _dtype_code(x), m_rows, None, _ptr(y64, _f64p), row_count, threads)
    return y64


def round_f16(values: np.ndarray) -> np.ndarray:
    flat = np.ascontiguousarray(values, dtype=np.float32).reshape(-1)
    out = np.empty(flat.size, dtype=np.uint16)
    lib().q4o_round_f16(_ptr(flat, _f32p), _ptr(out, _u16p), flat.size)
    return out.view(np.float16).reshape(values.shape)


def max_threads() -> int:
    return int(lib().q4o_max_threads())


# ---------------------------------------------------------------------------
# the reference's own packer code (oracle/_ref), when built
# ---------------------------------------------------------------------------
_ref = None


def ref() -> ctypes.CDLL | None:
    """The shared object made from the reference's packer sources, or None."""
    global _ref
    if _ref is None:
        path = os.path.join(_HERE, "_ref", "libq4ref.so")
        if not os.path.exists(path):
            return None
        handle = ctypes.CDLL(path)
        handle.ref_float_to_half_bits.restype = ctypes.c_uint16
        handle.ref_float_to_half_bits.argtypes = [ctypes.c_float]
        handle.ref_half_bits_to_float.restype = ctypes.c_float
        handle.ref_half_bits_to_float.argtypes = [ctypes.c_uint16]
        handle.ref_bf16_to_half.restype = ctypes.c_uint16
        handle.ref_bf16_to_half.argtypes = [ctypes.c_uint16]
        handle.ref_convert_metadata.argtypes = [_u16p, _u16p, _c_size, _u16p]
        handle.ref_gate_up_first8.argtypes = [_u8p, _u16p, _u16p, _u8p, _u16p,
                                              _u16p, _f32p]
        handle.ref_mlp_first8.argtypes = [_u8p, _u16p, _u16p, _u8p, _u16p, _u16p,
                                          _u8p, _u16p, _u16p, _f32p]
        _ref = handle
    return _ref
