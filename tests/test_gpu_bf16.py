"""bf16 activations through the C ABI: the arithmetic of the H3 projections
(minimax_h3_attention.metal:512-592; CPU check benchmarks/minimax_h3_m3_real_gemm.c:
25-42): weights rounded to bf16, bf16 x, fp32 sums, bf16 or fp32 out.  The
weights reach the library as H3 keeps them, bf16 scale and bias planes
(q4b_weight_upload_planes).

Gates: (1) the multiplied weights are bit-exact -- an identity matrix as x makes
the kernel hand them back; (2) outputs within max|y - ref| / max|ref| <= 2e-3 of
the oracle (fp32 out), and within that plus half a bf16 ulp of the largest value
(2^-9) for bf16 out."""
import numpy as np
import pytest

from q4_cases import TOLERANCE, assert_close, bits_equal, relative_error

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx(q4b):
    context = q4b.Q4Context(0)
    yield context
    context.close()


def planes_case(orc, seed, projection, rows, groups):
    quants, _ = orc.synth_weight(seed, projection, rows, groups)
    _, scales, biases = orc.bf16_exact_meta(seed, projection, rows, groups)
    return quants, scales, biases


def bf16_x(orc, seed, m, k):
    return orc.round_bf16(orc.synth_x(seed, 0, m, k).astype(np.float32))


@pytest.mark.parametrize("rows,groups", [(128, 1), (256, 4), (200, 3)])
def test_multiplied_weights_are_bit_exact(q4b, orc, ctx, rows, groups):
    k = 64 * groups
    quants, scales, biases = planes_case(orc, 21, 0, rows, groups)
    weight = ctx.upload_planes(quants, scales, biases, q4b.BF16, rows, groups)
    identity = orc.round_bf16(np.eye(k, dtype=np.float32))
    dx = ctx.to_device(identity)
    want = orc.dequant_wbf16(quants, scales, biases, rows, groups)          # [rows, k] bf16 bits
    out32, out16 = ctx.alloc(k * rows * 4), ctx.alloc(k * rows * 2)
    ctx.matmul(weight, dx.ptr, q4b.BF16, k, out32.ptr, q4b.F32)
    ctx.matmul(weight, dx.ptr, q4b.BF16, k, out16.ptr, q4b.BF16)
    assert bits_equal(out32.download(np.float32, (k, rows)), orc.bf16_to_f32(want).T.copy())
    assert bits_equal(out16.download(np.uint16, (k, rows)), want.T.copy())
    weight.free()


@pytest.mark.parametrize("n,k,m", [(512, 1024, 1), (512, 1024, 4), (384, 320, 40), (1000, 1024, 300),
                                   (2048, 5376, 512)])
def test_bf16_matmul_matches_oracle(q4b, orc, ctx, n, k, m):
    groups = k // 64
    quants, scales, biases = planes_case(orc, 22, 0, n, groups)
    weight = ctx.upload_planes(quants, scales, biases, q4b.BF16, n, groups)
    x = bf16_x(orc, 22, m, k)
    ref = orc.matmul_bf16(quants, scales, biases, groups, x)               # fp32 sums, [m, n]
    dx = ctx.to_device(x)
    out32, out16 = ctx.alloc(m * n * 4), ctx.alloc(m * n * 2)
    ctx.matmul(weight, dx.ptr, q4b.BF16, m, out32.ptr, q4b.F32)
    ctx.matmul(weight, dx.ptr, q4b.BF16, m, out16.ptr, q4b.BF16)
    assert_close(out32.download(np.float32, (m, n)), ref, f"bf16 x, fp32 out {n}x{k} M={m}")
    y16 = orc.bf16_to_f32(out16.download(np.uint16, (m, n)))
    assert relative_error(y16, ref) <= TOLERANCE + 2.0 ** -9
    # residuals: bf16 and fp32, added to the un-rounded sums
    residual = orc.synth_x(23, 0, m, n).astype(np.float32)
    for dtype, values in ((q4b.F32, residual), (q4b.BF16, orc.round_bf16(residual))):
        as_f32 = residual if dtype == q4b.F32 else orc.bf16_to_f32(values)
        dr = ctx.to_device(values)
        ctx.matmul(weight, dx.ptr, q4b.BF16, m, out32.ptr, q4b.F32, residual_ptr=dr.ptr, residual_dtype=dtype,
                   ld_residual=n)
        assert_close(out32.download(np.float32, (m, n)), ref.astype(np.float64) + as_f32, "bf16 x with residual")
    weight.free()


def test_bf16_gate_up_silu(q4b, orc, ctx):
    n, k, m = 640, 1024, 48
    groups = k // 64
    gate_planes, up_planes = planes_case(orc, 24, 0, n, groups), planes_case(orc, 24, 1, n, groups)
    gate = ctx.upload_planes(*gate_planes, q4b.BF16, n, groups)
    up = ctx.upload_planes(*up_planes, q4b.BF16, n, groups)
    x = bf16_x(orc, 24, m, k)
    g = orc.matmul_bf16(*gate_planes, groups, x).astype(np.float64)
    u = orc.matmul_bf16(*up_planes, groups, x).astype(np.float64)
    ref = g / (1.0 + np.exp(-g)) * u
    dx, out = ctx.to_device(x), ctx.alloc(m * n * 4)
    ctx.gate_up_silu(gate, up, dx.ptr, q4b.BF16, m, out.ptr, q4b.F32)
    assert_close(out.download(np.float32, (m, n)), ref, "bf16 fused gate/up")
    gate.free()
    up.free()


def test_dtype_pairs_are_checked(q4b, orc, ctx):
    quants, scales, biases = planes_case(orc, 25, 0, 128, 2)
    weight = ctx.upload_planes(quants, scales, biases, q4b.BF16, 128, 2)
    buffer = ctx.alloc(128 * 128 * 4)
    for x_dtype, y_dtype in ((q4b.F16, q4b.BF16), (q4b.F32, q4b.BF16), (q4b.BF16, q4b.F16)):
        with pytest.raises(q4b.Q4Error) as refused:
            ctx.matmul(weight, buffer.ptr, x_dtype, 4, buffer.ptr, y_dtype)
        assert refused.value.status == 1
    weight.free()
