"""The affine-Q8 sibling (minimax_h3_q8_gemm_bf16_meta, minimax_h3_attention.metal:594-676): code bytes, bf16
scale and bias per group, w = half(float(scale) * q + float(bias)), fp16 activations, fp32 sums.

Gates as for Q4: codes and dequantised weights bit-exact over whole matrices (the upload keeps the bf16 metadata
as they are), outputs within 2e-3 of the oracle's double sum.  The reference holds no CPU check for this kernel
(its benchmark multiplies zero-filled buffers), so the oracle is the kernel's own formula restated."""
import numpy as np
import pytest

from q4_cases import assert_close, bits_equal

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx(q4b):
    context = q4b.Q4Context(0)
    yield context
    context.close()


@pytest.mark.parametrize("rows,groups", [(128, 1), (200, 3), (1000, 16)])
def test_q8_unpack_is_bit_exact(q4b, orc, ctx, rows, groups):
    quants, scales, biases = orc.synth_q8(61, rows, groups)
    # metadata far outside fp16's range stay what they are: nothing is narrowed on the way in
    scales[0, 0] = orc.round_bf16(np.array([3.0e-7], dtype=np.float32))[0]
    biases[0, 0] = orc.round_bf16(np.array([-2.0e-5], dtype=np.float32))[0]
    weight = ctx.upload_q8(quants, scales, biases, rows, groups)
    codes, w32, w16 = weight.unpack()
    want32, want16 = orc.dequant_q8(quants, scales, biases, rows, groups)
    assert (codes == quants).all()
    assert bits_equal(w32, want32)
    assert bits_equal(w16, want16)
    begin, count = 128, rows - 128
    if count > 0:
        shard = ctx.upload_q8(quants, scales, biases, rows, groups, begin, count)
        _, part32, _ = shard.unpack(codes=False, w16=False)
        assert bits_equal(part32, want32[begin:])
        shard.free()
    weight.free()


@pytest.mark.parametrize("n,k,m", [(256, 128, 1), (512, 1024, 4), (384, 320, 40), (1000, 1024, 300), (2048, 5376, 512)])
def test_q8_matmul_matches_oracle(q4b, orc, ctx, n, k, m):
    groups = k // 64
    quants, scales, biases = orc.synth_q8(62, n, groups)
    weight = ctx.upload_q8(quants, scales, biases, n, groups)
    x = orc.synth_x(62, 0, m, k)
    ref = orc.matmul_q8(quants, scales, biases, groups, x)
    dx = ctx.to_device(x)
    out32, out16 = ctx.alloc(m * n * 4), ctx.alloc(m * n * 2)
    ctx.matmul(weight, dx.ptr, q4b.F16, m, out32.ptr, q4b.F32)
    ctx.matmul(weight, dx.ptr, q4b.F16, m, out16.ptr, q4b.F16)
    assert_close(out32.download(np.float32, (m, n)), ref, f"Q8 {n}x{k} M={m}, fp32 out")
    assert_close(out16.download(np.float16, (m, n)), ref, f"Q8 {n}x{k} M={m}, fp16 out")
    # the multiplied weights themselves: an identity as x hands them back
    if k <= 320:
        identity = np.eye(k, dtype=np.float16)
        di, dw = ctx.to_device(identity), ctx.alloc(k * n * 2)
        ctx.matmul(weight, di.ptr, q4b.F16, k, dw.ptr, q4b.F16)
        _, want16 = orc.dequant_q8(quants, scales, biases, n, groups)
        assert bits_equal(dw.download(np.float16, (k, n)), want16.T.copy())
    weight.free()


def test_q8_is_refused_where_it_has_no_kernel(q4b, orc, ctx):
    quants, scales, biases = orc.synth_q8(63, 128, 2)
    weight = ctx.upload_q8(quants, scales, biases, 128, 2)
    buffer = ctx.alloc(128 * 128 * 4)
    with pytest.raises(q4b.Q4Error) as refused:
        ctx.gate_up_silu(weight, weight, buffer.ptr, q4b.F16, 1, buffer.ptr)
    assert refused.value.status == 1
    with pytest.raises(q4b.Q4Error):
        ctx.matmul_no_alloc(weight, buffer.ptr, q4b.F16, 1, buffer.ptr)
    with pytest.raises(q4b.Q4Error):
        ctx.matmul(weight, buffer.ptr, q4b.BF16, 4, buffer.ptr, q4b.BF16)
    with pytest.raises(q4b.Q4Error):
        weight.rows_view(0, 128)
    ctx.sync()
    weight.free()
