"""Parity of the CUDA path (through the C ABI) with the CPU oracle.

Bit-exact gates: device-unpacked codes, W32 = scale*(float)q+bias and W16 =
fp16_rn(scale*q+bias) over whole matrices.  Tolerance gate for outputs:
max|y - ref| / max|ref| <= 2e-3 against the oracle's double-precision sum.
"""
import numpy as np
import pytest

from q4_cases import assert_close, bits_equal, relative_error

pytestmark = pytest.mark.gpu

SMALL = [("q", 1024, 2048), ("k", 1024, 512), ("v", 1024, 512), ("o", 2048, 1024), ("down", 3072, 1024)]
BIG = [("q", 5120, 6144), ("k", 5120, 1024), ("o", 6144, 5120), ("down", 17408, 5120)]


@pytest.fixture(scope="module")
def ctx(q4b):
    context = q4b.Q4Context(0)
    yield context
    context.close()


def run_matmul(q4b, ctx, weight, x, y_dtype=None, residual=None):
    y_dtype = q4b.F16 if y_dtype is None else y_dtype
    np_out = np.float16 if y_dtype == q4b.F16 else np.float32
    m = x.shape[0]
    dx = ctx.to_device(x)
    dy = ctx.alloc(m * weight.rows * np.dtype(np_out).itemsize)
    x_code = q4b.F16 if x.dtype == np.float16 else q4b.F32
    if residual is not None:
        dr = ctx.to_device(residual)
        r_code = q4b.F16 if residual.dtype == np.float16 else q4b.F32
        ctx.matmul(weight, dx.ptr, x_code, m, dy.ptr, y_dtype, None, dr.ptr, r_code, residual.shape[1])
    else:
        ctx.matmul(weight, dx.ptr, x_code, m, dy.ptr, y_dtype)
    return dy.download(np_out, (m, weight.rows))


# ---------------------------------------------------------------- loader / dequant
@pytest.mark.parametrize("rows,groups", [(3072, 16), (48, 3), (100, 5), (17, 1), (1024, 80)])
def test_unpack_is_bit_exact(q4b, orc, ctx, rows, groups):
    quants, meta = orc.synth_weight(0, 0, rows, groups)
    weight = ctx.upload(quants, meta, rows, groups)
    codes, w32, w16 = weight.unpack()
    assert (codes == orc.unpack_codes(quants, rows, groups)).all()
    assert bits_equal(w32, orc.dequant_w32(quants, meta, rows, groups))
    assert bits_equal(w16, orc.dequant_w16(quants, meta, rows, groups))


def test_unpack_bit_exact_on_adversarial_metadata(q4b, orc, ctx):
    # scales/biases across the whole fp16 range incl. subnormal results and ties
    rows, groups = 64, 8
    rng = np.random.default_rng(3)
    quants = rng.integers(0, 256, size=(rows, groups * 32), dtype=np.uint8)
    scale = (rng.standard_normal((rows, groups)) * 10.0 ** rng.integers(-6, 1, (rows, groups))).astype(np.float16)
    bias = (-8 * scale.astype(np.float32) + rng.standard_normal((rows, groups)) * 1e-4).astype(np.float16)
    bias[::7] = np.float16(6e-6)  # subnormal biases
    meta = np.stack([scale.view(np.uint16), bias.view(np.uint16)], axis=-1)
    weight = ctx.upload(quants, meta, rows, groups)
    codes, w32, w16 = weight.unpack()
    assert (codes == orc.unpack_codes(quants, rows, groups)).all()
    assert bits_equal(w16, orc.dequant_w16(quants, meta, rows, groups))


def test_row_slices_are_the_matching_rows(q4b, orc, ctx):
    rows, groups = 256, 4
    quants, meta = orc.synth_weight(5, 0, rows, groups)
    full = orc.dequant_w32(quants, meta, rows, groups)
    for begin, count in [(0, 64), (64, 64), (100, 37), (255, 1)]:
        shard = ctx.upload(quants, meta, rows, groups, begin, count)
        _, w32, _ = shard.unpack(codes=False, w16=False)
        assert shard.rows == count and bits_equal(w32, full[begin:begin + count])


def test_device_generator_matches_cpu_generator(q4b, orc, ctx):
    rows, groups = 512, 16
    for seed, projection, begin, count in [(0, 0, 0, 512), (9, 3, 128, 200)]:
        quants, meta = orc.synth_weight(seed, projection, rows, groups)
        weight = ctx.synth_weight(seed, projection, rows, groups, begin, count)
        codes, w32, _ = weight.unpack(w16=False)
        assert (codes == orc.unpack_codes(quants, rows, groups)[begin:begin + count]).all()
        assert bits_equal(w32, orc.dequant_w32(quants, meta, rows, groups)[begin:begin + count])
    x = orc.synth_x(4, 0, 3, 1024)
    dx = ctx.synth_x(4, 0, 3, 1024)
    assert bits_equal(dx.download(np.float16, (3, 1024)), x)


def test_bf16_planes_convert_like_the_packer(q4b, orc, ctx):
    rows, groups = 64, 4
    quants, _ = orc.synth_weight(2, 0, rows, groups)
    rng = np.random.default_rng(8)
    scales = rng.integers(0x3800, 0x3C00, size=(rows, groups), dtype=np.uint16)
    biases = (rng.integers(0x3800, 0x3E00, size=(rows, groups), dtype=np.uint16) | 0x8000).astype(np.uint16)
    lib = orc.lib()
    meta = np.empty((rows, groups, 2), dtype=np.uint16)
    for r in range(rows):
        for g in range(groups):
            meta[r, g, 0] = lib.q4o_bf16_to_f16(int(scales[r, g]))
            meta[r, g, 1] = lib.q4o_bf16_to_f16(int(biases[r, g]))
    weight = ctx.upload_planes(quants, scales, biases, q4b.BF16, rows, groups)
    _, w32, _ = weight.unpack(codes=False, w16=False)
    assert bits_equal(w32, orc.dequant_w32(quants, meta, rows, groups))


# ---------------------------------------------------------------- GEMV / small M
def test_config0_single_gemv(q4b, orc, ctx):
    rows, groups = 3072, 16
    quants, meta = orc.synth_weight(0, 0, rows, groups)
    x = orc.synth_x(0, 0, 1, 1024)
    weight = ctx.upload(quants, meta, rows, groups)
    y = run_matmul(q4b, ctx, weight, x)
    _, ref = orc.matmul(quants, meta, groups, x, want32=False)
    assert_close(y, ref, "config[0]")
    # fp32 output: what remains is the 15-bit digits of the integer form (M <= 4) ...
    y32 = run_matmul(q4b, ctx, weight, x, q4b.F32)
    assert relative_error(y32, ref) < 1.5e-4
    # ... and accumulation order alone in the fp16 form
    try:
        ctx.set_variant(0x10)
        y32 = run_matmul(q4b, ctx, weight, x, q4b.F32)
    finally:
        ctx.set_variant(0)
    assert relative_error(y32, ref) < 2e-5


@pytest.mark.parametrize("m", [1, 4])
@pytest.mark.parametrize("name,k,n", SMALL)
def test_small_layer_projections(q4b, orc, ctx, name, k, n, m):
    quants, meta = orc.synth_weight(0, 1, n, k // 64)
    x = orc.synth_x(0, 0, m, k)
    weight = ctx.upload(quants, meta, n, k // 64)
    y = run_matmul(q4b, ctx, weight, x)
    _, ref = orc.matmul(quants, meta, k // 64, x, want32=False)
    assert_close(y, ref, f"{name} M={m}")


@pytest.mark.parametrize("m", [1, 4])
@pytest.mark.parametrize("k,n", [(1024, 3072), (5120, 17408)])
def test_fused_gate_up_silu(q4b, orc, ctx, k, n, m):
    gq, gm = orc.synth_weight(0, 4, n, k // 64)
    uq, um = orc.synth_weight(0, 5, n, k // 64)
    x = orc.synth_x(0, 0, m, k)
    gate, up = ctx.upload(gq, gm, n, k // 64), ctx.upload(uq, um, n, k // 64)
    dx, dy = ctx.to_device(x), ctx.alloc(m * n * 2)
    ctx.gate_up_silu(gate, up, dx.ptr, q4b.F16, m, dy.ptr)
    y = dy.download(np.float16, (m, n))
    _, ref = orc.gate_up_silu(gq, gm, uq, um, k // 64, x, want32=False)
    assert_close(y, ref, f"gate/up {k}->{n} M={m}")


@pytest.mark.parametrize("m", [1, 4])
@pytest.mark.parametrize("name,k,n", BIG)
def test_27b_projections(q4b, orc, ctx, name, k, n, m):
    weight = ctx.synth_weight(0, 2, n, k // 64)
    quants, meta = orc.synth_weight(0, 2, n, k // 64)
    x = orc.synth_x(0, 0, m, k)
    y = run_matmul(q4b, ctx, weight, x)
    _, ref = orc.matmul(quants, meta, k // 64, x, want32=False)
    assert_close(y, ref, f"27B {name} M={m}")


@pytest.mark.parametrize("m", [2, 8, 9, 16, 17, 32, 45])
def test_other_batch_sizes(q4b, orc, ctx, m):
    n, k = 1024, 2048
    quants, meta = orc.synth_weight(1, 0, n, k // 64)
    x = orc.synth_x(1, 0, m, k)
    weight = ctx.upload(quants, meta, n, k // 64)
    y = run_matmul(q4b, ctx, weight, x)
    _, ref = orc.matmul(quants, meta, k // 64, x, want32=False)
    assert_close(y, ref, f"M={m}")


def test_grouped_qkv_launch_equals_separate(q4b, orc, ctx):
    k = 5120
    shapes = [6144, 1024, 1024]
    x = orc.synth_x(0, 0, 4, k)
    dx = ctx.to_device(x)
    weights, refs = [], []
    for index, n in enumerate(shapes):
        quants, meta = orc.synth_weight(0, index, n, k // 64)
        weights.append(ctx.upload(quants, meta, n, k // 64))
        refs.append(orc.matmul(quants, meta, k // 64, x, want32=False)[1])
    outs = [ctx.alloc(4 * n * 2) for n in shapes]
    ctx.matmul_group(weights, dx.ptr, q4b.F16, 4, [o.ptr for o in outs])
    for n, out, ref in zip(shapes, outs, refs):
        assert_close(out.download(np.float16, (4, n)), ref, f"group member {n}")


def test_float_x_and_residuals(q4b, orc, ctx):
    # second projections take fp32 x and add a residual (qwen38_layer.metal:193-255)
    n, k = 1024, 3072
    quants, meta = orc.synth_weight(0, 6, n, k // 64)
    weight = ctx.upload(quants, meta, n, k // 64)
    for m in (1, 4):
        x = orc.synth_x(0, 0, m, k).astype(np.float32) * np.float32(1.0009765625)
        for residual in (orc.synth_x(0, 7, m, n), orc.synth_x(0, 7, m, n).astype(np.float32)):
            y = run_matmul(q4b, ctx, weight, x, q4b.F32, residual)
            _, ref = orc.matmul(quants, meta, k // 64, x, residual=residual, want32=False)
            assert_close(y, ref, f"fp32 x + {residual.dtype} residual M={m}")


def test_ragged_rows_and_wide_output(q4b, orc, ctx):
    # N not a multiple of 16 and ldy > N (a shard writing its slice of a wider y)
    n, k, m, ldy = 100, 320, 3, 160
    quants, meta = orc.synth_weight(2, 0, n, k // 64)
    x = orc.synth_x(2, 0, m, k)
    weight = ctx.upload(quants, meta, n, k // 64)
    dx = ctx.to_device(x)
    canvas = np.full((m, ldy), 7.0, dtype=np.float16)
    dy = ctx.to_device(canvas)
    ctx.matmul(weight, dx.ptr, q4b.F16, m, dy.ptr + 2 * 20, q4b.F16, ldy)
    out = dy.download(np.float16, (m, ldy))
    _, ref = orc.matmul(quants, meta, k // 64, x, want32=False)
    assert_close(out[:, 20:120], ref, "ragged")
    assert (out[:, :20] == 7.0).all() and (out[:, 120:] == 7.0).all()  # guard columns untouched


def test_reference_fixture_patterns(q4b, orc, ctx):
    # the reference benches' closed-form inputs (qwen38_m3.m:64-87,:568-580)
    hidden, rows = 5120, 256
    groups = hidden // 64
    x = orc.activation_sincos(hidden).reshape(1, hidden)
    gq, gm = orc.fill_weights_xorshift(rows * groups, 0x36a110c)
    uq, um = orc.fill_weights_xorshift(rows * groups, 0x27b4c51)
    gate, up = ctx.upload(gq, gm, rows, groups), ctx.upload(uq, um, rows, groups)
    y, _ = ctx.gate_up_silu_host(gate, up, x, q4b.F32)
    ref32, ref64 = orc.gate_up_silu(gq, gm, uq, um, groups, x)
    assert_close(y, ref64, "xorshift gate/up")
    # the reference's own self-check style: first 8 rows against the fp32 scalar CPU sum
    assert np.max(np.abs(y[0, :8] - ref32[0, :8])) < 2.6e-3
    # H3 arithmetic pattern (minimax_h3_m3_gemm.m:75-104)
    hq, hm, hx = orc.h3_pattern(128, 84, 5376, 17)
    weight = ctx.upload(hq, hm, 128, 84)
    y, _ = ctx.matmul_host(weight, hx.reshape(1, -1), q4b.F32)
    _, ref = orc.matmul(hq, hm, 84, hx.reshape(1, -1), want32=False)
    assert_close(y, ref, "H3 pattern")


# bits 0-3 CTAs per SM, bit 4 fp16 form at M <= 4, bits 8-11 limit on K parts, bit 13 no clusters for a split K,
# bit 14 no dependent launch, bit 16 first ring fill not held back
@pytest.mark.parametrize("variant", [0x0001, 0x0002, 0x0010, 0x0100, 0x0300, 0x0211, 0x2000, 0x2010, 0x4000, 0x4012, 0x10000])
def test_kernel_variants_agree(q4b, orc, ctx, variant):
    n, k = 2048, 5120
    quants, meta = orc.synth_weight(3, 0, n, k // 64)
    weight = ctx.upload(quants, meta, n, k // 64)
    try:
        ctx.set_variant(variant)
        for m in (1, 4):
            x = orc.synth_x(3, 0, m, k)
            y = run_matmul(q4b, ctx, weight, x)
            _, ref = orc.matmul(quants, meta, k // 64, x, want32=False)
            assert_close(y, ref, f"variant {variant:#x} M={m}")
    finally:
        ctx.set_variant(0)


# ---------------------------------------------------------------- errors
def test_bad_arguments_return_status_1(q4b, orc, ctx):
    quants, meta = orc.synth_weight(0, 0, 64, 2)
    with pytest.raises(q4b.Q4Error) as info:
        ctx.upload(quants, meta, 64, 2, 60, 10)  # slice past the end
    assert info.value.status == 1
    weight = ctx.upload(quants, meta, 64, 2)
    dx = ctx.alloc(4096)
    with pytest.raises(q4b.Q4Error) as info:
        ctx.matmul(weight, dx.ptr, q4b.F16, 0, dx.ptr)  # M = 0
    assert info.value.status == 1
    with pytest.raises(q4b.Q4Error) as info:
        ctx.matmul(weight, dx.ptr + 2, q4b.F16, 1, dx.ptr)  # misaligned x
    assert info.value.status == 1
    with pytest.raises(q4b.Q4Error):
        ctx.matmul(weight, dx.ptr, q4b.F16, 1, dx.ptr, q4b.F16, 8)  # ldy < rows
    ctx.sync()  # the context is still usable


def test_gate_up_integer_form_on_awkward_activations(q4b, orc, ctx):
    """Fused gate/up at M <= 4 turns x into two 8-bit digits per value with a power-of-two step per group
    (the default there; variant bit 4 keeps the fp16 form).  Rows that stress the digits: zeros, values around
    the top of a binade (high digit at its limit), ties of the high digit, tiny and huge magnitudes, and one
    outlier per group that pushes everything else into the low digit."""
    n, k = 640, 1024
    groups = k // 64
    gq, gm = orc.synth_weight(51, 0, n, groups)
    uq, um = orc.synth_weight(51, 1, n, groups)
    gate, up = ctx.upload(gq, gm, n, groups), ctx.upload(uq, um, n, groups)
    rng = np.random.default_rng(51)
    base = rng.standard_normal((4, k)).astype(np.float32)
    cases = {
        "zeros and binade tops": np.stack([np.zeros(k, np.float32), np.where(base[1] > 0, 1.9990234, -1.9990234),
                                           np.where(base[2] > 0, 0.99951172, 0.5), base[3]]),
        "ties of the high digit": np.stack([np.round(base[0] * 8) / 8 + 0.0625, np.full(k, 1.5, np.float32),
                                            np.full(k, -1.5, np.float32), np.round(base[3] * 16) / 16]),
        "tiny and huge": np.stack([base[0] * 1e-4, base[1] * 3e-3, base[2] * 900.0, base[3] * 6000.0]),
        "one outlier per group": np.stack([np.where(np.arange(k) % 64 == 5, 200.0, base[m] * 0.01)
                                           for m in range(4)]).astype(np.float32),
    }
    for name, values in cases.items():
        x = values.astype(np.float16)
        for m in (1, 4):
            _, ref = orc.gate_up_silu(gq, gm, uq, um, groups, x[:m], want32=False)
            dx, dy = ctx.to_device(x[:m]), ctx.alloc(m * n * 4)
            got = {}
            try:
                for variant in (0, 0x10):
                    ctx.set_variant(variant)
                    ctx.gate_up_silu(gate, up, dx.ptr, q4b.F16, m, dy.ptr, q4b.F32)
                    got[variant] = dy.download(np.float32, (m, n))
            finally:
                ctx.set_variant(0)
            for row in range(m):
                scale = float(np.max(np.abs(ref[row])))
                if scale == 0.0:
                    assert not got[0][row].any() and not got[0x10][row].any(), name
                    continue
                for variant in (0, 0x10):
                    error = float(np.max(np.abs(got[variant][row] - ref[row]))) / scale
                    assert error <= 2e-3, (name, m, row, hex(variant), error)
    gate.free()
    up.free()
