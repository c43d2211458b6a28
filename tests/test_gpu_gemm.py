"""Parity of the tcgen05 prefill GEMM (M > 16, through the C ABI) with the oracle.

Outputs: max|y - ref| / max|ref| <= 2e-3 against the oracle's double sum on
sampled weight rows (the oracle is a scalar loop); the multiplied weights are the
bit-exact W16 values (gate in test_gpu_parity.py).  At the full sizes of the 27B
layer set (M up to 8192) the oracle runs on sampled weight rows x sampled
activation rows, the edges of the first and last weight block and activation
block among them.
"""
import numpy as np
import pytest

from q4_cases import assert_close, relative_error

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx(q4b):
    context = q4b.Q4Context(0)
    yield context
    context.close()


def oracle_rows(orc, quants, meta, groups, x, rows, residual=None):
    """Oracle output for a sample of weight rows: [M, len(rows)] in double."""
    cols = []
    for row in rows:
        res = None if residual is None else np.ascontiguousarray(residual[:, row:row + 1])
        cols.append(orc.matmul(quants, meta, groups, x, row_begin=int(row), row_count=1, residual=res,
                               want32=False)[1])
    return np.concatenate(cols, axis=1)


# the last four have few tiles for 148 SMs: their (tile, group) iterations are split evenly over the CTAs
@pytest.mark.parametrize("n,k,m", [(256, 128, 64), (128, 64, 17), (384, 320, 300), (1024, 2048, 128),
                                   (1000, 1024, 257), (2048, 5120, 512), (5120, 17408, 512), (640, 6144, 512),
                                   (2560, 5120, 100), (1100, 4096, 700)])
def test_gemm_matches_oracle(q4b, orc, ctx, n, k, m):
    groups = k // 64
    quants, meta = orc.synth_weight(3, 0, n, groups)
    x = orc.synth_x(3, 0, m, k)
    weight = ctx.upload(quants, meta, n, groups)
    dx, dy = ctx.to_device(x), ctx.to_device(np.full((m, n), 7.0, dtype=np.float16))
    ctx.matmul(weight, dx.ptr, q4b.F16, m, dy.ptr)
    y = dy.download(np.float16, (m, n))
    rows = np.unique(np.concatenate([np.arange(0, min(n, 20)), np.arange(n - 20, n),
                                     np.random.default_rng(1).integers(0, n, 40)]))
    ref = oracle_rows(orc, quants, meta, groups, x, rows)
    assert_close(y[:, rows], ref, f"gemm {n}x{k} M={m}")
    assert np.isfinite(y.astype(np.float32)).all()


@pytest.mark.parametrize("m,n,k", [(64, 640, 1024), (200, 640, 1024), (300, 3072, 5120), (512, 2176, 5120)])
def test_gemm_fused_gate_up(q4b, orc, ctx, m, n, k):
    groups = k // 64
    gq, gm = orc.synth_weight(0, 4, n, groups)
    uq, um = orc.synth_weight(0, 5, n, groups)
    x = orc.synth_x(0, 0, m, k)
    gate, up = ctx.upload(gq, gm, n, groups), ctx.upload(uq, um, n, groups)
    dx, dy = ctx.to_device(x), ctx.alloc(m * n * 2)
    ctx.gate_up_silu(gate, up, dx.ptr, q4b.F16, m, dy.ptr)
    y = dy.download(np.float16, (m, n))
    _, ref = orc.gate_up_silu(gq, gm, uq, um, groups, x, want32=False)
    assert_close(y, ref, f"fused gemm M={m}")


def test_gemm_float_x_residual_and_wide_output(q4b, orc, ctx):
    n, k, m, ldy = 200, 512, 70, 256
    groups = k // 64
    quants, meta = orc.synth_weight(2, 0, n, groups)
    weight = ctx.upload(quants, meta, n, groups)
    x = orc.synth_x(2, 0, m, k).astype(np.float32)
    residual = orc.synth_x(2, 9, m, n).astype(np.float32)
    dx, dr = ctx.to_device(x), ctx.to_device(residual)
    canvas = np.full((m, ldy), 5.0, dtype=np.float32)
    dy = ctx.to_device(canvas)
    ctx.matmul(weight, dx.ptr, q4b.F32, m, dy.ptr + 4 * 16, q4b.F32, ldy, dr.ptr, q4b.F32, n)
    out = dy.download(np.float32, (m, ldy))
    _, ref = orc.matmul(quants, meta, groups, x, residual=residual, want32=False)
    assert_close(out[:, 16:216], ref, "fp32 x + residual")
    assert (out[:, :16] == 5.0).all() and (out[:, 216:] == 5.0).all()


@pytest.mark.parametrize("name,k,n", [("q", 5120, 6144), ("down", 17408, 5120)])
def test_gemm_full_size_agrees_with_small_m_kernel(q4b, orc, ctx, name, k, n):
    m = 2048
    weight = ctx.synth_weight(0, 2, n, k // 64)
    dx = ctx.synth_x(0, 0, m, k)
    dy = ctx.alloc(m * n * 2)
    ctx.matmul(weight, dx.ptr, q4b.F16, m, dy.ptr)
    y = dy.download(np.float16, (m, n))
    picks = [0, 1, 255, 256, 1000, 2047]
    x_rows = dx.download(np.float16, (m, k))[picks]
    dxs, dys = ctx.to_device(x_rows), ctx.alloc(len(picks) * n * 2)
    ctx.matmul(weight, dxs.ptr, q4b.F16, len(picks), dys.ptr)   # small-M kernel
    small = dys.download(np.float16, (len(picks), n))
    assert relative_error(y[picks], small.astype(np.float64)) < 1e-3
    # and a sample against the oracle itself
    quants, meta = orc.synth_weight(0, 2, n, k // 64)
    rows = np.array([0, 63, 64, 127, 128, n - 1])
    ref = oracle_rows(orc, quants, meta, k // 64, x_rows, rows)
    assert_close(small[:, rows], ref, f"{name} small-M")
    assert_close(y[picks][:, rows], ref, f"{name} gemm")


def test_gemm_grouped_launch(q4b, orc, ctx):
    # q, k, v share x and one launch (the reference fuses them into one matrix)
    k, m = 1024, 150
    shapes = [640, 128, 200]
    x = orc.synth_x(0, 0, m, k)
    dx = ctx.to_device(x)
    weights, refs = [], []
    for index, n in enumerate(shapes):
        quants, meta = orc.synth_weight(0, index, n, k // 64)
        weights.append(ctx.upload(quants, meta, n, k // 64))
        refs.append(orc.matmul(quants, meta, k // 64, x, want32=False)[1])
    outs = [ctx.alloc(m * n * 2) for n in shapes]
    before = ctx.launches
    ctx.matmul_group(weights, dx.ptr, q4b.F16, m, [o.ptr for o in outs])
    assert ctx.launches - before == 1
    for n, out, ref in zip(shapes, outs, refs):
        assert_close(out.download(np.float16, (m, n)), ref, f"group member {n}")


def sampled(count, rng, picks=24):
    edges = [0, 1, 63, 64, 127, 128, 255, 256, count - 257, count - 256, count - 129, count - 128, count - 65,
             count - 64, count - 2, count - 1]
    return np.unique(np.concatenate([np.array([e for e in edges if 0 <= e < count]), rng.integers(0, count, picks)]))


# the 27B layer set at the prefill sizes: every weight block and every activation block is hit by the
# samples' edges; whole outputs must be finite
@pytest.mark.parametrize("name,k,n,m", [("q", 5120, 6144, 8192), ("k", 5120, 1024, 512), ("k", 5120, 1024, 8192),
                                        ("o", 6144, 5120, 8192), ("down", 17408, 5120, 8192)])
def test_gemm_27b_shapes_on_sampled_rows(q4b, orc, ctx, name, k, n, m):
    groups = k // 64
    seed, projection = 31, 2
    weight = ctx.synth_weight(seed, projection, n, groups)
    dx = ctx.synth_x(seed, 0, m, k)
    dy = ctx.alloc(m * n * 2)
    ctx.matmul(weight, dx.ptr, q4b.F16, m, dy.ptr)
    y = dy.download(np.float16, (m, n))
    assert np.isfinite(y.astype(np.float32)).all()
    rng = np.random.default_rng(m + n)
    rows, acts = sampled(n, rng), sampled(m, rng, 8)
    x = dx.download(np.float16, (m, k))[acts]
    quants, meta = orc.synth_weight_rows(seed, projection, groups, rows)
    _, ref = orc.matmul(quants, meta, groups, x, want32=False)
    scale = float(np.max(np.abs(y.astype(np.float32))))
    error = float(np.max(np.abs(y[np.ix_(acts, rows)].astype(np.float64) - ref))) / scale
    assert error <= 2e-3, f"{name} M={m}: {error:.3e}"
    weight.free()


@pytest.mark.parametrize("m", [512, 2048, 8192])
def test_gemm_fused_gate_up_full_width(q4b, orc, ctx, m):
    k, n = 5120, 17408
    groups = k // 64
    seed = 32
    gate, up = ctx.synth_weight(seed, 4, n, groups), ctx.synth_weight(seed, 5, n, groups)
    dx = ctx.synth_x(seed, 0, m, k)
    dy = ctx.alloc(m * n * 2)
    ctx.gate_up_silu(gate, up, dx.ptr, q4b.F16, m, dy.ptr)
    y = dy.download(np.float16, (m, n))
    assert np.isfinite(y.astype(np.float32)).all()
    rng = np.random.default_rng(m)
    rows, acts = sampled(n, rng), sampled(m, rng, 8)
    x = dx.download(np.float16, (m, k))[acts]
    gq, gm = orc.synth_weight_rows(seed, 4, groups, rows)
    uq, um = orc.synth_weight_rows(seed, 5, groups, rows)
    _, ref = orc.gate_up_silu(gq, gm, uq, um, groups, x, want32=False)
    scale = float(np.max(np.abs(y.astype(np.float32))))
    error = float(np.max(np.abs(y[np.ix_(acts, rows)].astype(np.float64) - ref))) / scale
    assert error <= 2e-3, f"fused gate/up M={m}: {error:.3e}"
    gate.free()
    up.free()


@pytest.mark.parametrize("m", [4646, 15485])
def test_h3_large_m_witness(q4b, orc, ctx, m):
    """The reference's largest affine-Q4 GEMM: 5376 -> 14336 at M = 15,485 rows and its 4,646-row sample
    (minimax_h3_m3_gemm.m:75-104 arithmetic fixture; models/minimax-h3/targets/apple-m3-pro/README.md:722-726),
    fp16 in and out.  Checked like the reference checks itself -- the first 8 outputs against a scalar fp32 sum,
    its bound 0.002581 -- and on sampled weight rows x sampled activation rows against the double sum."""
    n, k = 14336, 5376
    groups = k // 64
    quants, meta, x = orc.h3_pattern(n, groups, m * k, 17)
    x = x.reshape(m, k)
    weight = ctx.upload(quants, meta, n, groups)
    dx, dy = ctx.to_device(x), ctx.alloc(m * n * 2)
    ctx.matmul(weight, dx.ptr, q4b.F16, m, dy.ptr)
    y = dy.download(np.float16, (m, n))
    assert np.isfinite(y.astype(np.float32)).all()
    ref32, _ = orc.matmul(quants, meta, groups, x[:1], row_count=8, want64=False)
    assert np.max(np.abs(y[0, :8].astype(np.float32) - ref32[0])) <= 0.002581 + 2.0 ** -9  # + half an fp16 ulp of 2..4
    rng = np.random.default_rng(m)
    rows, acts = sampled(n, rng, 12), sampled(m, rng, 6)
    cols = []
    for row in rows:
        cols.append(orc.matmul(quants, meta, groups, np.ascontiguousarray(x[acts]), row_begin=int(row), row_count=1,
                               want32=False)[1])
    ref = np.concatenate(cols, axis=1)
    scale = float(np.max(np.abs(y.astype(np.float32))))
    assert float(np.max(np.abs(y[np.ix_(acts, rows)].astype(np.float64) - ref))) / scale <= 2e-3
    weight.free()
