"""Properties of the decode kernel that need no second implementation to compare with, and its less common inputs.

* The reference's exact batched GEMM gives row r of a batch the bits of a batch of one
  (qwen38_prefill.metal:5-9, :144-175).  Here that holds inside each arithmetic form: the integer form
  (M <= 4) and the fp16 form (M = 5..16, or any M with variant bit 4).
* fp32 activations are multiplied as the reference's second projections do (cpu_q4_dot_float,
  qwen38_m3_layer.m:375-393) whatever their magnitude: a row mixing 1e-3 and 3e4, and one far outside
  fp16's range.
* Non-finite activations give non-finite outputs in the row they sit in and leave the other rows alone.
* A sequence launch recorded into a graph replays correctly (the launch count lives in device memory).
* A K split whose parts meet in a cluster's shared memory gives the bits of the same split summed through
  global memory (variant bit 13), for every arithmetic form, plain and fused.
"""
import numpy as np
import pytest

from q4_cases import assert_close, bits_equal, relative_error

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx(q4b):
    context = q4b.Q4Context(0)
    yield context
    context.close()


def run(q4b, ctx, weight, x, y_dtype, up=None):
    m = x.shape[0]
    dx = ctx.to_device(x)
    width = 4 if y_dtype == q4b.F32 else 2
    dy = ctx.alloc(m * weight.rows * width)
    x_code = q4b.F16 if x.dtype == np.float16 else q4b.F32
    if up is None:
        ctx.matmul(weight, dx.ptr, x_code, m, dy.ptr, y_dtype)
    else:
        ctx.gate_up_silu(weight, up, dx.ptr, x_code, m, dy.ptr, y_dtype)
    return dy.download(np.float32 if y_dtype == q4b.F32 else np.float16, (m, weight.rows))


@pytest.mark.parametrize("n,k", [(1024, 2048), (5120, 17408), (200, 320)])
@pytest.mark.parametrize("fused", [False, True])
def test_row_result_does_not_depend_on_batch(q4b, orc, ctx, n, k, fused):
    groups = k // 64
    weight = ctx.synth_weight(11, 0, n, groups)
    up = ctx.synth_weight(11, 1, n, groups) if fused else None
    x = orc.synth_x(11, 0, 16, k)
    try:
        # integer form: M = 1..4
        single = [run(q4b, ctx, weight, x[r:r + 1], q4b.F32, up) for r in range(4)]
        for m in (2, 3, 4):
            batch = run(q4b, ctx, weight, x[:m], q4b.F32, up)
            for r in range(m):
                assert bits_equal(batch[r], single[r][0]), f"integer form M={m} row {r}"
        # fp16 form: any M up to 16 (variant bit 4 keeps it at M <= 4)
        ctx.set_variant(0x10)
        single = [run(q4b, ctx, weight, x[r:r + 1], q4b.F32, up) for r in (0, 3, 7, 15)]
        for m in (4, 8, 9, 16):
            batch = run(q4b, ctx, weight, x[:m], q4b.F32, up)
            for index, r in enumerate((0, 3, 7, 15)):
                if r < m:
                    assert bits_equal(batch[r], single[index][0]), f"fp16 form M={m} row {r}"
    finally:
        ctx.set_variant(0)
        weight.free()
        if up is not None:
            up.free()


@pytest.mark.parametrize("n,k,fused", [(5120, 6144, False), (5120, 17408, False), (1024, 5120, False),
                                       (3072, 1024, True), (200, 2048, False), (640, 6144, False)])
def test_cluster_sum_equals_global_memory_sum(q4b, orc, ctx, n, k, fused):
    groups = k // 64
    weight = ctx.synth_weight(17, 0, n, groups)
    up = ctx.synth_weight(17, 1, n, groups) if fused else None
    x = orc.synth_x(17, 0, 16, k)
    try:
        for m, form in ((1, 0), (3, 0), (4, 0x10), (8, 0), (16, 0)):
            got = {}
            for clusters_off in (0, 0x2000):
                ctx.set_variant(form | clusters_off)
                got[clusters_off] = run(q4b, ctx, weight, x[:m], q4b.F32, up)
                again = run(q4b, ctx, weight, x[:m], q4b.F32, up)
                assert bits_equal(got[clusters_off], again), f"M={m} variant {form | clusters_off:#x} repeats"
            assert bits_equal(got[0], got[0x2000]), f"M={m} form {form:#x}"
        quants, meta = orc.synth_weight(17, 0, n, groups)
        if not fused:
            _, ref = orc.matmul(quants, meta, groups, x[:4], want32=False)
            ctx.set_variant(0)
            assert_close(run(q4b, ctx, weight, x[:4], q4b.F32), ref, "cluster sum against the oracle")
    finally:
        ctx.set_variant(0)
        weight.free()
        if up is not None:
            up.free()


@pytest.mark.parametrize("m", [1, 4, 7, 16])
def test_float_activations_of_any_magnitude(q4b, orc, ctx, m):
    n, k = 768, 3072
    groups = k // 64
    quants, meta = orc.synth_weight(12, 0, n, groups)
    weight = ctx.upload(quants, meta, n, groups)
    rng = np.random.default_rng(12)
    base = rng.standard_normal((m, k)).astype(np.float32)
    # magnitudes from 1e-3 to 3e4 inside one row, as silu(g) * u produces them
    wide = base * (10.0 ** rng.uniform(-3.0, 4.5, size=(m, k))).astype(np.float32)
    # far outside fp16's range, and far below it
    huge = base * np.float32(3.0e7)
    tiny = base * np.float32(1.0e-9)
    for name, x in (("wide", wide), ("huge", huge), ("tiny", tiny)):
        y = run(q4b, ctx, weight, x, q4b.F32)
        _, ref = orc.matmul(quants, meta, groups, x, want32=False)
        assert np.isfinite(y).all(), name
        assert_close(y, ref, f"fp32 x ({name}) M={m}")
    weight.free()


@pytest.mark.parametrize("m", [2, 4, 6])
@pytest.mark.parametrize("x_type", [np.float16, np.float32])
def test_non_finite_activations_propagate(q4b, orc, ctx, m, x_type):
    n, k = 256, 1024
    groups = k // 64
    quants, meta = orc.synth_weight(13, 0, n, groups)
    weight = ctx.upload(quants, meta, n, groups)
    uq, um = orc.synth_weight(13, 1, n, groups)
    up = ctx.upload(uq, um, n, groups)
    x = orc.synth_x(13, 0, m, k).astype(x_type)
    x[0, 70] = np.inf
    x[1, 1000] = np.nan
    try:
        if m > 4:
            ctx.set_variant(0x10)  # so that the run without the bad rows (M - 2 <= 4) uses the same arithmetic form
        for fused in (False, True):
            y = run(q4b, ctx, weight, x, q4b.F32, up if fused else None)
            assert not np.isfinite(y[0]).any() and not np.isfinite(y[1]).any(), "rows holding inf / NaN"
            if m > 2:
                clean = run(q4b, ctx, weight, np.ascontiguousarray(x[2:]), q4b.F32, up if fused else None)
                assert np.isfinite(y[2:]).all()
                assert bits_equal(y[2:], clean), "the other rows are untouched"
    finally:
        ctx.set_variant(0)
        weight.free()
        up.free()


def test_recorded_sequence_replays(q4b, orc, ctx):
    """A chain in which every job reads what the job before it wrote, recorded once and replayed: every replay
    must wait for its own predecessors (a launch counter frozen into the recording would let the second replay
    read x before it is written)."""
    k0, n1, n2, n3, m = 1024, 2048, 1024, 512, 2
    w1q, w1m = orc.synth_weight(14, 0, n1, k0 // 64)
    w2q, w2m = orc.synth_weight(14, 1, n2, n1 // 64)
    w3q, w3m = orc.synth_weight(14, 2, n3, n2 // 64)
    w1, w2, w3 = (ctx.upload(w1q, w1m, n1, k0 // 64), ctx.upload(w2q, w2m, n2, n1 // 64),
                  ctx.upload(w3q, w3m, n3, n2 // 64))
    dx = ctx.alloc(m * k0 * 2)
    a, b, c = ctx.alloc(m * n1 * 2), ctx.alloc(m * n2 * 2), ctx.alloc(m * n3 * 4)
    sequence = q4b.Q4Sequence(ctx, m)
    sequence.add_matmul([w1], dx.ptr, [a.ptr])
    sequence.add_matmul([w2], a.ptr, [b.ptr])
    sequence.add_matmul([w3], b.ptr, [c.ptr], y_dtype=q4b.F32)
    sequence.finalize()

    def expected(x):
        y1 = orc.matmul(w1q, w1m, k0 // 64, x, want32=False)[1].astype(np.float16)
        y2 = orc.matmul(w2q, w2m, n1 // 64, y1, want32=False)[1].astype(np.float16)
        return orc.matmul(w3q, w3m, n2 // 64, y2, want32=False)[1]

    x = orc.synth_x(14, 0, m, k0)
    dx.upload(x)
    sequence.launch()   # a plain launch first
    assert relative_error(c.download(np.float32, (m, n3)), expected(x)) < 5e-3
    ctx.graph_begin()
    sequence.launch()
    graph = ctx.graph_end()
    for replay in range(4):
        x = orc.synth_x(15 + replay, 0, m, k0)
        dx.upload(x)
        # poison the intermediates: a replay that does not wait would read these
        a.upload(np.full((m, n1), 300.0, np.float16))
        b.upload(np.full((m, n2), -300.0, np.float16))
        graph.launch()
        got = c.download(np.float32, (m, n3))
        assert relative_error(got, expected(x)) < 5e-3, f"replay {replay}"
    sequence.launch()   # and a plain launch after the replays still counts correctly
    assert relative_error(c.download(np.float32, (m, n3)), expected(x)) < 5e-3
    graph.free()
    sequence.free()
    for w in (w1, w2, w3):
        w.free()


def test_sequence_with_float_activations_and_residual(q4b, orc, ctx):
    # the reference's second projections inside a sequence: fp32 x, residual added (qwen38_layer.metal:193-255)
    n, k, m = 1024, 3072, 3
    groups = k // 64
    quants, meta = orc.synth_weight(16, 0, n, groups)
    weight = ctx.upload(quants, meta, n, groups)
    x = (orc.synth_x(16, 0, m, k).astype(np.float32) * np.float32(700.0))
    residual = orc.synth_x(16, 1, m, n).astype(np.float32)
    dx, dr, dy = ctx.to_device(x), ctx.to_device(residual), ctx.alloc(m * n * 4)
    sequence = q4b.Q4Sequence(ctx, m)
    sequence.add_projection(weight, dx.ptr, q4b.F32, dy.ptr, q4b.F32, None, dr.ptr, q4b.F32, n)
    sequence.finalize()
    sequence.launch()
    _, ref = orc.matmul(quants, meta, groups, x, residual=residual, want32=False)
    assert_close(dy.download(np.float32, (m, n)), ref, "sequence fp32 x + residual")
    sequence.free()
    weight.free()
