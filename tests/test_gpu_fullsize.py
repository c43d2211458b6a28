"""The largest matrices of the reference model at their full sizes, checked through
sampled rows (the oracle generates just those rows of the seeded matrix) and
through properties that need no oracle: the lm_head 5120 -> 248,320
(qwen38_q4_lm_head, qwen38_global.metal:37-61), the fused attention in-projection
5120 -> 14,336 (qwen38_attention.metal:28-52) and the DeltaNet in-projection
5120 -> 16,480, whose row count is not a multiple of 64 (qwen38_layer.metal:71-100)."""
import numpy as np
import pytest

from q4_cases import assert_close, bits_equal

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx(q4b):
    context = q4b.Q4Context(0)
    yield context
    context.close()


def sample_rows(n, rng):
    edges = [0, 1, 15, 16, 63, 64, 127, 128, n - 129, n - 65, n - 64, n - 17, n - 16, n - 2, n - 1]
    return np.unique(np.concatenate([np.array([r for r in edges if 0 <= r < n]), rng.integers(0, n, 48)]))


@pytest.mark.parametrize("name,n,k,m", [("lm_head", 248320, 5120, 1), ("lm_head", 248320, 5120, 4),
                                        ("attention_inputs", 14336, 5120, 1), ("delta_inputs", 16480, 5120, 1),
                                        ("delta_inputs", 16480, 5120, 4), ("delta_inputs", 16480, 5120, 64)])
def test_full_size_matrix_on_sampled_rows(q4b, orc, ctx, name, n, k, m):
    groups = k // 64
    seed, projection = 21, 3
    weight = ctx.synth_weight(seed, projection, n, groups)
    x = orc.synth_x(seed, 0, m, k)
    dx = ctx.to_device(x)
    dy = ctx.to_device(np.full((m, n), 9.0, dtype=np.float16))
    ctx.matmul(weight, dx.ptr, q4b.F16, m, dy.ptr)
    y = dy.download(np.float16, (m, n))
    assert np.isfinite(y.astype(np.float32)).all()
    rows = sample_rows(n, np.random.default_rng(n + m))
    quants, meta = orc.synth_weight_rows(seed, projection, groups, rows)
    _, ref = orc.matmul(quants, meta, groups, x, want32=False)
    assert_close(y[:, rows], ref, f"{name} M={m}")
    # the same call again gives the same bits: the split-K sums do not depend on timing
    ctx.matmul(weight, dx.ptr, q4b.F16, m, dy.ptr)
    assert bits_equal(dy.download(np.float16, (m, n)), y)
    # linearity in x: y(2x) = 2 y(x) bit for bit (fp32 outputs, so that no result is an fp16 subnormal)
    d32 = ctx.alloc(m * n * 4)
    ctx.matmul(weight, dx.ptr, q4b.F16, m, d32.ptr, q4b.F32)
    single = d32.download(np.float32, (m, n))
    d2 = ctx.to_device((x.astype(np.float32) * 2).astype(np.float16))
    ctx.matmul(weight, d2.ptr, q4b.F16, m, d32.ptr, q4b.F32)
    assert np.array_equal(d32.download(np.float32, (m, n)), single * 2)
    weight.free()
