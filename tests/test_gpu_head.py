"""The restricted head of the reference's draft passes (qwen38_m3_decode.m:1847-1866): the first rows of the
lm_head as an ordinary matmul on a row range of the loaded weight, and the listed extra rows after them
(qwen38_q4_lm_head_gathered, qwen38_global.metal:68-96)."""
import numpy as np
import pytest

from q4_cases import assert_close, bits_equal

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx(q4b):
    context = q4b.Q4Context(0)
    yield context
    context.close()


@pytest.mark.parametrize("m", [1, 3, 16])
def test_listed_rows_match_the_oracle(q4b, orc, ctx, m):
    n, k = 4000, 5120
    groups = k // 64
    quants, meta = orc.synth_weight(41, 0, n, groups)
    weight = ctx.upload(quants, meta, n, groups)
    x = orc.synth_x(41, 0, m, k)
    rng = np.random.default_rng(41)
    ids = np.concatenate([np.array([0, 7, 8, 15, 16, 63, 64, n - 1, n - 9, 5, 5]), rng.integers(0, n, 300)]).astype(np.uint32)
    d_ids, dx = ctx.to_device(ids), ctx.to_device(x)
    base = 24  # the reference writes the extras after the static prefix: logits[base + slot]
    ldy = base + len(ids) + 8
    canvas = np.full((m, ldy), 3.0, dtype=np.float32)
    dy = ctx.to_device(canvas)
    ctx.matmul_rows(weight, d_ids.ptr, len(ids), dx.ptr, q4b.F16, m, dy.ptr + 4 * base, q4b.F32, ldy)
    out = dy.download(np.float32, (m, ldy))
    _, ref = orc.matmul(quants, meta, groups, x, want32=False)
    assert_close(out[:, base:base + len(ids)], ref[:, ids], f"listed rows M={m}")
    assert (out[:, :base] == 3.0).all() and (out[:, base + len(ids):] == 3.0).all()
    # the reference's own check style: against its fp32 scalar sum on the first 8 listed rows
    ref32, _ = orc.matmul(quants, meta, groups, x, want64=False)
    assert np.max(np.abs(out[:, base:base + 8] - ref32[:, ids[:8]])) < 2.6e-3
    weight.free()


def test_listed_rows_of_a_shard_and_float_activations(q4b, orc, ctx):
    n, k, m = 1024, 1024, 2
    groups = k // 64
    quants, meta = orc.synth_weight(42, 0, n, groups)
    begin, count = 256, 512
    shard = ctx.upload(quants, meta, n, groups, begin, count)
    x = orc.synth_x(42, 0, m, k).astype(np.float32) * np.float32(1234.5)
    ids = np.array([0, 255, 256, 300, 767, 768, 1023], dtype=np.uint32)   # whole-matrix numbering
    d_ids, dx = ctx.to_device(ids), ctx.to_device(x)
    dy = ctx.to_device(np.full((m, len(ids)), -1.0, dtype=np.float32))
    ctx.matmul_rows(shard, d_ids.ptr, len(ids), dx.ptr, q4b.F32, m, dy.ptr, q4b.F32)
    out = dy.download(np.float32, (m, len(ids)))
    _, ref = orc.matmul(quants, meta, groups, x, want32=False)
    held = (ids >= begin) & (ids < begin + count)
    assert_close(out[:, held], ref[:, ids[held]], "rows of the shard")
    assert (out[:, ~held] == -1.0).all(), "rows of other shards are left to them"
    shard.free()


@pytest.mark.parametrize("m", [1, 4, 12, 64])
def test_row_range_of_a_weight_is_a_weight(q4b, orc, ctx, m):
    """The draft head's static prefix: the first `draft_vocab` rows of the lm_head through the ordinary matmul."""
    n, k = 3000, 2048
    groups = k // 64
    quants, meta = orc.synth_weight(43, 0, n, groups)
    weight = ctx.upload(quants, meta, n, groups)
    x = orc.synth_x(43, 0, m, k)
    dx = ctx.to_device(x)
    _, ref = orc.matmul(quants, meta, groups, x, want32=False)
    whole = ctx.alloc(m * n * 4)
    ctx.matmul(weight, dx.ptr, q4b.F16, m, whole.ptr, q4b.F32)
    full = whole.download(np.float32, (m, n))
    for begin, count in [(0, 1000), (0, 64), (128, 2872), (1024, 100), (2944, 56)]:
        part = weight.rows_view(begin, count)
        assert part.rows == count
        dy = ctx.alloc(m * count * 4)
        ctx.matmul(part, dx.ptr, q4b.F16, m, dy.ptr, q4b.F32)
        y = dy.download(np.float32, (m, count))
        assert_close(y, ref[:, begin:begin + count], f"rows [{begin}, +{count}) M={m}")
        if m <= 4:  # same split of K for the whole matrix and the range here: a row keeps its bits
            assert bits_equal(y, full[:, begin:begin + count])
        part.free()
    with pytest.raises(q4b.Q4Error):
        weight.rows_view(64, 100)   # not a multiple of 128
    with pytest.raises(q4b.Q4Error):
        weight.rows_view(2944, 100)  # past the end
    weight.free()
