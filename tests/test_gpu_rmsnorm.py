"""RMS norm in front of the matmuls (q4b_rmsnorm) against the oracle's restatement of
qwen38_rmsnorm_f16_to_f16 / _f32_to_f16 (qwen38_layer.metal:21-69): bit-exact, because
both sides do the same separately rounded fp32 operations in the same order; and as the
producer of x for an in-projection, within the matmul tolerance."""
import numpy as np
import pytest

from q4_cases import assert_close, bits_equal

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx(q4b):
    context = q4b.Q4Context(0)
    yield context
    context.close()


@pytest.mark.parametrize("hidden,batch", [(5120, 1), (5120, 4), (1024, 33), (200, 3), (17408, 2)])
@pytest.mark.parametrize("dtype_name", ["F16", "F32"])
def test_rmsnorm_is_bit_exact(q4b, orc, ctx, hidden, batch, dtype_name):
    rng = np.random.default_rng(hidden + batch)
    values = (rng.standard_normal((batch, hidden)) * rng.uniform(0.01, 30.0, size=(batch, 1))).astype(np.float32)
    if dtype_name == "F16":
        values = values.astype(np.float16)
    weight = rng.uniform(0.5, 1.5, size=hidden).astype(np.float32)
    want = orc.rmsnorm(values, weight, 1e-6)
    d_in, d_w, d_out = ctx.to_device(values), ctx.to_device(weight), ctx.alloc(batch * hidden * 2)
    ctx.rmsnorm(d_in.ptr, getattr(q4b, dtype_name), d_w.ptr, d_out.ptr, hidden, batch, 1e-6)
    got = d_out.download(np.float16, (batch, hidden))
    assert bits_equal(got, want)
    # and the reference's own CPU check of this step (cpu_rms_half / cpu_rms_float, qwen38_m3_layer.m:395-420:
    # double sum, float inverse): its sum is taken in another order, so equal to one fp16 ulp, mostly bit for bit
    reference = orc.rmsnorm_reference(values, weight, 1e-6)
    steps = np.abs(got.view(np.int16).astype(np.int32) - reference.view(np.int16).astype(np.int32))
    assert steps.max() <= 1 and np.mean(steps == 0) > 0.9


def test_rmsnorm_feeds_an_in_projection(q4b, orc, ctx):
    hidden, rows, batch = 1024, 768, 4
    groups = hidden // 64
    quants, meta = orc.synth_weight(41, 0, rows, groups)
    weight = ctx.upload(quants, meta, rows, groups)
    rng = np.random.default_rng(41)
    state = rng.standard_normal((batch, hidden)).astype(np.float32) * 3.0
    gain = rng.uniform(0.5, 1.5, size=hidden).astype(np.float32)
    d_state, d_gain = ctx.to_device(state), ctx.to_device(gain)
    d_x, d_y = ctx.alloc(batch * hidden * 2), ctx.alloc(batch * rows * 4)
    ctx.rmsnorm(d_state.ptr, q4b.F32, d_gain.ptr, d_x.ptr, hidden, batch)
    ctx.matmul(weight, d_x.ptr, q4b.F16, batch, d_y.ptr, q4b.F32)
    _, want = orc.matmul(quants, meta, groups, orc.rmsnorm(state, gain), want32=False)
    assert_close(d_y.download(np.float32, (batch, rows)), want, "rms norm -> in-projection")
    weight.free()


def test_rmsnorm_refuses_bad_arguments(q4b, ctx):
    buffer = ctx.alloc(4096)
    for arguments in ((0, q4b.F32, buffer.ptr, buffer.ptr, 64, 1), (buffer.ptr, q4b.BF16, buffer.ptr, buffer.ptr, 64, 1),
                      (buffer.ptr, q4b.F32, buffer.ptr, buffer.ptr, 0, 1), (buffer.ptr, q4b.F32, buffer.ptr, buffer.ptr, 64, 0)):
        with pytest.raises(q4b.Q4Error) as refused:
            ctx.rmsnorm(*arguments)
        assert refused.value.status == 1
