"""The allocation-free entry point against the ordinary one.

Some hosts cannot let a library allocate device memory behind their back: they
own a fixed pool, or they cannot afford the device-wide stall that an allocation
or a free causes while other streams are mid-token.  q4b_matmul_no_alloc runs the
same kernel with its split-K scratch in an array built into the library, so its
results must equal q4b_matmul's -- on the first call and on the call after it,
which finds the array as the first one left it.  Collected last so that a failure
here cannot hide the other tests from a run that stops at the first failure.
"""
import numpy as np
import pytest

from q4_cases import assert_close

pytestmark = pytest.mark.gpu


def test_no_alloc_entry_point_matches_matmul_twice_in_a_row(q4b, orc):
    with q4b.Q4Context(0) as ctx:
        # shapes whose K range is split over thread blocks (they use the scratch) and one that is not
        for seed, (n, k, m) in enumerate([(1024, 5120, 1), (6144, 5120, 4), (5120, 17408, 1), (128, 64, 3), (1024, 2048, 7)]):
            quants, meta = orc.synth_weight(seed, 0, n, k // 64)
            weight = ctx.upload(quants, meta, n, k // 64)
            x = orc.synth_x(seed, 0, m, k)
            dx = ctx.to_device(x)
            want_buffer = ctx.alloc(m * n * 2)
            ctx.matmul(weight, dx.ptr, q4b.F16, m, want_buffer.ptr)
            want = want_buffer.download(np.float16, (m, n))
            _, ref = orc.matmul(quants, meta, k // 64, x, want32=False)
            assert_close(want, ref, "existing entry point")
            for attempt in range(2):
                got_buffer = ctx.to_device(np.full((m, n), 9.0, dtype=np.float16))
                ctx.matmul_no_alloc(weight, dx.ptr, q4b.F16, m, got_buffer.ptr)
                got = got_buffer.download(np.float16, (m, n))
                assert_close(got, want.astype(np.float64), f"no-alloc call {attempt + 1} for {n}x{k} M={m}")
                assert_close(got, ref, f"no-alloc call {attempt + 1} against the oracle")
            weight.free()


def test_no_alloc_entry_point_refuses_what_does_not_fit(q4b, orc):
    with q4b.Q4Context(0) as ctx:
        # 17408 -> 5120 has 40 blocks of 128 rows, so its K range is cut into 6 or 7 parts per block: 240 or 280
        # pieces.  At M = 16 a piece parks 8 KB of sums: 1.9 MB or more, beyond the 1 MiB the library carries.
        n, k, m = 5120, 17408, 16
        weight = ctx.synth_weight(0, 0, n, k // 64)
        dx = ctx.synth_x(0, 0, m, k)
        dy = ctx.alloc(m * n * 2)
        with pytest.raises(q4b.Q4Error) as info:
            ctx.matmul_no_alloc(weight, dx.ptr, q4b.F16, m, dy.ptr)
        assert info.value.status == 1 and "built-in scratch" in info.value.message
        ctx.matmul(weight, dx.ptr, q4b.F16, m, dy.ptr)  # the allocating entry point takes it
        ctx.matmul_no_alloc(weight, dx.ptr, q4b.F16, 4, dy.ptr)  # and at M = 4 it fits
        ctx.sync()
        # a matrix with more 128-row blocks than resident thread blocks needs no scratch at all
        n, k = 300_000, 64
        weight = ctx.synth_weight(0, 0, n, 1)
        dx = ctx.synth_x(0, 0, 1, k)
        dy = ctx.alloc(n * 2)
        ctx.matmul_no_alloc(weight, dx.ptr, q4b.F16, 1, dy.ptr)
        ctx.sync()
