"""The layer launch sequence (grouped q/k/v, o, fused gate/up, down) and its
recorded replay, against the oracle, on one GPU."""
import importlib

import numpy as np
import pytest

from q4_cases import assert_close

pytestmark = pytest.mark.gpu


def oracle_layer(orc, layer_set, seed, m):
    out, index = {}, 0
    for p in layer_set:
        groups = p.k // 64
        x = orc.synth_x(seed, 0, m, p.k)
        if p.fused:
            gq, gm = orc.synth_weight(seed, index, p.n, groups)
            uq, um = orc.synth_weight(seed, index + 1, p.n, groups)
            out[p.name] = orc.gate_up_silu(gq, gm, uq, um, groups, x, want32=False)[1]
            index += 2
        else:
            q, mt = orc.synth_weight(seed, index, p.n, groups)
            out[p.name] = orc.matmul(q, mt, groups, x, want32=False)[1]
            index += 1
    return out


@pytest.mark.parametrize("mode", ["sequence", "graph"])
@pytest.mark.parametrize("m", [1, 4, 9])
def test_small_layer_stack_matches_oracle(q4b, orc, m, mode):
    sharded = importlib.import_module("cpu-llms-in-c_b200.sharded")
    with q4b.Q4Context(0) as ctx:
        stack = sharded.ShardedLayerStack(ctx, q4b.LAYER_SMALL, 3, m, mode=mode)
        before = ctx.launches
        stack.step()   # graph mode: plain launches + recording
        stack.step()   # graph mode: replay; sequence mode: second launch of the same sequence
        ctx.sync()
        assert ctx.launches - before >= (2 if mode == "sequence" else 3 * 4 * 2)
        for index in (0, 2):
            got = stack.outputs(index)
            want = oracle_layer(orc, q4b.LAYER_SMALL, index, m)
            for name in want:
                assert_close(got[name], want[name], f"layer {index} {name} M={m}")
        stack.step_from_host()
        got = stack.outputs(1)
        want = oracle_layer(orc, q4b.LAYER_SMALL, 1, m)
        for name in want:
            assert_close(got[name], want[name], f"host path {name}")
        stack.free()


@pytest.mark.parametrize("mode", ["sequence", "graph"])
def test_27b_layer_matches_oracle_at_decode(q4b, orc, mode):
    sharded = importlib.import_module("cpu-llms-in-c_b200.sharded")
    with q4b.Q4Context(0) as ctx:
        stack = sharded.ShardedLayerStack(ctx, q4b.LAYER_27B, 1, 1, mode=mode)
        stack.step()
        got = stack.outputs(0)
        want = oracle_layer(orc, q4b.LAYER_27B, 0, 1)
        for name in want:
            assert_close(got[name], want[name], f"27B {name}")
        stack.free()


def rank_slice_set(q4b, world):
    """The projections one of `world` column-parallel ranks works on: 1/world of every N, the whole of every K."""
    projection = importlib.import_module("cpu-llms-in-c_b200.shapes").Projection
    return tuple(projection(p.name, p.k, p.n // world, p.fused, p.group) for p in q4b.LAYER_27B)


@pytest.mark.parametrize("world", [4, 8])
@pytest.mark.parametrize("m,mode", [(1, "sequence"), (4, "sequence"), (1, "graph"), (512, "graph")])
def test_shapes_of_one_rank_among_many(q4b, orc, world, m, mode):
    """One GPU stands in for a single rank of a 4- or 8-rank job: same shapes, same kernels and work split
    (few row blocks, long K), checked on sampled weight rows."""
    sharded = importlib.import_module("cpu-llms-in-c_b200.sharded")
    layer_set = rank_slice_set(q4b, world)
    with q4b.Q4Context(0) as ctx:
        stack = sharded.ShardedLayerStack(ctx, layer_set, 2, m, mode=mode)
        stack.step()
        stack.step()
        got = stack.outputs(1)
        seed, index = 1, 0
        for p in layer_set:
            groups = p.k // 64
            x = orc.synth_x(seed, 0, m, p.k)
            rows = sorted({0, 1, p.n // 2, p.n - 65, p.n - 1})
            for row in rows:
                if p.fused:
                    gq, gm = orc.synth_weight_rows(seed, index, groups, [row])
                    uq, um = orc.synth_weight_rows(seed, index + 1, groups, [row])
                    want = orc.gate_up_silu(gq, gm, uq, um, groups, x, want32=False)[1]
                else:
                    q, mt = orc.synth_weight_rows(seed, index, groups, [row])
                    want = orc.matmul(q, mt, groups, x, want32=False)[1]
                # sampled rows, so max|ref| is taken from the device's whole output of this projection
                scale = float(np.max(np.abs(got[p.name].astype(np.float32))))
                assert np.max(np.abs(got[p.name][:, row:row + 1] - want)) / scale <= 2e-3, (p.name, row, m, mode)
            index += 2 if p.fused else 1
        stack.free()


def test_push_rows_and_pushing_decode_launch_on_one_device(q4b, orc):
    """The two ways a rank's slice reaches the other ranks' copies, with the "peers" played by further buffers
    of the same GPU: the decode kernel's epilogue storing into them (q4b_context_push_outputs, M <= 16) and the
    copy kernel (q4b_push_rows); the bytes between the slices stay as they were."""
    with q4b.Q4Context(0) as ctx:
        n_total, n_local, begin, k, m = 1024, 256, 384, 2048, 3
        groups = k // 64
        quants, meta = orc.synth_weight(5, 0, n_local, groups)
        weight = ctx.upload(quants, meta, n_local, groups)
        x = orc.synth_x(5, 0, m, k)
        dx = ctx.to_device(x)
        _, ref = orc.matmul(quants, meta, groups, x, want32=False)
        fill = np.full((m, n_total), 7.0, dtype=np.float16)
        own, peer_a, peer_b = (ctx.to_device(fill) for _ in range(3))
        offset = begin * 2
        ctx.push_outputs(3, [[None, peer_a.ptr + offset, peer_b.ptr + offset]])
        ctx.matmul(weight, dx.ptr, q4b.F16, m, own.ptr + offset, q4b.F16, n_total)
        ctx.sync()
        for buffer in (own, peer_a, peer_b):
            got = buffer.download(np.float16, (m, n_total))
            assert_close(got[:, begin:begin + n_local], ref, "pushed by the epilogue")
            assert (got[:, :begin] == 7.0).all() and (got[:, begin + n_local:] == 7.0).all()
        # the copy kernel: the own block into two fresh "peers"
        peer_c, peer_d = (ctx.to_device(fill) for _ in range(2))
        ctx.push_rows(own.ptr + offset, [peer_c.ptr + offset, peer_d.ptr + offset], m, n_local * 2, n_total * 2)
        ctx.sync()
        want = own.download(np.float16, (m, n_total))
        for buffer in (peer_c, peer_d):
            got = buffer.download(np.float16, (m, n_total))
            assert (got.view(np.uint16) == want.view(np.uint16)).all()
        with pytest.raises(q4b.Q4Error):
            ctx.push_rows(own.ptr + offset, [peer_c.ptr + offset], m, n_local * 2 + 2, n_total * 2)
        weight.free()


def test_recorded_barrier_counts_on_at_every_replay(q4b, orc):
    """A barrier's round lives in device memory: recorded into a graph between two launches it passes at every
    replay (a one-rank barrier meets itself), and a barrier queued afterwards outside the graph still agrees with
    the count."""
    with q4b.Q4Context(0) as ctx:
        n, k, m = 512, 1024, 2
        quants, meta = orc.synth_weight(9, 0, n, k // 64)
        weight = ctx.upload(quants, meta, n, k // 64)
        x = orc.synth_x(9, 0, m, k)
        dx = ctx.to_device(x)
        dy = ctx.alloc(m * n * 2)
        barrier = q4b.Q4Barrier(ctx, 1, 0)
        ctx.matmul(weight, dx.ptr, q4b.F16, m, dy.ptr)  # once outside: attributes and scratch
        barrier.queue()
        ctx.sync()
        ctx.graph_begin()
        for _ in range(3):
            ctx.matmul(weight, dx.ptr, q4b.F16, m, dy.ptr)
            barrier.queue()
        graph = ctx.graph_end()
        for _ in range(4):
            graph.launch()
        barrier.queue()
        ctx.sync()  # a barrier that lost count would run into its bounded wait: status 2 here
        _, ref = orc.matmul(quants, meta, k // 64, x, want32=False)
        assert_close(dy.download(np.float16, (m, n)), ref, "after the replays")
        graph.free()
        barrier.free()
        weight.free()
