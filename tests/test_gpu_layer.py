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
