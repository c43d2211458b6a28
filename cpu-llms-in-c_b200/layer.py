"""One decoder layer's set of Q4 projections, column-parallel over the ranks.

The reference dispatches a layer as a fixed sequence of Q4 matmuls
(encode_attention / encode_delta / encode_mlp, qwen38_m3_decode.m:639-805):
fused q/k/v in-projection, out-projection, fused gate/up with SiLU, down.  Here
every projection's output rows are split into `world` contiguous slices (the
tile stream is per-row, so a slice is a contiguous range of both image planes);
each rank computes its slice from the full x and an all-gather reassembles
[M, N].  With world == 1 the gather disappears.

Inputs follow the benchmark configurations: every projection reads its own
seeded x ~ N(0,1) of its K (stream 0 for K = hidden, derived streams otherwise),
so projections of a layer are independent and individually checkable.
"""
from __future__ import annotations

from .host import F16, Q4Context, Q4Weight
from .shapes import Projection


def slice_of(n: int, rank: int, world: int) -> tuple[int, int]:
    """Contiguous row slice [begin, begin+count) of rank; 16-row granular."""
    tiles = (n + 15) // 16
    per, extra = divmod(tiles, world)
    begin_tile = rank * per + min(rank, extra)
    count_tile = per + (1 if rank < extra else 0)
    begin = min(begin_tile * 16, n)
    end = min((begin_tile + count_tile) * 16, n)
    return begin, end - begin


class Q4Layer:
    """Weights of one layer on one rank plus the launch sequence."""

    def __init__(self, ctx: Q4Context, layer, seed: int, rank: int = 0, world: int = 1):
        self.ctx, self.layer, self.seed, self.rank, self.world = ctx, tuple(layer), seed, rank, world
        self.weights: dict[str, tuple[Q4Weight, ...]] = {}
        self.slices: dict[str, tuple[int, int]] = {}
        index = 0
        for p in self.layer:
            begin, count = slice_of(p.n, rank, world)
            self.slices[p.name] = (begin, count)
            members = []
            for _ in range(2 if p.fused else 1):
                members.append(ctx.synth_weight(seed, index, p.n, p.k // 64, begin, count))
                index += 1
            self.weights[p.name] = tuple(members)

    def launch_plan(self):
        """[(kind, projections)] in launch order: grouped, fused or single."""
        plan, seen = [], set()
        for p in self.layer:
            if p.name in seen:
                continue
            if p.group:
                members = [q for q in self.layer if q.group == p.group]
                seen.update(q.name for q in members)
                plan.append(("group", members))
            elif p.fused:
                plan.append(("fused", [p]))
            else:
                plan.append(("single", [p]))
            seen.add(p.name)
        return plan

    def forward(self, x_ptrs: dict[int, int], y_ptrs: dict[str, int], m_rows: int, ldy: dict[str, int] | None = None):
        """Queue the layer's launches.  x_ptrs maps K -> device x [M, K] fp16;
        y_ptrs maps projection name -> device output (this rank's slice start);
        ldy gives each output's row stride (default: the slice width)."""
        ctx = self.ctx
        for kind, members in self.launch_plan():
            first = members[0]
            x = x_ptrs[first.k]
            stride = lambda p: (ldy[p.name] if ldy else self.slices[p.name][1])
            if kind == "group":
                ctx.matmul_group([self.weights[p.name][0] for p in members], x, F16, m_rows,
                                 [y_ptrs[p.name] for p in members], F16, [stride(p) for p in members])
            elif kind == "fused":
                gate, up = self.weights[first.name]
                ctx.gate_up_silu(gate, up, x, F16, m_rows, y_ptrs[first.name], F16, stride(first))
            else:
                ctx.matmul(self.weights[first.name][0], x, F16, m_rows, y_ptrs[first.name], F16, stride(first))

    def add_to(self, sequence, x_ptrs: dict[int, int], y_ptrs: dict[str, int], ldy: dict[str, int] | None = None):
        """Append the layer's projections to a decode sequence, in launch order.
        Returns [(job index, [projection per segment])]."""
        jobs = []
        for kind, members in self.launch_plan():
            first = members[0]
            stride = lambda p: (ldy[p.name] if ldy else self.slices[p.name][1])
            if kind == "fused":
                gate, up = self.weights[first.name]
                job = sequence.add_gate_up(gate, up, x_ptrs[first.k], y_ptrs[first.name], stride(first))
            else:
                job = sequence.add_matmul([self.weights[p.name][0] for p in members], x_ptrs[first.k],
                                          [y_ptrs[p.name] for p in members], [stride(p) for p in members])
            jobs.append((job, members))
        return jobs

    def launches_per_forward(self) -> int:
        return len(self.launch_plan())

    def free(self):
        for members in self.weights.values():
            for weight in members:
                weight.free()
        self.weights = {}
