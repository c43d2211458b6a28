"""A stack of Q4 layers on one rank of a column-parallel job.

Every projection of every layer is split by output rows over `world` ranks;
each rank owns its slice's tile stream, computes Y[:, n0:n1] from the full x and
the slices are gathered so that every rank ends with the whole [M, N].

Two gather paths:
  * "push"  : every epilogue stores its slice straight into every rank's copy of
              y over NVLink -- no collective call per projection.  M <= 16: the
              whole pass is one decode sequence (q4b_decode.cu) and a job starts
              only when all ranks have published the previous one; M > 16: the
              tensor-core GEMM pushes (q4b_context_push_outputs) and a one-thread
              barrier kernel follows every projection group (q4b_barrier_queue);
  * "nccl"  : q4b_all_gather_columns (ncclAllGather + interleave) per gather
              point, queued on the context's stream (the baseline and the
              cross-check).
With world == 1 neither runs.  The caller's process group (world > 1) only
carries handles and the communicator's id between the ranks.
"""
from __future__ import annotations

import ctypes

import numpy as np

from .host import F16, Q4Barrier, Q4Comm, Q4Context, Q4Sequence, library
from .layer import Q4Layer, slice_of


# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the decode kernel on the 27B gate/up pair at M = 1
NCU_GATE_UP_TRAFFIC_BYTES = 103.8e6


class ShardedLayerStack:
    def __init__(self, ctx: Q4Context, layer_set, n_layers: int, m_rows: int, rank: int = 0, world: int = 1,
                 dist=None, gather: str = "push", mode: str = "graph", layers=None, push_in_epilogue=None):
        self.ctx, self.layer_set, self.n_layers, self.m = ctx, tuple(layer_set), n_layers, m_rows
        self.rank, self.world, self.dist, self.gather = rank, world, dist, gather
        # weights do not depend on M: a second stack (another M) may share the first one's layers
        self.owns_layers = layers is None
        self.layers = layers if layers is not None else [Q4Layer(ctx, layer_set, seed, rank, world)
                                                         for seed in range(n_layers)]
        self.ks = sorted({p.k for p in self.layer_set})
        self.graph = None
        self.sequence = None
        # large M, ranks that push: from the GEMM's epilogue, or by a copy kernel after it (None: by rank count)
        self.push_in_epilogue = push_in_epilogue
        # "sequence": the whole pass is one persistent launch (M <= 16); "graph": one launch per projection
        # group, replayed from a recorded graph
        self.mode = mode if m_rows <= 16 else "graph"

        # activations: per layer, one [M, K] fp16 block per distinct K
        self.x_offsets, offset = {}, 0
        for k in self.ks:
            self.x_offsets[k] = offset
            offset += m_rows * k * 2
        self.x_layer_bytes = offset
        self.x_all = ctx.alloc(self.x_layer_bytes * n_layers)
        lib = library()
        for index in range(n_layers):
            for k in self.ks:
                pointer = self.x_all.ptr + index * self.x_layer_bytes + self.x_offsets[k]
                ctx._check(lib.q4b_synth_x(ctx.handle, index, 0, pointer, 0, m_rows * k, ctx._err, 512))
        # outputs: per layer, the full [M, N] of every projection
        self.y_offsets, offset = {}, 0
        for p in self.layer_set:
            self.y_offsets[p.name] = offset
            offset += m_rows * p.n * 2
        self.y_layer_bytes = offset
        self.h2d_bytes_per_step = self.x_layer_bytes * n_layers
        self.d2h_bytes_per_step = self.y_layer_bytes * n_layers
        self.comm = None
        self.barrier = None
        if world > 1 and gather == "push" and m_rows <= 16 and self.mode == "sequence":
            self._setup_push()
        elif world > 1 and gather == "push":
            # one launch per projection group, each storing into every rank's y, and a barrier between the ranks
            # after it; the whole pass is recorded into a graph
            self._setup_push_gemm()
        elif world > 1:
            self.gather = "nccl"
            # the process group only carries the communicator's id; the gathers themselves are q4b_all_gather*
            def exchange(payload: bytes):
                everyone = [None] * world
                dist.all_gather_object(everyone, payload)
                return everyone
            self.comm = Q4Comm(ctx, world, rank, exchange)
            self.y_all = ctx.alloc(self.y_layer_bytes * n_layers)
            self.y_base = self.y_all.ptr
            # this rank's slices, one contiguous block per layer: [projection][M][n_local]
            self.local_offsets, offset = {}, 0
            for p in self.layer_set:
                self.local_offsets[p.name] = offset
                offset += m_rows * slice_of(p.n, rank, world)[1] * 2
            self.local_layer_bytes = offset
            self.local_all = ctx.alloc(offset * n_layers)
            self.local_base = self.local_all.ptr
            self.staging = ctx.alloc(max(m_rows * p.n for p in self.layer_set) * 2)
        else:
            self.y_all = ctx.alloc(self.y_layer_bytes * n_layers)
            self.y_base = self.y_all.ptr
        # pinned host mirrors for the end-to-end measurement
        self.x_host = self._pinned(self.x_layer_bytes * n_layers)
        self.y_host = self._pinned(self.y_layer_bytes * n_layers)
        ctx._check(lib.q4b_copy_to_host(ctx.handle, self.x_host, self.x_all.ptr, self.x_layer_bytes * n_layers,
                                        ctx._err, 512))
        ctx.sync()

    def _setup_push(self):
        """Full y on every rank, shared through IPC handles; one sequence with peer outputs."""
        ctx, dist = self.ctx, self.dist
        self.y_all = ctx.alloc(self.y_layer_bytes * self.n_layers)
        self.y_base = self.y_all.ptr
        handles = [None] * self.world
        dist.all_gather_object(handles, ctx.ipc_export(self.y_all.ptr))
        self.peer_y = [self.y_base if r == self.rank else ctx.ipc_open(handles[r]) for r in range(self.world)]
        sequence = Q4Sequence(ctx, self.m, self.world, self.rank)
        for index, layer in enumerate(self.layers):
            offsets = {p.name: index * self.y_layer_bytes + self.y_offsets[p.name] + layer.slices[p.name][0] * 2
                       for p in self.layer_set}
            jobs = layer.add_to(sequence, self._x_ptrs(index), {n: self.y_base + o for n, o in offsets.items()},
                                {p.name: p.n for p in self.layer_set})
            for job, members in jobs:
                sequence.set_job_blocks(job, sum(-(-slice_of(p.n, r, self.world)[1] // 64)
                                                 for p in members for r in range(self.world)))
                for segment, p in enumerate(members):
                    for r in range(self.world):
                        if r != self.rank:
                            sequence.set_peer_output(job, segment, r, self.peer_y[r] + offsets[p.name])
        sequence.finalize()
        counters = [None] * self.world
        dist.all_gather_object(counters, ctx.ipc_export(sequence.done_counters))
        self.peer_counters = []
        for r in range(self.world):
            if r != self.rank:
                pointer = ctx.ipc_open(counters[r])
                self.peer_counters.append(pointer)
                sequence.set_peer_counters(r, pointer)
        self.sequence = sequence
        self.mode = "sequence"
        ctx.sync()
        dist.barrier()  # every rank's counters are zero and mapped before anyone launches

    def _setup_push_gemm(self):
        """Full y on every rank, shared through IPC handles; a barrier between the ranks."""
        ctx, dist = self.ctx, self.dist
        self.y_all = ctx.alloc(self.y_layer_bytes * self.n_layers)
        self.y_base = self.y_all.ptr
        handles = [None] * self.world
        dist.all_gather_object(handles, ctx.ipc_export(self.y_all.ptr))
        self.peer_y = [self.y_base if r == self.rank else ctx.ipc_open(handles[r]) for r in range(self.world)]
        self.barrier = Q4Barrier(ctx, self.world, self.rank)
        counters = [None] * self.world
        dist.all_gather_object(counters, ctx.ipc_export(self.barrier.counter))
        self.peer_counters = []
        for r in range(self.world):
            if r != self.rank:
                pointer = ctx.ipc_open(counters[r])
                self.peer_counters.append(pointer)
                self.barrier.set_peer(r, pointer)
        ctx.sync()
        dist.barrier()

    def _queue_sharded_push_gemm(self):
        """Every projection group: GEMM on this rank's slices, stored into all ranks' y; then the barrier."""
        ctx = self.ctx
        for index, layer in enumerate(self.layers):
            x_ptrs = self._x_ptrs(index)
            for kind, members in layer.launch_plan():
                offsets = [index * self.y_layer_bytes + self.y_offsets[p.name] + layer.slices[p.name][0] * 2
                           for p in members]
                # small M: the kernel's epilogue stores into the peers; large M: a copy kernel after the GEMM
                # (wide requests on every link at once; the epilogue's 32-byte stores between tiles are far slower)
                in_epilogue = self.m <= 16 or (self.push_in_epilogue if self.push_in_epilogue is not None
                                               else self.world <= 2)
                if in_epilogue:
                    ctx.push_outputs(self.world, [[None if r == self.rank else self.peer_y[r] + offset
                                                   for r in range(self.world)] for offset in offsets])
                x = x_ptrs[members[0].k]
                if kind == "group":
                    ctx.matmul_group([layer.weights[p.name][0] for p in members], x, F16, self.m,
                                     [self.y_base + o for o in offsets], F16, [p.n for p in members])
                elif kind == "fused":
                    gate, up = layer.weights[members[0].name]
                    ctx.gate_up_silu(gate, up, x, F16, self.m, self.y_base + offsets[0], F16, members[0].n)
                else:
                    ctx.matmul(layer.weights[members[0].name][0], x, F16, self.m, self.y_base + offsets[0], F16,
                               members[0].n)
                if not in_epilogue:
                    for p, offset in zip(members, offsets):
                        ctx.push_rows(self.y_base + offset, [self.peer_y[r] + offset for r in range(self.world)
                                                            if r != self.rank],
                                      self.m, layer.slices[p.name][1] * 2, p.n * 2)
                self.barrier.queue()

    def _pinned(self, nbytes: int) -> int:
        pointer = ctypes.c_void_p()
        self.ctx._check(library().q4b_alloc_host(self.ctx.handle, nbytes, ctypes.byref(pointer), self.ctx._err, 512))
        return pointer.value

    # ------------------------------------------------------------------
    def _x_ptrs(self, index: int):
        base = self.x_all.ptr + index * self.x_layer_bytes
        return {k: base + self.x_offsets[k] for k in self.ks}

    def _queue_single_gpu(self):
        for index, layer in enumerate(self.layers):
            base = self.y_base + index * self.y_layer_bytes
            layer.forward(self._x_ptrs(index), {p.name: base + self.y_offsets[p.name] for p in self.layer_set}, self.m)

    def _queue_sharded_nccl(self):
        for index, layer in enumerate(self.layers):
            local = self.local_base + index * self.local_layer_bytes
            layer.forward(self._x_ptrs(index), {p.name: local + self.local_offsets[p.name] for p in self.layer_set},
                          self.m)
            for p in self.layer_set:
                n_local = slice_of(p.n, self.rank, self.world)[1]
                piece = local + self.local_offsets[p.name]
                full = self.y_base + index * self.y_layer_bytes + self.y_offsets[p.name]
                self.comm.all_gather_columns(piece, full, self.m, n_local, 2, self.staging.ptr)

    def step(self):
        """One pass over all layers, queued on the context stream."""
        if self.world > 1 and self.gather == "nccl":
            self._queue_sharded_nccl()
            return
        if self.barrier is not None:
            if self.graph is None:
                self._queue_sharded_push_gemm()  # plain launches once (sets kernel attributes, allocates scratch)
                self.ctx.sync()
                self.ctx.graph_begin()
                self._queue_sharded_push_gemm()
                self.graph = self.ctx.graph_end()
            self.graph.launch()
            return
        if self.mode == "sequence":
            if self.sequence is None:
                self.sequence = Q4Sequence(self.ctx, self.m)
                for index, layer in enumerate(self.layers):
                    base = self.y_base + index * self.y_layer_bytes
                    layer.add_to(self.sequence, self._x_ptrs(index),
                                 {p.name: base + self.y_offsets[p.name] for p in self.layer_set},
                                 {p.name: p.n for p in self.layer_set})
                self.sequence.finalize()
            self.sequence.launch()
            return
        if self.graph is None:
            self._queue_single_gpu()  # plain launches once (also sets kernel attributes)
            self.ctx.sync()
            self.ctx.graph_begin()
            self._queue_single_gpu()
            self.graph = self.ctx.graph_end()
        self.graph.launch()

    def step_from_host(self):
        """The same pass with x starting in pinned host memory and every output
        copied back to pinned host memory."""
        lib, ctx = library(), self.ctx
        ctx._check(lib.q4b_copy_to_device(ctx.handle, self.x_all.ptr, self.x_host, self.h2d_bytes_per_step,
                                          ctx._err, 512))
        self.step()
        ctx._check(lib.q4b_copy_to_host(ctx.handle, self.y_host, self.y_base, self.d2h_bytes_per_step,
                                        ctx._err, 512))
        ctx.sync()

    def dominant_kernel_pass(self):
        """The fused gate/up kernel alone, once per layer (distinct weights)."""
        self.projection_pass(next(p.name for p in self.layer_set if p.fused))

    def projection_pass(self, name: str):
        """One launch group of the layer alone (the group's first member names it), once per layer: this rank's
        slice, outputs where the whole pass puts them, no gather."""
        for index, layer in enumerate(self.layers):
            kind, members = next((k, ms) for k, ms in layer.launch_plan() if ms[0].name == name)
            outs = []
            for p in members:
                if self.world > 1 and self.gather == "nccl":
                    outs.append(self.local_base + index * self.local_layer_bytes + self.local_offsets[p.name])
                else:
                    outs.append(self.y_base + index * self.y_layer_bytes + self.y_offsets[p.name] +
                                layer.slices[p.name][0] * 2)
            wide = self.world > 1 and self.gather != "nccl"
            strides = [p.n if wide else layer.slices[p.name][1] for p in members]
            x = self._x_ptrs(index)[members[0].k]
            if kind == "group":
                self.ctx.matmul_group([layer.weights[p.name][0] for p in members], x, F16, self.m, outs, F16, strides)
            elif kind == "fused":
                gate, up = layer.weights[name]
                self.ctx.gate_up_silu(gate, up, x, F16, self.m, outs[0], F16, strides[0])
            else:
                self.ctx.matmul(layer.weights[name][0], x, F16, self.m, outs[0], F16, strides[0])

    def outputs(self, index: int) -> dict[str, np.ndarray]:
        """Host copies of layer `index`'s gathered outputs, for checks."""
        self.ctx.sync()
        result = {}
        for p in self.layer_set:
            out = np.empty((self.m, p.n), dtype=np.float16)
            pointer = self.y_base + index * self.y_layer_bytes + self.y_offsets[p.name]
            self.ctx._check(library().q4b_copy_to_host(self.ctx.handle, out.ctypes.data, pointer, out.nbytes,
                                                       self.ctx._err, 512))
            self.ctx.sync()
            result[p.name] = out
        return result

    def ncu_traffic_bytes(self):
        """DRAM bytes (read + written) per launch of the dominant kernel (fused gate/up, 5120 -> 17408, M = 1),
        from the profiler capture summarised under profiles/; a rank's slice moves 1/world of the weight
        stream.  None where no capture exists (other shapes, other M)."""
        fused = next(p for p in self.layer_set if p.fused)
        if (fused.k, fused.n) != (5120, 17408) or self.m != 1 or NCU_GATE_UP_TRAFFIC_BYTES is None:
            return None
        return NCU_GATE_UP_TRAFFIC_BYTES / self.world

    def free(self):
        if self.world > 1 and self.gather == "push":
            self.ctx.sync()
            self.dist.barrier()  # nobody stores into a peer that is about to unmap
            for pointer in [p for r, p in enumerate(self.peer_y) if r != self.rank] + self.peer_counters:
                self.ctx.ipc_close(pointer)
            if self.barrier is not None:
                self.barrier.free()
        if self.comm is not None:
            self.comm.free()
        if self.owns_layers:
            for layer in self.layers:
                layer.free()
        if self.graph is not None:
            self.graph.free()
        if self.sequence is not None:
            self.sequence.free()
        library().q4b_free_host(self.ctx.handle, self.x_host)
        library().q4b_free_host(self.ctx.handle, self.y_host)
