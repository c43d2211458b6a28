"""Host logic of the column-parallel layer, on CPU: the row slices partition
every projection, and two gloo ranks that each compute their slice with the
oracle and gather reproduce the unsharded result bit for bit."""
import importlib
import os
import socket

import numpy as np
import pytest


def test_slices_partition_every_projection(q4b):
    layer = importlib.import_module("cpu-llms-in-c_b200.layer")
    for layer_set in (q4b.LAYER_SMALL, q4b.LAYER_27B):
        for p in layer_set:
            for world in (1, 2, 3, 4, 8):
                covered = 0
                for rank in range(world):
                    begin, count = layer.slice_of(p.n, rank, world)
                    assert begin == covered and begin % 16 == 0
                    covered += count
                assert covered == p.n
    # ragged: 100 rows over 3 ranks, 16-row granular
    assert [layer.slice_of(100, r, 3) for r in range(3)] == [(0, 48), (48, 32), (80, 20)]


def _rank_main(rank, world, port, queue):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import q4_oracle as orc
    layer = importlib.import_module("cpu-llms-in-c_b200.layer")
    n, k, m = 208, 256, 3
    quants, meta = orc.synth_weight(4, 0, n, k // 64)
    x = orc.synth_x(4, 0, m, k)
    begin, count = layer.slice_of(n, rank, world)
    mine, _ = orc.matmul(quants, meta, k // 64, x, row_begin=begin, row_count=count, want64=False)
    pieces = [None] * world
    dist.all_gather_object(pieces, (begin, mine))
    full = np.zeros((m, n), dtype=np.float32)
    for start, piece in pieces:
        full[:, start:start + piece.shape[1]] = piece
    want, _ = orc.matmul(quants, meta, k // 64, x, want64=False)
    queue.put((rank, bool((full.view(np.uint32) == want.view(np.uint32)).all())))
    dist.barrier()
    dist.destroy_process_group()


def test_two_gloo_ranks_gather_to_the_unsharded_result():
    import torch.multiprocessing as mp
    with socket.socket() as probe:
        probe.bind(("127.0.0.1", 0))
        port = probe.getsockname()[1]
    context = mp.get_context("spawn")
    queue = context.Queue()
    procs = [context.Process(target=_rank_main, args=(rank, 2, port, queue)) for rank in range(2)]
    for proc in procs:
        proc.start()
    results = [queue.get(timeout=120) for _ in procs]
    for proc in procs:
        proc.join(timeout=60)
        assert proc.exitcode == 0
    assert sorted(results) == [(0, True), (1, True)]
