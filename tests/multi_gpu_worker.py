"""One rank of the column-parallel parity check (launched by torch.distributed.run).

Every rank holds its N-slice of every projection, runs the small layer stack
twice and must end with the WHOLE [M, N] of every projection equal to the
oracle's: through the persistent launch that pushes, through per-projection launches that push
with a barrier between the ranks, and through the NCCL baseline."""
import importlib
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))


def main():
    import torch
    import torch.distributed as dist
    from q4_cases import assert_close
    from test_gpu_layer import oracle_layer
    from oracle import q4_oracle as orc
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    q4b = importlib.import_module("cpu-llms-in-c_b200")
    sharded = importlib.import_module("cpu-llms-in-c_b200.sharded")
    layer_set = q4b.LAYER_SMALL if len(sys.argv) < 2 or sys.argv[1] == "small" else q4b.LAYER_27B
    layers = 3 if layer_set is q4b.LAYER_SMALL else 1
    ctx = q4b.Q4Context(local)
    # M = 64 and 300 take the tensor-core GEMM on every rank's slice
    sizes = (1, 4, 64, 300) if layer_set is q4b.LAYER_SMALL else (1, 4)
    # the ranks share outputs through one persistent launch whose epilogue stores into every rank's copy, through
    # one launch per projection that does the same with a barrier between the ranks after it (recorded into a
    # graph), or through NCCL all-gathers
    for gather, mode in (("push", "sequence"), ("push", "graph"), ("nccl", "graph")):
        for m in sizes:
            if mode == "sequence" and m > 16:
                continue
            stack = sharded.ShardedLayerStack(ctx, layer_set, layers, m, rank, world, dist, gather=gather, mode=mode)
            assert stack.gather == gather and (stack.mode == mode or m > 16)
            for _ in range(3):
                stack.step()
            ctx.sync()
            torch.cuda.synchronize()
            dist.barrier()
            for index in range(layers):
                got = stack.outputs(index)
                want = oracle_layer(orc, layer_set, index, m)
                for name in want:
                    assert_close(got[name], want[name], f"rank {rank} {gather} {mode} layer {index} {name} M={m}")
            dist.barrier()
            stack.free()
    # large M with the slice pushed by the copy kernel after the GEMM (the default from three ranks on)
    for m in ((64, 300) if layer_set is q4b.LAYER_SMALL else ()):
        stack = sharded.ShardedLayerStack(ctx, layer_set, layers, m, rank, world, dist, gather="push",
                                          push_in_epilogue=False)
        for _ in range(3):
            stack.step()
        ctx.sync()
        torch.cuda.synchronize()
        dist.barrier()
        for index in range(layers):
            got = stack.outputs(index)
            want = oracle_layer(orc, layer_set, index, m)
            for name in want:
                assert_close(got[name], want[name], f"rank {rank} copy-kernel push layer {index} {name} M={m}")
        dist.barrier()
        stack.free()
    # the publish-and-wait exchange between ranks 0 and 1 answers within its bounded waits
    if layer_set is q4b.LAYER_SMALL:
        words = ctx.to_device(np.zeros(1024, dtype=np.uint32))
        handles = [None] * world
        dist.all_gather_object(handles, ctx.ipc_export(words.ptr))
        peer = ctx.ipc_open(handles[1 - rank]) if rank < 2 else None
        ctx.sync()
        dist.barrier()
        if rank < 2:
            round_trip_us = ctx.probe_signal(words.ptr, peer, 1024, 200, 0, rank == 0)
            assert 0.5 < round_trip_us < 200.0, round_trip_us
        dist.barrier()
        if rank < 2:
            ctx.ipc_close(peer)
    ctx.close()
    dist.barrier()
    dist.destroy_process_group()
    if rank == 0:
        print("multi-gpu parity ok", world, "ranks")


if __name__ == "__main__":
    main()
