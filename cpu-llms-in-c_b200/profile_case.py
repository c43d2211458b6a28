"""A small, self-ending case of one kernel, for a profiler capture.

    python cpu-llms-in-c_b200/profile_case.py gemv gate_up 1     # decode kernel, fused gate/up, M = 1
    python cpu-llms-in-c_b200/profile_case.py gemv down 4        # decode kernel, down projection, M = 4
    python cpu-llms-in-c_b200/profile_case.py gemm gate_up 2048  # tcgen05 kernel, fused gate/up, M = 2048
    python cpu-llms-in-c_b200/profile_case.py sequence 2 1       # decode sequence: 2 whole 27B layers, M = 1
    python cpu-llms-in-c_b200/profile_case.py gemm h3_fc1 2048 bf16  # tcgen05 kernel, H3 fc1, bf16 activations

The 27B shapes over a few sets of distinct weights (about 0.4 GB on the device,
more than L2, so DRAM counters mean something), two passes, a handful of
launches in all.
"""
import importlib
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

SHAPES = {"q": (5120, 6144, False), "o": (6144, 5120, False), "gate_up": (5120, 17408, True),
          "down": (17408, 5120, False),
          # MiniMax-H3 block projections (compiler/minimax-h3/apple-m3-pro/minimax_h3_q4_layer.c:15-20)
          "h3_qkv": (5376, 21504, False), "h3_fc1": (5376, 28672, False), "h3_fc2": (14336, 5376, False)}


def sequence(q4b, layers, m):
    """The whole layer set as one persistent launch per pass, three passes."""
    sharded = importlib.import_module("cpu-llms-in-c_b200.sharded")
    ctx = q4b.Q4Context(0)
    stack = sharded.ShardedLayerStack(ctx, q4b.LAYER_27B, layers, m, mode="sequence")
    for _ in range(3):
        stack.step()
    ctx.sync()
    print(f"sequence of {layers} layers, M={m}: 3 launches")
    stack.free()
    ctx.close()


def main(argv):
    q4b = importlib.import_module("cpu-llms-in-c_b200")
    kind = argv[1] if len(argv) > 1 else "gemv"
    if kind == "sequence":
        return sequence(q4b, int(argv[2]) if len(argv) > 2 else 2, int(argv[3]) if len(argv) > 3 else 1)
    which = argv[2] if len(argv) > 2 else "gate_up"
    m = int(argv[3]) if len(argv) > 3 else (1 if kind == "gemv" else 2048)
    if kind == "gemv" and m > 16 or kind == "gemm" and m <= 16:
        raise SystemExit("gemv takes M <= 16, gemm M > 16")
    k, n, fused = SHAPES[which]
    dtype = q4b.BF16 if len(argv) > 4 and argv[4] == "bf16" else q4b.F16
    if dtype == q4b.BF16 and kind != "gemm":
        raise SystemExit("bf16 activations run on the tcgen05 kernel: use gemm")
    sets = max(2, int(0.4e9 // (k * n * (1.0 if fused else 0.5) * 1.125)))
    ctx = q4b.Q4Context(0)
    weights = [(ctx.synth_weight(index, 0, n, k // 64), ctx.synth_weight(index, 1, n, k // 64) if fused else None)
               for index in range(sets)]
    x = ctx.synth_x(0, 0, m, k)
    y = ctx.alloc(m * n * 2)
    for _ in range(2):
        for gate, up in weights:
            if fused:
                ctx.gate_up_silu(gate, up, x.ptr, dtype, m, y.ptr, dtype)
            else:
                ctx.matmul(gate, x.ptr, dtype, m, y.ptr, dtype)
    ctx.sync()
    print(f"{kind} {which} M={m}: {2 * sets} launches over {sets} weight sets")
    ctx.close()


if __name__ == "__main__":
    main(sys.argv)
