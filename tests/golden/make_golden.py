"""Generate tests/golden/ref_pins.json from the reference's own packer code.

Run in a container that has the reference tree (it builds oracle/_ref from the
reference sources first):

    python tests/golden/make_golden.py

Every input is regenerated from a seed by the counter-based generator in
oracle/q4_oracle.c, so the fixture stores only seeds, shapes and the outputs
that the reference code produced (as IEEE-754 bit patterns).
"""
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import q4_oracle as orc  # noqa: E402

HIDDEN, MLP = 5120, 17408


bf16_exact_meta = orc.bf16_exact_meta


def bits32(values):
    return [int(v) for v in np.asarray(values, dtype=np.float32).view(np.uint32)]


def main():
    ref = orc.ref() if orc.build_ref() else None
    if ref is None:
        raise SystemExit("oracle/_ref could not be built (reference tree absent)")
    out = {"generator": "tests/golden/make_golden.py",
           "source": "compiler/qwen3.8-27b/apple-m3-pro/qwen38_m3_pack.c "
                     "(static functions, via oracle/ref_shim.c)"}

    # 1. scalar conversions on a fixed probe set
    rng = np.random.default_rng(1234)
    probe = rng.integers(0, 2**32, size=4096, dtype=np.uint64).astype(np.uint32)
    probe = probe[np.isfinite(probe.view(np.float32))]
    small = (rng.standard_normal(2048) * 1e-4).astype(np.float32).view(np.uint32)
    probe = np.concatenate([probe, small])
    out["float_to_half"] = {
        "inputs_f32_bits": [int(v) for v in probe],
        "outputs_f16_bits": [int(ref.ref_float_to_half_bits(float(v)))
                             for v in probe.view(np.float32)]}
    bf = np.arange(0, 65536, 37, dtype=np.uint32).astype(np.uint16)
    bf = bf[np.isfinite((bf.astype(np.uint32) << 16).view(np.float32))]
    out["bf16_to_half"] = {
        "inputs_bf16_bits": [int(v) for v in bf],
        "outputs_f16_bits": [int(ref.ref_bf16_to_half(int(v))) for v in bf]}

    # 2. fused gate/up + SiLU, first 8 rows, hidden 5120, sin/cos activation
    cases = []
    for seed in (0, 1, 7):
        gq, _ = orc.synth_weight(seed, 0, 8, HIDDEN // 64)
        uq, _ = orc.synth_weight(seed, 1, 8, HIDDEN // 64)
        _, gs, gb = bf16_exact_meta(seed, 0, 8, HIDDEN // 64)
        _, us, ub = bf16_exact_meta(seed, 1, 8, HIDDEN // 64)
        result = np.zeros(8, dtype=np.float32)
        status = ref.ref_gate_up_first8(
            gq.ctypes.data_as(orc._u8p), gs.ctypes.data_as(orc._u16p),
            gb.ctypes.data_as(orc._u16p), uq.ctypes.data_as(orc._u8p),
            us.ctypes.data_as(orc._u16p), ub.ctypes.data_as(orc._u16p),
            result.ctypes.data_as(orc._f32p))
        assert status == 0
        cases.append({"seed": seed, "first8_f32_bits": bits32(result)})
    out["gate_up_silu_first8"] = {"hidden": HIDDEN, "rows": 8, "cases": cases}

    # 3. whole MLP (gate/up 17408x5120, down first 8 rows of 5120x17408) + residual
    seed = 3
    gq, _ = orc.synth_weight(seed, 0, MLP, HIDDEN // 64)
    uq, _ = orc.synth_weight(seed, 1, MLP, HIDDEN // 64)
    dq, _ = orc.synth_weight(seed, 2, 8, MLP // 64)
    _, gs, gb = bf16_exact_meta(seed, 0, MLP, HIDDEN // 64)
    _, us, ub = bf16_exact_meta(seed, 1, MLP, HIDDEN // 64)
    _, ds, db = bf16_exact_meta(seed, 2, 8, MLP // 64)
    result = np.zeros(8, dtype=np.float32)
    status = ref.ref_mlp_first8(
        gq.ctypes.data_as(orc._u8p), gs.ctypes.data_as(orc._u16p),
        gb.ctypes.data_as(orc._u16p), uq.ctypes.data_as(orc._u8p),
        us.ctypes.data_as(orc._u16p), ub.ctypes.data_as(orc._u16p),
        dq.ctypes.data_as(orc._u8p), ds.ctypes.data_as(orc._u16p),
        db.ctypes.data_as(orc._u16p), result.ctypes.data_as(orc._f32p))
    assert status == 0
    out["mlp_first8"] = {"seed": seed, "hidden": HIDDEN, "mlp": MLP,
                         "first8_f32_bits": bits32(result)}

    # 4. metadata transform BF16 planes -> interleaved fp16 records (general bf16)
    count = 4096
    sc = rng.integers(0x3800, 0x3C00, size=count, dtype=np.uint16)   # ~[3e-5, 8e-3]
    bi = (rng.integers(0x3800, 0x3E00, size=count, dtype=np.uint16) | 0x8000).astype(np.uint16)
    inter = np.zeros(count * 2, dtype=np.uint16)
    status = ref.ref_convert_metadata(sc.ctypes.data_as(orc._u16p),
                                      bi.ctypes.data_as(orc._u16p), count,
                                      inter.ctypes.data_as(orc._u16p))
    assert status == 0
    out["convert_metadata"] = {"scales_bf16": [int(v) for v in sc],
                               "biases_bf16": [int(v) for v in bi],
                               "interleaved_f16": [int(v) for v in inter]}

    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "ref_pins.json")
    with open(path, "w") as handle:
        json.dump(out, handle, separators=(",", ":"))
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
