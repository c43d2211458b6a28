"""The C binding documented for the reference's runtime, compiled and run.

tests/c/encode_mlp.c is the `b200_encode_mlp` of the integration notes (the counterpart of encode_mlp,
qwen38_m3_decode.m:639-660) inside a small C11 program that includes only include/q4b200.h and links
libq4b200.so.  Without a GPU it must compile and link (the header is valid C, every symbol it uses exists);
with one it runs, and its outputs are compared with the oracle."""
import os
import shutil
import subprocess

import numpy as np
import pytest

from q4_cases import assert_close

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SOURCE = os.path.join(ROOT, "tests", "c", "encode_mlp.c")


def build_program(q4b, directory):
    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no gcc")
    library = q4b.library_path()
    q4b.library()  # builds it when stale
    program = os.path.join(directory, "encode_mlp")
    command = [gcc, "-std=c11", "-Wall", "-Wextra", "-Werror", "-O1", "-I", os.path.join(ROOT, "include"), SOURCE,
               "-o", program, library, f"-Wl,-rpath,{os.path.dirname(library)}", "-Wl,--allow-shlib-undefined"]
    result = subprocess.run(command, capture_output=True, text=True)
    assert result.returncode == 0, result.stderr
    return program


def test_documented_binding_compiles_and_links(q4b, tmp_path):
    build_program(q4b, str(tmp_path))


@pytest.mark.gpu
@pytest.mark.parametrize("batch", [1, 4, 40])
def test_documented_binding_runs(q4b, orc, tmp_path, batch):
    program = build_program(q4b, str(tmp_path))
    hidden, intermediate, seed = 1024, 3072, 77
    out = os.path.join(str(tmp_path), "out.bin")
    result = subprocess.run([program, str(hidden), str(intermediate), str(batch), str(seed), out], capture_output=True,
                            text=True, timeout=300)
    assert result.returncode == 0, result.stdout + result.stderr
    assert "encode_mlp ok" in result.stdout
    raw = open(out, "rb").read()
    middle = np.frombuffer(raw[:batch * intermediate * 2], dtype=np.float16).reshape(batch, intermediate)
    final = np.frombuffer(raw[batch * intermediate * 2:], dtype=np.float32).reshape(batch, hidden)
    gq, gm = orc.synth_weight(seed, 0, intermediate, hidden // 64)
    uq, um = orc.synth_weight(seed, 1, intermediate, hidden // 64)
    dq, dm = orc.synth_weight(seed, 2, hidden, intermediate // 64)
    x = orc.synth_x(seed, 0, batch, hidden)
    residual = orc.synth_x(seed, 1, batch, hidden).astype(np.float32)
    _, want_middle = orc.gate_up_silu(gq, gm, uq, um, hidden // 64, x, want32=False)
    assert_close(middle, want_middle, "gate/up + SiLU through the C binding")
    # down multiplies what the device wrote (fp16), as the reference's second projection reads its input buffer
    _, want_final = orc.matmul(dq, dm, intermediate // 64, middle, residual=residual, want32=False)
    assert_close(final, want_final, "down + residual through the C binding")
