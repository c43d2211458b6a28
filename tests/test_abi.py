"""CPU-side checks of the C-ABI library: it loads, exports everything the header
declares, and refuses to work without a GPU instead of falling back."""
import ctypes
import os

import numpy as np
import pytest


def test_library_exports_every_declared_symbol(q4b):
    lib = q4b.library()
    names = q4b.declared_symbols()
    assert len(names) >= 30
    missing = [name for name in names if not hasattr(lib, name)]
    assert missing == []


def test_header_cites_reference_for_each_entry_point():
    header = os.path.join(os.path.dirname(os.path.dirname(__file__)), "include", "q4b200.h")
    text = open(header).read()
    for anchor in ("qwen38_m3_decode.m", "qwen38_q4.metal", "minimax_h3_m3_gemm.h", "qwen38_m3_pack.c"):
        assert anchor in text


def test_no_gpu_means_loud_failure(q4b):
    lib = q4b.library()
    if lib.q4b_device_count() > 0:
        pytest.skip("a GPU is present")
    with pytest.raises(q4b.Q4Error) as info:
        q4b.Q4Context(0)
    assert "no CUDA device" in info.value.message


def test_null_arguments_are_rejected_without_touching_a_device(q4b):
    lib = q4b.library()
    err = ctypes.create_string_buffer(256)
    assert lib.q4b_weight_info(None, None, None, None) == 1
    assert lib.q4b_sync(None, None, err, 256) == 1
    assert b"NULL" in err.value
    assert lib.q4b_matmul(None, None, None, 0, 1, None, 0, 0, None, -1, 0, err, 256) == 1
    assert lib.q4b_graph_launch(None, None, err, 256) == 1
    # the multi-rank, image and layer entry points refuse missing objects the same way
    assert lib.q4b_context_push_outputs(None, 2, None, 1) == 1
    assert lib.q4b_barrier_set_peer(None, 0, None) == 1
    assert lib.q4b_barrier_queue(None, None, err, 256) == 1
    assert lib.q4b_image_describe(None, None) == 1
    assert lib.q4b_image_weight(None, None, 0, 0, 1, None, err, 256) == 1
    assert lib.q4b_layer_wrap(None, None, None, 0, 1, None) == 1
    assert lib.q4b_layer_encode_mlp(None, None, None, 1, None, 0, None, 0, None, 0, err, 256) == 1
    assert lib.q4b_embedding_lookup(None, None, None, 0, None, 0, err, 256) == 1
    assert lib.q4b_rmsnorm(None, None, 0, None, None, 0, 0, ctypes.c_float(1e-6), err, 256) == 1
    assert lib.q4b_sequence_launch(None, None, err, 256) == 1


def test_algorithmic_bytes_match_the_stated_anchors(q4b):
    # 27B layer: 191,692,800 weight bytes; config[0]: 1,769,472
    weights = sum(q4b.shapes.weight_bytes(p) for p in q4b.LAYER_27B)
    assert weights == 191_692_800
    small = sum(q4b.shapes.weight_bytes(p) for p in q4b.LAYER_SMALL)
    assert small == 8_257_536
    single = q4b.Projection("config0", 1024, 3072)
    assert q4b.shapes.weight_bytes(single) == 1_769_472
    assert q4b.layer_flops(q4b.LAYER_27B, 1) == 681_574_400


def test_bf16_planes_that_do_not_fit_fp16_are_counted(q4b):
    """q4b_planes_narrowed: every bf16 value in fp16's normal range is an fp16 number; the others change."""
    lib = q4b.library()
    def bf16(values):
        return (np.asarray(values, dtype=np.float32).view(np.uint32) >> 16).astype(np.uint16)
    inside = bf16([1.0, -0.00390625, 6.103515625e-05, 65280.0, 0.0, -2.0 ** -14])
    outside = bf16([1.0e-6, 1.0e5, -3.0e38, 2.0 ** -26])
    assert lib.q4b_planes_narrowed(inside.ctypes.data, inside.ctypes.data, q4b.BF16, inside.size) == 0
    assert lib.q4b_planes_narrowed(outside.ctypes.data, inside.ctypes.data, q4b.BF16, 4) == 4
    assert lib.q4b_planes_narrowed(outside.ctypes.data, outside.ctypes.data, q4b.F16, 4) == 0
