"""Layer-image files on CPU: the restated header layouts against the offsets the
reference's own headers give, and the loader's validation rules
(qwen38_m3_decode.m:374-446) on synthetic images -- good ones and broken ones."""
import importlib
import json
import os
import struct

import numpy as np
import pytest

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "image_header_offsets.json")


@pytest.fixture(scope="module")
def image(q4b):
    return importlib.import_module("cpu-llms-in-c_b200.image")


def small_matrices(orc, hidden=256, intermediate=512, input_rows=320, output_groups=6, seed=11):
    """gate/up [intermediate, hidden], down [hidden, intermediate], input [input_rows, hidden],
    output [hidden, 64 * output_groups]"""
    shapes = [(intermediate, hidden // 64), (intermediate, hidden // 64), (hidden, intermediate // 64),
              (input_rows, hidden // 64), (hidden, output_groups)]
    return {m: orc.synth_weight(seed, m, rows, groups) for m, (rows, groups) in enumerate(shapes)}


def test_restated_layouts_match_the_reference_headers(image):
    golden = json.load(open(GOLDEN))
    for kind, key in ((image.DELTA, "delta"), (image.ATTENTION, "attention"), (image.GLOBAL, "global"),
                      (image.MTP, "mtp")):
        assert golden[key]["sizeof"][0] == image.PAGE
        assert golden[key]["magic"] == [0, 8]
        for name, (offset, fmt) in image.FIELDS[kind].items():
            assert golden[key][name] == [offset, struct.calcsize(fmt)], (key, name)


def test_good_images_open_and_describe_themselves(image, orc, tmp_path):
    matrices = small_matrices(orc)
    constants = np.arange(37, dtype=np.float32) * 0.5
    for kind, layer in ((image.DELTA, 5), (image.ATTENTION, 7), (image.ATTENTION, 64)):
        path = str(tmp_path / f"layer{kind}_{layer}.img")
        image.write_layer_image(path, kind, layer, 256, 512, matrices, constants, source_sha256="ab" * 32,
                                gate_up_reference=range(8), mlp_reference=[0.25] * 8)
        opened = image.Q4Image(path, kind, layer)
        info = opened.info
        assert (info.kind, info.layer_index, info.hidden_size, info.intermediate_size) == (kind, layer, 256, 512)
        assert [opened.shape(m) for m in range(5)] == [(512, 4), (512, 4), (256, 8), (320, 4), (256, 6)]
        assert np.array_equal(opened.constants(), constants)
        assert info.source_sha256 == b"ab" * 32
        if kind == image.DELTA:
            assert list(info.gate_up_reference_first_8) == [float(v) for v in range(8)]
            assert list(info.mlp_reference_first_8) == [0.25] * 8
            assert list(info.reference_counts) == [8, 8, 0]
        opened.close()
        # the digests the caller accepts (the role of pinned_sha)
        image.Q4Image(path, kind, layer, allowed_sha256=["cd" * 32, "ab" * 32]).close()
        with pytest.raises(image.Q4Error) as refused:
            image.Q4Image(path, kind, layer, allowed_sha256=["cd" * 32])
        assert refused.value.status == 3 and "digest" in refused.value.message


def test_broken_images_are_refused(image, orc, tmp_path):
    matrices = small_matrices(orc)
    path = str(tmp_path / "good.img")
    image.write_layer_image(path, image.DELTA, 5, 256, 512, matrices, np.zeros(8, np.float32))
    good = open(path, "rb").read()
    fields = image.FIELDS[image.DELTA]

    def refused(data: bytes, needle: str, layer=5, kind=image.DELTA, strict=False):
        broken = str(tmp_path / "broken.img")
        with open(broken, "wb") as handle:
            handle.write(data)
        with pytest.raises(image.Q4Error) as info:
            image.Q4Image(broken, kind, layer, check_27b_shapes=strict)
        assert info.value.status == 3, info.value.message
        assert needle in info.value.message, info.value.message

    def patched(name, value):
        data = bytearray(good)
        struct.pack_into(fields[name][1], data, fields[name][0], value)
        return bytes(data)

    refused(good[:100], "cannot open")                                   # shorter than one page
    refused(b"X" + good[1:], "magic")
    refused(patched("version", 2), "version")
    refused(patched("header_bytes", 8192), "one page")
    refused(patched("group_size", 128), "group size")
    refused(good, "layer index", layer=6)
    refused(patched("layer_index", 7), "attention layers", layer=7)      # DeltaNet image at an attention layer
    refused(good, "magic", kind=image.ATTENTION, layer=7)
    refused(patched("gate_metadata_offset", struct.unpack_from("<Q", good, fields["gate_metadata_offset"][0])[0] + 16),
            "page-aligned")
    refused(good[:-4096], "outside the file")
    refused(good + b"\0" * 4096, "does not end")
    refused(patched("up_quants_offset", 1 << 40), "outside the file")
    refused(patched("rows", 1024), "smaller than its matrix")
    refused(patched("constants_f32_count", 1 << 24), "constants")
    refused(good, "27B", strict=True)
    with pytest.raises(image.Q4Error) as missing:
        image.Q4Image(str(tmp_path / "absent.img"), image.DELTA, 5)
    assert missing.value.status == 3


def test_segments_are_the_bytes_the_writer_put_there(image, orc, tmp_path):
    import ctypes
    matrices = small_matrices(orc)
    path = str(tmp_path / "layer.img")
    image.write_layer_image(path, image.DELTA, 1, 256, 512, matrices)
    opened = image.Q4Image(path, image.DELTA, 1)
    lib = importlib.import_module("cpu-llms-in-c_b200").library()
    for m, (quants, meta) in matrices.items():
        q, md = ctypes.c_void_p(), ctypes.c_void_p()
        assert lib.q4b_image_segments(opened.handle, m, ctypes.byref(q), ctypes.byref(md)) == 0
        got_q = np.ctypeslib.as_array(ctypes.cast(q, ctypes.POINTER(ctypes.c_uint8)), shape=(quants.size,))
        got_m = np.ctypeslib.as_array(ctypes.cast(md, ctypes.POINTER(ctypes.c_uint16)), shape=(meta.size,))
        assert np.array_equal(got_q, quants.reshape(-1)) and np.array_equal(got_m, meta.reshape(-1))
    opened.close()


def test_row_slices_of_the_c_layer_match_the_python_rule(image, q4b):
    layer = importlib.import_module("cpu-llms-in-c_b200.layer")
    for rows in (16, 100, 1024, 5120, 6144, 16480, 17408, 248320):
        for world in (1, 2, 3, 4, 8):
            covered = 0
            for rank in range(world):
                got = image.Q4LayerMatmuls.slice_of(rows, rank, world)
                assert got == layer.slice_of(rows, rank, world)
                assert got[0] == covered
                covered += got[1]
            assert covered == rows


def test_global_image_opens_and_is_validated(image, orc, tmp_path):
    vocab, hidden = 1000, 256          # a vocabulary that is no multiple of 64
    embedding = orc.synth_weight(5, 0, vocab, hidden // 64)
    lm_head = orc.synth_weight(5, 1, vocab, hidden // 64)
    constants = np.arange(hidden, dtype=np.float32)
    path = str(tmp_path / "global.img")
    image.write_global_image(path, hidden, embedding, lm_head, constants, "aa" * 32, "bb" * 32)
    opened = image.Q4Image(path, image.GLOBAL, 0)
    assert (opened.info.intermediate_size, opened.info.hidden_size) == (vocab, hidden)
    assert opened.shape(image.EMBEDDING) == (vocab, 4) and opened.shape(image.LM_HEAD) == (vocab, 4)
    assert opened.info.source_sha256 == b"aa" * 32 and opened.info.mlp_source_sha256 == b"bb" * 32
    assert np.array_equal(opened.constants(), constants)
    opened.close()
    image.Q4Image(path, image.GLOBAL, 0, allowed_sha256=["aa" * 32, "bb" * 32]).close()
    for bad_list in (["aa" * 32], ["bb" * 32]):
        with pytest.raises(image.Q4Error):
            image.Q4Image(path, image.GLOBAL, 0, allowed_sha256=bad_list)
    with pytest.raises(image.Q4Error) as strict:
        image.Q4Image(path, image.GLOBAL, 0, check_27b_shapes=True)
    assert "27B" in strict.value.message
    data = open(path, "rb").read()
    broken = str(tmp_path / "broken.img")
    with open(broken, "wb") as handle:
        handle.write(data + b"\0" * 4096)
    with pytest.raises(image.Q4Error) as tail:
        image.Q4Image(broken, image.GLOBAL, 0)
    assert "does not end with the constants" in tail.value.message


def test_mtp_extras_image_opens_and_is_validated(image, orc, tmp_path):
    """The rules of qwen38_m3_model_mtp_open (qwen38_m3_decode.m:2365-2380) on a small synthetic image."""
    hidden = 256
    fc = orc.synth_weight(9, 0, hidden, 2 * hidden // 64)
    norms = [np.full(hidden, value, dtype=np.float32) for value in (1.0, 2.0, 3.0)]
    path = str(tmp_path / "mtp.img")
    image.write_mtp_image(path, hidden, fc, *norms, source_sha256="cc" * 32)
    opened = image.Q4Image(path, image.MTP, 0)
    info = opened.info
    assert (info.kind, info.hidden_size, info.constants_f32_count) == (image.MTP, hidden, 3 * hidden)
    assert opened.shape(image.FC) == (hidden, 8)
    assert list(info.constants_index) == [0, hidden, 2 * hidden]
    assert info.source_sha256 == b"cc" * 32
    constants = opened.constants()
    for index, value in zip(info.constants_index, (1.0, 2.0, 3.0)):
        assert np.all(constants[index:index + hidden] == value)
    opened.close()
    image.Q4Image(path, image.MTP, 0, allowed_sha256=["cc" * 32]).close()
    with pytest.raises(image.Q4Error) as digest:
        image.Q4Image(path, image.MTP, 0, allowed_sha256=["dd" * 32])
    assert digest.value.status == 3 and "digest" in digest.value.message
    with pytest.raises(image.Q4Error) as strict:
        image.Q4Image(path, image.MTP, 0, check_27b_shapes=True)
    assert "27B" in strict.value.message
    # another kind's magic, a norm vector past the constants, bytes after the constants
    with pytest.raises(image.Q4Error) as magic:
        image.Q4Image(path, image.GLOBAL, 0)
    assert "magic" in magic.value.message
    outside = str(tmp_path / "outside.img")
    image.write_mtp_image(outside, hidden, fc, *norms, extra_fields={"final_norm_constants_index": 2 * hidden + 1})
    with pytest.raises(image.Q4Error) as norm:
        image.Q4Image(outside, image.MTP, 0)
    assert "norm vector" in norm.value.message
    longer = str(tmp_path / "longer.img")
    with open(longer, "wb") as handle:
        handle.write(open(path, "rb").read() + b"\0" * 4096)
    with pytest.raises(image.Q4Error) as tail:
        image.Q4Image(longer, image.MTP, 0)
    assert "does not end with the constants" in tail.value.message
