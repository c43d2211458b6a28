"""Layer-image files of the reference runtime: a writer for synthetic images and
the host-side view of the library's loader.

File layouts (little-endian, one 4096-byte header, page-aligned segments):
  * DeltaNet layer  -- models/qwen3.8-27b/targets/apple-m3-pro/qwen38_m3_image.h:26-94,
    magic "Q38M3Q4\\0", version 3;
  * attention layer -- qwen38_m3_attention_image.h:21-72, magic "Q38M3ATT", version 1;
  * global          -- qwen38_m3_global_image.h:14-38, magic "Q38M3GLB", version 1;
  * MTP extras      -- qwen38_m3_mtp_image.h:21-51, magic "Q38M3MTP", version 1.
The packer that writes the real files is compiler/qwen3.8-27b/apple-m3-pro/
qwen38_m3_pack.c; the checkpoint it reads is not available here, so tests and
benchmarks build images from seeded matrices with `write_layer_image`.
"""
from __future__ import annotations

import ctypes
import struct

import numpy as np

from .host import Q4Context, Q4Error, Q4Weight, _vp, library

PAGE = 4096
DELTA, ATTENTION, GLOBAL, MTP = 0, 1, 2, 3
EMBEDDING, LM_HEAD = 0, 1
FC = 0
GATE, UP, DOWN, INPUT, OUTPUT = range(5)
MATRIX_NAMES = ("gate", "up", "down", "input", "output")

# field -> (byte offset, struct format); the restated header layouts
_DELTA_FIELDS = {
    "version": (8, "<I"), "header_bytes": (12, "<I"), "hidden_size": (16, "<I"), "rows": (20, "<I"),
    "group_size": (24, "<I"), "source_reference_count": (32, "<I"), "down_rows": (40, "<I"),
    "down_groups_per_row": (44, "<I"), "source_mlp_reference_count": (48, "<I"),
    "gate_quants_offset": (56, "<Q"), "gate_quants_bytes": (64, "<Q"), "gate_metadata_offset": (72, "<Q"),
    "gate_metadata_bytes": (80, "<Q"), "up_quants_offset": (88, "<Q"), "up_quants_bytes": (96, "<Q"),
    "up_metadata_offset": (104, "<Q"), "up_metadata_bytes": (112, "<Q"), "down_quants_offset": (120, "<Q"),
    "down_quants_bytes": (128, "<Q"), "down_metadata_offset": (136, "<Q"), "down_metadata_bytes": (144, "<Q"),
    "source_sha256": (152, "65s"), "source_reference_first_8": (220, "<8f"),
    "source_mlp_reference_first_8": (252, "<8f"), "layer_index": (284, "<I"), "delta_input_rows": (288, "<I"),
    "delta_input_groups_per_row": (292, "<I"), "delta_output_rows": (296, "<I"),
    "delta_output_groups_per_row": (300, "<I"), "constants_f32_count": (304, "<I"),
    "source_layer_reference_count": (308, "<I"), "constants_offset": (320, "<Q"), "constants_bytes": (328, "<Q"),
    "delta_input_quants_offset": (384, "<Q"), "delta_input_quants_bytes": (392, "<Q"),
    "delta_input_metadata_offset": (400, "<Q"), "delta_input_metadata_bytes": (408, "<Q"),
    "delta_output_quants_offset": (416, "<Q"), "delta_output_quants_bytes": (424, "<Q"),
    "delta_output_metadata_offset": (432, "<Q"), "delta_output_metadata_bytes": (440, "<Q"),
    "source_layer_reference_first_8": (448, "<8f"), "mlp_source_sha256": (480, "65s"),
}
_ATTENTION_FIELDS = {
    "version": (8, "<I"), "header_bytes": (12, "<I"), "layer_index": (16, "<I"), "hidden_size": (20, "<I"),
    "intermediate_size": (24, "<I"), "group_size": (28, "<I"), "q_heads": (32, "<I"), "kv_heads": (36, "<I"),
    "head_size": (40, "<I"), "rotary_size": (44, "<I"), "input_rows": (48, "<I"),
    "input_groups_per_row": (52, "<I"), "output_rows": (56, "<I"), "output_groups_per_row": (60, "<I"),
    "constants_f32_count": (64, "<I"),
    "gate_quants_offset": (72, "<Q"), "gate_quants_bytes": (80, "<Q"), "gate_metadata_offset": (88, "<Q"),
    "gate_metadata_bytes": (96, "<Q"), "up_quants_offset": (104, "<Q"), "up_quants_bytes": (112, "<Q"),
    "up_metadata_offset": (120, "<Q"), "up_metadata_bytes": (128, "<Q"), "down_quants_offset": (136, "<Q"),
    "down_quants_bytes": (144, "<Q"), "down_metadata_offset": (152, "<Q"), "down_metadata_bytes": (160, "<Q"),
    "constants_offset": (168, "<Q"), "constants_bytes": (176, "<Q"),
    "attention_input_quants_offset": (216, "<Q"), "attention_input_quants_bytes": (224, "<Q"),
    "attention_input_metadata_offset": (232, "<Q"), "attention_input_metadata_bytes": (240, "<Q"),
    "attention_output_quants_offset": (248, "<Q"), "attention_output_quants_bytes": (256, "<Q"),
    "attention_output_metadata_offset": (264, "<Q"), "attention_output_metadata_bytes": (272, "<Q"),
    "source_sha256": (280, "65s"),
}
_GLOBAL_FIELDS = {
    "version": (8, "<I"), "header_bytes": (12, "<I"), "vocab_size": (16, "<I"), "hidden_size": (20, "<I"),
    "group_size": (24, "<I"), "constants_f32_count": (28, "<I"),
    "embedding_quants_offset": (40, "<Q"), "embedding_quants_bytes": (48, "<Q"),
    "embedding_metadata_offset": (56, "<Q"), "embedding_metadata_bytes": (64, "<Q"),
    "lm_head_quants_offset": (72, "<Q"), "lm_head_quants_bytes": (80, "<Q"),
    "lm_head_metadata_offset": (88, "<Q"), "lm_head_metadata_bytes": (96, "<Q"),
    "constants_offset": (104, "<Q"), "constants_bytes": (112, "<Q"),
    "embedding_source_sha256": (120, "65s"), "lm_head_source_sha256": (185, "65s"),
}
_MTP_FIELDS = {
    "version": (8, "<I"), "header_bytes": (12, "<I"), "hidden_size": (16, "<I"), "fc_rows": (20, "<I"),
    "fc_groups_per_row": (24, "<I"), "group_size": (28, "<I"), "constants_f32_count": (32, "<I"),
    "fc_quants_offset": (40, "<Q"), "fc_quants_bytes": (48, "<Q"), "fc_metadata_offset": (56, "<Q"),
    "fc_metadata_bytes": (64, "<Q"), "constants_offset": (72, "<Q"), "constants_bytes": (80, "<Q"),
    "embedding_norm_constants_index": (88, "<Q"), "hidden_norm_constants_index": (96, "<Q"),
    "final_norm_constants_index": (104, "<Q"), "source_sha256": (112, "65s"),
}
FIELDS = {DELTA: _DELTA_FIELDS, ATTENTION: _ATTENTION_FIELDS, GLOBAL: _GLOBAL_FIELDS, MTP: _MTP_FIELDS}
MAGIC = {DELTA: b"Q38M3Q4\0", ATTENTION: b"Q38M3ATT", GLOBAL: b"Q38M3GLB", MTP: b"Q38M3MTP"}
VERSION = {DELTA: 3, ATTENTION: 1, GLOBAL: 1, MTP: 1}
_SEGMENT_PREFIX = {DELTA: ("gate", "up", "down", "delta_input", "delta_output"),
                   ATTENTION: ("gate", "up", "down", "attention_input", "attention_output")}


def _padded(data: bytes) -> bytes:
    return data + b"\0" * (-len(data) % PAGE)


def write_layer_image(path: str, kind: int, layer_index: int, hidden_size: int, intermediate_size: int,
                      matrices, constants: np.ndarray | None = None, source_sha256: str = "0" * 64,
                      gate_up_reference=None, mlp_reference=None, extra_fields: dict | None = None) -> dict:
    """Write one layer image.  `matrices` maps GATE..OUTPUT to (quants, meta):
    quants uint8 [rows, K/2] (code j of a group in byte j>>1, low nibble even),
    meta uint16 [rows, K/64, 2] (fp16 scale and bias bits).  Shapes: gate/up
    [intermediate, hidden], down [hidden, intermediate], input [any, hidden],
    output [hidden, any].  Returns the header fields written."""
    fields = FIELDS[kind]
    constants = np.zeros(0, dtype=np.float32) if constants is None else np.ascontiguousarray(constants, np.float32)
    header = bytearray(PAGE)
    header[0:8] = MAGIC[kind]
    values: dict = {"version": VERSION[kind], "header_bytes": PAGE, "hidden_size": hidden_size, "group_size": 64,
                    "layer_index": layer_index, "constants_f32_count": int(constants.size),
                    "source_sha256": source_sha256.encode()}
    shapes = {m: (int(q.shape[0]), int(meta.shape[1])) for m, (q, meta) in matrices.items()}
    if kind == DELTA:
        values.update(rows=intermediate_size, down_rows=shapes[DOWN][0], down_groups_per_row=shapes[DOWN][1],
                      delta_input_rows=shapes[INPUT][0], delta_input_groups_per_row=shapes[INPUT][1],
                      delta_output_rows=shapes[OUTPUT][0], delta_output_groups_per_row=shapes[OUTPUT][1])
        if gate_up_reference is not None:
            values.update(source_reference_first_8=tuple(float(v) for v in gate_up_reference),
                          source_reference_count=8)
        if mlp_reference is not None:
            values.update(source_mlp_reference_first_8=tuple(float(v) for v in mlp_reference),
                          source_mlp_reference_count=8)
    else:
        values.update(intermediate_size=intermediate_size, input_rows=shapes[INPUT][0],
                      input_groups_per_row=shapes[INPUT][1], output_rows=shapes[OUTPUT][0],
                      output_groups_per_row=shapes[OUTPUT][1])
    body = bytearray()

    def append(data: bytes) -> tuple[int, int]:
        offset = PAGE + len(body)
        padded = _padded(data)
        body.extend(padded)
        return offset, len(padded)

    order = [GATE, UP, DOWN, "constants", INPUT, OUTPUT]  # the output metadata must end the file
    for item in order:
        if item == "constants":
            values["constants_offset"], values["constants_bytes"] = append(constants.tobytes())
            continue
        quants, meta = matrices[item]
        prefix = _SEGMENT_PREFIX[kind][item]
        values[f"{prefix}_quants_offset"], values[f"{prefix}_quants_bytes"] = append(
            np.ascontiguousarray(quants, np.uint8).tobytes())
        values[f"{prefix}_metadata_offset"], values[f"{prefix}_metadata_bytes"] = append(
            np.ascontiguousarray(meta, np.uint16).tobytes())
    values.update(extra_fields or {})
    for name, value in values.items():
        offset, fmt = fields[name]
        if fmt.endswith("f"):
            struct.pack_into(fmt, header, offset, *value)
        else:
            struct.pack_into(fmt, header, offset, value)
    with open(path, "wb") as handle:
        handle.write(header)
        handle.write(body)
    return values


def write_global_image(path: str, hidden_size: int, embedding, lm_head, constants: np.ndarray | None = None,
                       embedding_sha256: str = "0" * 64, lm_head_sha256: str = "0" * 64) -> dict:
    """Write a global image (qwen38_m3_global_image.h): embedding and lm_head, each (quants uint8
    [vocab, hidden/2], meta uint16 [vocab, hidden/64, 2]); the fp32 constants end the file."""
    fields = FIELDS[GLOBAL]
    constants = np.zeros(0, dtype=np.float32) if constants is None else np.ascontiguousarray(constants, np.float32)
    header = bytearray(PAGE)
    header[0:8] = MAGIC[GLOBAL]
    values: dict = {"version": VERSION[GLOBAL], "header_bytes": PAGE, "vocab_size": int(embedding[0].shape[0]),
                    "hidden_size": hidden_size, "group_size": 64, "constants_f32_count": int(constants.size),
                    "embedding_source_sha256": embedding_sha256.encode(),
                    "lm_head_source_sha256": lm_head_sha256.encode()}
    body = bytearray()

    def append(data: bytes) -> tuple[int, int]:
        offset = PAGE + len(body)
        padded = _padded(data)
        body.extend(padded)
        return offset, len(padded)

    for prefix, (quants, meta) in (("embedding", embedding), ("lm_head", lm_head)):
        values[f"{prefix}_quants_offset"], values[f"{prefix}_quants_bytes"] = append(
            np.ascontiguousarray(quants, np.uint8).tobytes())
        values[f"{prefix}_metadata_offset"], values[f"{prefix}_metadata_bytes"] = append(
            np.ascontiguousarray(meta, np.uint16).tobytes())
    values["constants_offset"], values["constants_bytes"] = append(constants.tobytes())
    for name, value in values.items():
        offset, fmt = fields[name]
        struct.pack_into(fmt, header, offset, value)
    with open(path, "wb") as handle:
        handle.write(header)
        handle.write(body)
    return values


def write_mtp_image(path: str, hidden_size: int, fc, embedding_norm, hidden_norm, final_norm,
                    source_sha256: str = "0" * 64, extra_fields: dict | None = None) -> dict:
    """Write an MTP extras image (qwen38_m3_mtp_image.h): the fused fc projection (quants uint8
    [hidden, hidden], meta uint16 [hidden, 2 * hidden / 64, 2]) and the three norm vectors, which
    become the constants (embedding norm, hidden norm, final norm) and end the file."""
    fields = FIELDS[MTP]
    constants = np.concatenate([np.ascontiguousarray(v, np.float32).ravel()
                                for v in (embedding_norm, hidden_norm, final_norm)])
    quants, meta = fc
    header = bytearray(PAGE)
    header[0:8] = MAGIC[MTP]
    values: dict = {"version": VERSION[MTP], "header_bytes": PAGE, "hidden_size": hidden_size,
                    "fc_rows": int(quants.shape[0]), "fc_groups_per_row": int(meta.shape[1]), "group_size": 64,
                    "constants_f32_count": int(constants.size), "embedding_norm_constants_index": 0,
                    "hidden_norm_constants_index": hidden_size, "final_norm_constants_index": 2 * hidden_size,
                    "source_sha256": source_sha256.encode()}
    body = bytearray()
    for prefix, data in (("fc_quants", np.ascontiguousarray(quants, np.uint8).tobytes()),
                         ("fc_metadata", np.ascontiguousarray(meta, np.uint16).tobytes()),
                         ("constants", constants.tobytes())):
        padded = _padded(data) if prefix != "constants" else data  # the runtime wants offset + bytes == file length
        values[f"{prefix}_offset"], values[f"{prefix}_bytes"] = PAGE + len(body), len(padded)
        body.extend(padded)
    values.update(extra_fields or {})
    for name, value in values.items():
        offset, fmt = fields[name]
        struct.pack_into(fmt, header, offset, value)
    with open(path, "wb") as handle:
        handle.write(header)
        handle.write(body)
    return values


class _Info(ctypes.Structure):
    _fields_ = [("kind", ctypes.c_uint32), ("version", ctypes.c_uint32), ("layer_index", ctypes.c_uint32),
                ("hidden_size", ctypes.c_uint32), ("intermediate_size", ctypes.c_uint32),
                ("group_size", ctypes.c_uint32), ("rows", ctypes.c_uint32 * 5), ("groups", ctypes.c_uint32 * 5),
                ("constants_f32_count", ctypes.c_uint32), ("reference_counts", ctypes.c_uint32 * 3),
                ("gate_up_reference_first_8", ctypes.c_float * 8), ("mlp_reference_first_8", ctypes.c_float * 8),
                ("layer_reference_first_8", ctypes.c_float * 8), ("source_sha256", ctypes.c_char * 65),
                ("mlp_source_sha256", ctypes.c_char * 65), ("constants_index", ctypes.c_uint64 * 3)]


class Q4Image:
    """An opened, validated layer image (q4b_image_open).  Needs no GPU until a matrix is uploaded."""

    def __init__(self, path: str, kind: int, layer_index: int, check_27b_shapes: bool = False,
                 allowed_sha256: list[str] | None = None):
        lib = library()
        lib.q4b_image_open.restype = ctypes.c_int
        lib.q4b_image_open.argtypes = [ctypes.c_char_p, ctypes.c_int, ctypes.c_uint32, ctypes.c_int,
                                       ctypes.POINTER(ctypes.c_char_p), ctypes.c_int, ctypes.POINTER(_vp),
                                       ctypes.c_char_p, ctypes.c_size_t]
        lib.q4b_image_describe.argtypes = [_vp, ctypes.POINTER(_Info)]
        lib.q4b_image_constants.restype = ctypes.POINTER(ctypes.c_float)
        lib.q4b_image_constants.argtypes = [_vp, ctypes.POINTER(ctypes.c_uint32)]
        lib.q4b_image_weight.argtypes = [_vp, _vp, ctypes.c_int, ctypes.c_uint32, ctypes.c_uint32,
                                         ctypes.POINTER(_vp), ctypes.c_char_p, ctypes.c_size_t]
        lib.q4b_image_close.argtypes = [_vp]
        lib.q4b_image_close.restype = None
        digests = None
        if allowed_sha256 is not None:
            digests = (ctypes.c_char_p * len(allowed_sha256))(*[d.encode() for d in allowed_sha256])
        handle = _vp()
        message = ctypes.create_string_buffer(512)
        code = lib.q4b_image_open(path.encode(), kind, layer_index, int(check_27b_shapes), digests,
                                  0 if allowed_sha256 is None else len(allowed_sha256), ctypes.byref(handle),
                                  message, 512)
        if code != 0:
            raise Q4Error(code, message.value.decode())
        self.handle = handle
        info = _Info()
        lib.q4b_image_describe(self.handle, ctypes.byref(info))
        self.info = info

    def shape(self, matrix: int) -> tuple[int, int]:
        """(rows, groups per row) of a matrix."""
        return int(self.info.rows[matrix]), int(self.info.groups[matrix])

    def constants(self) -> np.ndarray:
        count = ctypes.c_uint32()
        pointer = library().q4b_image_constants(self.handle, ctypes.byref(count))
        return np.ctypeslib.as_array(pointer, shape=(count.value,)).copy() if count.value else np.zeros(0, np.float32)

    def weight(self, ctx: Q4Context, matrix: int, row_begin: int = 0, row_count: int | None = None) -> Q4Weight:
        rows, _ = self.shape(matrix)
        handle = _vp()
        ctx._check(library().q4b_image_weight(ctx.handle, self.handle, matrix, row_begin,
                                              rows - row_begin if row_count is None else row_count,
                                              ctypes.byref(handle), ctx._err, 512))
        return Q4Weight(ctx, handle)

    def close(self):
        if self.handle:
            library().q4b_image_close(self.handle)
            self.handle = None


class Q4LayerMatmuls:
    """The Q4 matmuls of one layer on one rank (q4b_layer_*): the host-side mirror
    of the reference's encode_mlp / in-projection / out-projection dispatch."""

    def __init__(self, ctx: Q4Context, handle):
        self.ctx, self.handle = ctx, handle

    @staticmethod
    def _prototypes():
        lib = library()
        err = [ctypes.c_char_p, ctypes.c_size_t]
        u32, i32 = ctypes.c_uint32, ctypes.c_int
        lib.q4b_layer_load.argtypes = [_vp, _vp, u32, u32, ctypes.POINTER(_vp)] + err
        lib.q4b_layer_wrap.argtypes = [ctypes.POINTER(_vp), ctypes.POINTER(u32), ctypes.POINTER(u32), u32, u32,
                                       ctypes.POINTER(_vp)]
        lib.q4b_layer_free.argtypes = [_vp, _vp]
        lib.q4b_layer_free.restype = None
        lib.q4b_layer_slice.argtypes = [u32, u32, u32, ctypes.POINTER(u32), ctypes.POINTER(u32)]
        lib.q4b_layer_slice.restype = None
        lib.q4b_layer_encode_input.argtypes = [_vp, _vp, _vp, u32, _vp, i32] + err
        lib.q4b_layer_encode_output.argtypes = [_vp, _vp, _vp, i32, u32, _vp, i32, _vp, i32] + err
        lib.q4b_layer_encode_gate_up.argtypes = [_vp, _vp, _vp, u32, _vp, i32] + err
        lib.q4b_layer_encode_down.argtypes = [_vp, _vp, _vp, i32, u32, _vp, i32, _vp, i32] + err
        lib.q4b_layer_encode_mlp.argtypes = [_vp, _vp, _vp, u32, _vp, i32, _vp, i32, _vp, i32] + err
        return lib

    @classmethod
    def load(cls, ctx: Q4Context, image: Q4Image, rank: int = 0, world: int = 1) -> "Q4LayerMatmuls":
        lib = cls._prototypes()
        handle = _vp()
        ctx._check(lib.q4b_layer_load(ctx.handle, image.handle, rank, world, ctypes.byref(handle), ctx._err, 512))
        return cls(ctx, handle)

    @classmethod
    def wrap(cls, ctx: Q4Context, matrices, rows_total, row_begin, rank: int = 0, world: int = 1) -> "Q4LayerMatmuls":
        lib = cls._prototypes()
        handles = (_vp * 5)(*[None if m is None else m.handle for m in matrices])
        totals = (ctypes.c_uint32 * 5)(*rows_total)
        begins = (ctypes.c_uint32 * 5)(*row_begin)
        handle = _vp()
        if lib.q4b_layer_wrap(handles, totals, begins, rank, world, ctypes.byref(handle)) != 0:
            raise Q4Error(1, "invalid layer description")
        return cls(ctx, handle)

    @classmethod
    def slice_of(cls, rows: int, rank: int, world: int) -> tuple[int, int]:
        lib = cls._prototypes()
        begin, count = ctypes.c_uint32(), ctypes.c_uint32()
        lib.q4b_layer_slice(rows, rank, world, ctypes.byref(begin), ctypes.byref(count))
        return begin.value, count.value

    def encode_input(self, normalized: int, batch: int, projected: int, dtype: int):
        self.ctx._check(library().q4b_layer_encode_input(self.ctx.handle, self.handle, normalized, batch, projected,
                                                         dtype, self.ctx._err, 512))

    def encode_output(self, mixer: int, mixer_dtype: int, batch: int, residual, residual_dtype: int, hidden: int,
                      hidden_dtype: int):
        self.ctx._check(library().q4b_layer_encode_output(self.ctx.handle, self.handle, mixer, mixer_dtype, batch,
                                                          residual, residual_dtype, hidden, hidden_dtype,
                                                          self.ctx._err, 512))

    def encode_gate_up(self, post_normalized: int, batch: int, intermediate: int, dtype: int):
        self.ctx._check(library().q4b_layer_encode_gate_up(self.ctx.handle, self.handle, post_normalized, batch,
                                                           intermediate, dtype, self.ctx._err, 512))

    def encode_down(self, intermediate: int, dtype: int, batch: int, residual, residual_dtype: int, out: int,
                    out_dtype: int):
        self.ctx._check(library().q4b_layer_encode_down(self.ctx.handle, self.handle, intermediate, dtype, batch,
                                                        residual, residual_dtype, out, out_dtype, self.ctx._err, 512))

    def encode_mlp(self, post_normalized: int, batch: int, intermediate: int, dtype: int, residual,
                   residual_dtype: int, out: int, out_dtype: int):
        self.ctx._check(library().q4b_layer_encode_mlp(self.ctx.handle, self.handle, post_normalized, batch,
                                                       intermediate, dtype, residual, residual_dtype, out, out_dtype,
                                                       self.ctx._err, 512))

    def free(self):
        if self.handle:
            library().q4b_layer_free(self.ctx.handle, self.handle)
            self.handle = None
