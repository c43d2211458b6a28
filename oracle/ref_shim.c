/*
 * Thin driver around the reference's OWN packer source -- TEST INFRASTRUCTURE.
 *
 * The reference's CPU code for the affine-Q4 path lives in `static` functions
 * of compiler/qwen3.8-27b/apple-m3-pro/qwen38_m3_pack.c that read MLX tensors
 * from a file descriptor.  This file textually includes that source (from the
 * reference tree, at build time; nothing is copied into this repository),
 * renames its main(), and exposes those static functions through a tiny C ABI
 * that writes the caller's arrays into an anonymous temporary file first.
 *
 * It exists to pin oracle/q4_oracle.c against the reference itself:
 *   - float_to_half_bits / half_bits_to_float / bf16_to_half   (:110-178)
 *   - convert_metadata (BF16 planes -> interleaved fp16 records) (:420-446)
 *   - source_reference_first_8      (fused gate/up + SiLU)       (:187-239)
 *   - source_mlp_reference_first_8  (whole MLP + residual)       (:241-349)
 * Built by oracle/Makefile into oracle/_ref/ only where the reference tree is
 * present.
 */
#define main qwen38_m3_pack_main
#include "qwen38_m3_pack.c"
#undef main

#include <stdio.h>

static int temp_file(void) {
    FILE *handle = tmpfile();
    if (handle == NULL) {
        return -1;
    }
    int copy = dup(fileno(handle));
    fclose(handle);
    return copy;
}

static int put(int file, const void *data, size_t bytes, uint64_t *offset,
               qwen38_tensor_view *view) {
    memset(view, 0, sizeof(*view));
    view->data_start = *offset;
    view->data_length = bytes;
    if (pwrite_exact(file, data, bytes, *offset) != 0) {
        return -1;
    }
    *offset += bytes;
    return 0;
}

uint16_t ref_float_to_half_bits(float value) { return float_to_half_bits(value); }
float ref_half_bits_to_float(uint16_t bits) { return half_bits_to_float(bits); }
uint16_t ref_bf16_to_half(uint16_t bits) { return bf16_to_half(bits); }

int ref_hidden_size(void) { return QWEN38_HIDDEN_SIZE; }
int ref_mlp_size(void) { return QWEN38_MLP_SIZE; }

/* BF16 scale/bias planes -> interleaved {fp16 scale, fp16 bias} records */
int ref_convert_metadata(const uint16_t *scales_bf16, const uint16_t *biases_bf16,
                         size_t value_count, uint16_t *interleaved_out) {
    int source = temp_file();
    int output = temp_file();
    if (source < 0 || output < 0) {
        return -1;
    }
    uint64_t offset = 0;
    qwen38_tensor_view scales, biases;
    int status = -1;
    if (put(source, scales_bf16, value_count * 2, &offset, &scales) == 0 &&
        put(source, biases_bf16, value_count * 2, &offset, &biases) == 0 &&
        convert_metadata(source, output, &scales, &biases, value_count, 0) == 0 &&
        pread_exact(output, interleaved_out, value_count * 4, 0) == 0) {
        status = 0;
    }
    close(source);
    close(output);
    return status;
}

/* gate/up: [rows][5120/2] code bytes, [rows][80] BF16 scales and biases;
 * at least 8 rows are read. */
int ref_gate_up_first8(const uint8_t *gate_q, const uint16_t *gate_s,
                       const uint16_t *gate_b, const uint8_t *up_q,
                       const uint16_t *up_s, const uint16_t *up_b,
                       float output[8]) {
    const size_t weight_bytes = 8 * (size_t)QWEN38_HIDDEN_SIZE / 2;
    const size_t meta_bytes = 8 * ((size_t)QWEN38_HIDDEN_SIZE / 64) * 2;
    int source = temp_file();
    if (source < 0) {
        return -1;
    }
    uint64_t offset = 0;
    qwen38_tensor_view gw, gs, gb, uw, us, ub;
    int status = -1;
    if (put(source, gate_q, weight_bytes, &offset, &gw) == 0 &&
        put(source, gate_s, meta_bytes, &offset, &gs) == 0 &&
        put(source, gate_b, meta_bytes, &offset, &gb) == 0 &&
        put(source, up_q, weight_bytes, &offset, &uw) == 0 &&
        put(source, up_s, meta_bytes, &offset, &us) == 0 &&
        put(source, up_b, meta_bytes, &offset, &ub) == 0) {
        status = source_reference_first_8(source, &gw, &gs, &gb, &uw, &us, &ub,
                                          output);
    }
    close(source);
    return status;
}

/* whole MLP: gate/up [17408][5120] and the first 8 rows of down [.][17408] */
int ref_mlp_first8(const uint8_t *gate_q, const uint16_t *gate_s,
                   const uint16_t *gate_b, const uint8_t *up_q,
                   const uint16_t *up_s, const uint16_t *up_b,
                   const uint8_t *down_q, const uint16_t *down_s,
                   const uint16_t *down_b, float output[8]) {
    const size_t rows = QWEN38_MLP_SIZE;
    const size_t weight_bytes = rows * (size_t)QWEN38_HIDDEN_SIZE / 2;
    const size_t meta_bytes = rows * ((size_t)QWEN38_HIDDEN_SIZE / 64) * 2;
    const size_t down_weight_bytes = 8 * rows / 2;
    const size_t down_meta_bytes = 8 * (rows / 64) * 2;
    int source = temp_file();
    if (source < 0) {
        return -1;
    }
    uint64_t offset = 0;
    qwen38_tensor_view gw, gs, gb, uw, us, ub, dw, ds, db;
    int status = -1;
    if (put(source, gate_q, weight_bytes, &offset, &gw) == 0 &&
        put(source, gate_s, meta_bytes, &offset, &gs) == 0 &&
        put(source, gate_b, meta_bytes, &offset, &gb) == 0 &&
        put(source, up_q, weight_bytes, &offset, &uw) == 0 &&
        put(source, up_s, meta_bytes, &offset, &us) == 0 &&
        put(source, up_b, meta_bytes, &offset, &ub) == 0 &&
        put(source, down_q, down_weight_bytes, &offset, &dw) == 0 &&
        put(source, down_s, down_meta_bytes, &offset, &ds) == 0 &&
        put(source, down_b, down_meta_bytes, &offset, &db) == 0) {
        status = source_mlp_reference_first_8(source, &gw, &gs, &gb, &uw, &us,
                                              &ub, &dw, &ds, &db, output);
    }
    close(source);
    return status;
}
