// The Q4 matmuls of one decoder layer as the reference's encoders issue them.
//
// Host-side counterpart of the reference runtime's per-layer dispatch
// (models/qwen3.8-27b/targets/apple-m3-pro/qwen38_m3_decode.m): encode_mlp
// (:639-660) and encode_prefill_mlp (:1016-1038) -- fused gate/up with the SiLU
// gate, then down with the residual added; the in-projection at the head of
// encode_delta (:668-674) / encode_attention (:747-753) and the out-projection with
// residual at their tails (:716-723, :788-795), with their batched forms
// encode_prefill_gemm_f16 (:885-928) and encode_prefill_gemm_residual (:930-1001).
// What sits between those matmuls (norms, the DeltaNet recurrence, attention) is not
// part of this library; the caller runs it on the same stream.
//
// A layer holds the row slice of each matrix that this rank owns (column-parallel
// over `world` ranks, 16-row granular).  Every call writes its slice at its
// column offset of the full-width output, so the caller's gather -- or the
// single-GPU case, where the slice is everything -- sees [batch, N] row-major.
#include "../../include/q4b200.h"

#include <cstdarg>
#include <cstdio>
#include <new>

namespace {

void layer_message(char *message, size_t capacity, const char *format, ...) {
    if (message == nullptr || capacity == 0) return;
    va_list arguments;
    va_start(arguments, format);
    vsnprintf(message, capacity, format, arguments);
    va_end(arguments);
}

size_t element_bytes(int dtype) { return dtype == Q4B_F32 ? 4 : 2; }

}  // namespace

struct q4b_layer {
    q4b_weight *matrix[5];     // by Q4B_MATRIX_*: this rank's rows
    uint32_t rows[5];          // rows of the whole matrix
    uint32_t begin[5], count[5];
    uint32_t rank, world;
    bool owns;                 // the layer frees its matrices
};

extern "C" {

void q4b_layer_slice(uint32_t rows, uint32_t rank, uint32_t world, uint32_t *row_begin, uint32_t *row_count) {
    // contiguous, 16-row granular, the first (tiles % world) ranks take one tile more
    const uint32_t tiles = (rows + 15) / 16;
    const uint32_t per = tiles / world, extra = tiles % world;
    const uint32_t begin_tile = rank * per + (rank < extra ? rank : extra);
    const uint32_t count_tile = per + (rank < extra ? 1u : 0u);
    uint32_t begin = begin_tile * 16, end = (begin_tile + count_tile) * 16;
    if (begin > rows) begin = rows;
    if (end > rows) end = rows;
    if (row_begin != nullptr) *row_begin = begin;
    if (row_count != nullptr) *row_count = end - begin;
}

int q4b_layer_load(q4b_context *context, const q4b_image *image, uint32_t rank, uint32_t world,
                   q4b_layer **layer, char *error_message, size_t error_capacity) {
    q4b_image_info info;
    if (layer == nullptr || world == 0 || rank >= world || q4b_image_describe(image, &info) != Q4B_OK) {
        layer_message(error_message, error_capacity, "no image, no result pointer or rank outside the world");
        return Q4B_BAD_ARGUMENT;
    }
    q4b_layer *result = new (std::nothrow) q4b_layer();
    if (result == nullptr) return Q4B_DEVICE_FAILURE;
    result->rank = rank;
    result->world = world;
    result->owns = true;
    for (int m = 0; m < 5; ++m) {
        result->rows[m] = info.rows[m];
        q4b_layer_slice(info.rows[m], rank, world, &result->begin[m], &result->count[m]);
        if (result->count[m] == 0) {
            layer_message(error_message, error_capacity, "matrix %d has fewer 16-row tiles than ranks", m);
            q4b_layer_free(context, result);
            return Q4B_BAD_ARGUMENT;
        }
        const int status = q4b_image_weight(context, image, m, result->begin[m], result->count[m], &result->matrix[m],
                                            error_message, error_capacity);
        if (status != Q4B_OK) {
            q4b_layer_free(context, result);
            return status;
        }
    }
    *layer = result;
    return Q4B_OK;
}

int q4b_layer_wrap(const q4b_weight *const *matrices, const uint32_t *rows_total, const uint32_t *row_begin,
                   uint32_t rank, uint32_t world, q4b_layer **layer) {
    if (matrices == nullptr || rows_total == nullptr || row_begin == nullptr || layer == nullptr || world == 0 ||
        rank >= world) {
        return Q4B_BAD_ARGUMENT;
    }
    q4b_layer *result = new (std::nothrow) q4b_layer();
    if (result == nullptr) return Q4B_DEVICE_FAILURE;
    result->rank = rank;
    result->world = world;
    result->owns = false;
    for (int m = 0; m < 5; ++m) {
        result->matrix[m] = const_cast<q4b_weight *>(matrices[m]);  // may be NULL: that call is then refused
        result->rows[m] = rows_total[m];
        result->begin[m] = row_begin[m];
        uint32_t rows = 0, groups = 0;
        uint64_t bytes = 0;
        if (matrices[m] != nullptr) q4b_weight_info(matrices[m], &rows, &groups, &bytes);
        result->count[m] = rows;
        if (matrices[m] != nullptr && row_begin[m] + rows > rows_total[m]) {
            delete result;
            return Q4B_BAD_ARGUMENT;
        }
    }
    *layer = result;
    return Q4B_OK;
}

void q4b_layer_free(q4b_context *context, q4b_layer *layer) {
    if (layer == nullptr) return;
    if (layer->owns) {
        for (int m = 0; m < 5; ++m) {
            if (layer->matrix[m] != nullptr) q4b_weight_free(context, layer->matrix[m]);
        }
    }
    delete layer;
}

// one matrix of the layer: y[:, begin:begin+count] = x W_slice^T (+ residual slice), outputs [batch, rows] wide
static int layer_matmul(q4b_context *context, const q4b_layer *layer, int m, const void *x, int x_dtype,
                        uint32_t batch, void *y, int y_dtype, const void *residual, int residual_dtype,
                        char *error_message, size_t error_capacity) {
    if (layer == nullptr || layer->matrix[m] == nullptr || y == nullptr) {
        layer_message(error_message, error_capacity, "the layer does not hold that matrix, or no output");
        return Q4B_BAD_ARGUMENT;
    }
    const uint32_t width = layer->rows[m], begin = layer->begin[m];
    void *out = static_cast<unsigned char *>(y) + (size_t)begin * element_bytes(y_dtype);
    const void *res = residual == nullptr
                          ? nullptr
                          : static_cast<const unsigned char *>(residual) + (size_t)begin * element_bytes(residual_dtype);
    return q4b_matmul(context, layer->matrix[m], x, x_dtype, batch, out, y_dtype, width, res,
                      residual == nullptr ? -1 : residual_dtype, width, error_message, error_capacity);
}

int q4b_layer_encode_input(q4b_context *context, const q4b_layer *layer, const void *normalized_f16, uint32_t batch,
                           void *projected, int projected_dtype, char *error_message, size_t error_capacity) {
    return layer_matmul(context, layer, Q4B_MATRIX_INPUT, normalized_f16, Q4B_F16, batch, projected, projected_dtype,
                        nullptr, -1, error_message, error_capacity);
}

int q4b_layer_encode_output(q4b_context *context, const q4b_layer *layer, const void *mixer_output, int mixer_dtype,
                            uint32_t batch, const void *residual, int residual_dtype, void *hidden,
                            int hidden_dtype, char *error_message, size_t error_capacity) {
    return layer_matmul(context, layer, Q4B_MATRIX_OUTPUT, mixer_output, mixer_dtype, batch, hidden, hidden_dtype,
                        residual, residual_dtype, error_message, error_capacity);
}

int q4b_layer_encode_gate_up(q4b_context *context, const q4b_layer *layer, const void *post_normalized_f16,
                             uint32_t batch, void *intermediate, int intermediate_dtype, char *error_message,
                             size_t error_capacity) {
    if (layer == nullptr || layer->matrix[Q4B_MATRIX_GATE] == nullptr || layer->matrix[Q4B_MATRIX_UP] == nullptr ||
        intermediate == nullptr) {
        layer_message(error_message, error_capacity, "the layer does not hold gate and up, or no output");
        return Q4B_BAD_ARGUMENT;
    }
    void *out = static_cast<unsigned char *>(intermediate) +
                (size_t)layer->begin[Q4B_MATRIX_GATE] * element_bytes(intermediate_dtype);
    return q4b_gate_up_silu(context, layer->matrix[Q4B_MATRIX_GATE], layer->matrix[Q4B_MATRIX_UP], post_normalized_f16,
                            Q4B_F16, batch, out, intermediate_dtype, layer->rows[Q4B_MATRIX_GATE], error_message,
                            error_capacity);
}

int q4b_layer_encode_down(q4b_context *context, const q4b_layer *layer, const void *intermediate,
                          int intermediate_dtype, uint32_t batch, const void *residual, int residual_dtype,
                          void *layer_output, int output_dtype, char *error_message, size_t error_capacity) {
    return layer_matmul(context, layer, Q4B_MATRIX_DOWN, intermediate, intermediate_dtype, batch, layer_output,
                        output_dtype, residual, residual_dtype, error_message, error_capacity);
}

int q4b_layer_encode_mlp(q4b_context *context, const q4b_layer *layer, const void *post_normalized_f16,
                         uint32_t batch, void *intermediate, int intermediate_dtype, const void *residual,
                         int residual_dtype, void *layer_output, int output_dtype, char *error_message,
                         size_t error_capacity) {
    if (layer != nullptr && layer->world != 1) {
        // down reads the WHOLE intermediate: with ranks, gather between the two halves
        layer_message(error_message, error_capacity,
                      "with %u ranks call q4b_layer_encode_mlp_gathered (gate/up, gather, down, gather)", layer->world);
        return Q4B_BAD_ARGUMENT;
    }
    const int status = q4b_layer_encode_gate_up(context, layer, post_normalized_f16, batch, intermediate,
                                                intermediate_dtype, error_message, error_capacity);
    if (status != Q4B_OK) return status;
    return q4b_layer_encode_down(context, layer, intermediate, intermediate_dtype, batch, residual, residual_dtype,
                                 layer_output, output_dtype, error_message, error_capacity);
}

int q4b_layer_gather(q4b_context *context, const q4b_layer *layer, q4b_comm *comm, int matrix, void *full_width,
                     int dtype, uint32_t batch, void *staging, char *error_message, size_t error_capacity) {
    if (layer == nullptr || comm == nullptr || full_width == nullptr || matrix < 0 || matrix >= 5 || batch == 0 ||
        q4b_comm_world(comm) != layer->world || q4b_comm_rank(comm) != layer->rank) {
        layer_message(error_message, error_capacity, "layer, communicator or buffer missing, or of different worlds");
        return Q4B_BAD_ARGUMENT;
    }
    const uint32_t rows = layer->rows[matrix], count = layer->count[matrix], world = layer->world;
    if (count * world != rows || layer->begin[matrix] != layer->rank * count) {
        layer_message(error_message, error_capacity, "the ranks' slices of matrix %d are not equal (%u rows over %u ranks)",
                      matrix, rows, world);
        return Q4B_BAD_ARGUMENT;
    }
    const size_t width = element_bytes(dtype);
    unsigned char *base = static_cast<unsigned char *>(full_width);
    if (batch == 1) {  // one row: every slice is already where the all-gather puts it
        return q4b_all_gather(context, comm, base + (size_t)layer->begin[matrix] * width, base, (size_t)count * width,
                              error_message, error_capacity);
    }
    if (staging == nullptr) {
        layer_message(error_message, error_capacity, "batch > 1 needs a staging buffer");
        return Q4B_BAD_ARGUMENT;
    }
    // pack this rank's columns, gather rank-major, interleave back into rows
    unsigned char *packed = static_cast<unsigned char *>(staging);
    unsigned char *blocks = packed + (size_t)batch * count * width;
    int status = q4b_copy_2d(context, packed, (size_t)count * width, base + (size_t)layer->begin[matrix] * width,
                             (size_t)rows * width, (size_t)count * width, batch, error_message, error_capacity);
    if (status != Q4B_OK) return status;
    return q4b_all_gather_columns(context, comm, packed, full_width, batch, count, (uint32_t)width, blocks,
                                  error_message, error_capacity);
}

int q4b_layer_encode_mlp_gathered(q4b_context *context, const q4b_layer *layer, q4b_comm *comm,
                                  const void *post_normalized_f16, uint32_t batch, void *intermediate,
                                  int intermediate_dtype, const void *residual, int residual_dtype,
                                  void *layer_output, int output_dtype, void *staging, char *error_message,
                                  size_t error_capacity) {
    int status = q4b_layer_encode_gate_up(context, layer, post_normalized_f16, batch, intermediate, intermediate_dtype,
                                          error_message, error_capacity);
    if (status != Q4B_OK) return status;
    status = q4b_layer_gather(context, layer, comm, Q4B_MATRIX_GATE, intermediate, intermediate_dtype, batch, staging,
                              error_message, error_capacity);
    if (status != Q4B_OK) return status;
    status = q4b_layer_encode_down(context, layer, intermediate, intermediate_dtype, batch, residual, residual_dtype,
                                   layer_output, output_dtype, error_message, error_capacity);
    if (status != Q4B_OK) return status;
    return q4b_layer_gather(context, layer, comm, Q4B_MATRIX_DOWN, layer_output, output_dtype, batch, staging,
                            error_message, error_capacity);
}

}  // extern "C"
