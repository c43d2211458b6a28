// Layer-image files: open, validate, hand matrices to the loader.
//
// Replaces map_file / validate_delta_header / validate_attention_header /
// validate_global_header / load_delta_layer / load_attention_layer / load_global of
// the reference runtime (models/qwen3.8-27b/targets/apple-m3-pro/
// qwen38_m3_decode.m:374-625) for the part that concerns the Q4 matmul path: the ten
// Q4 segments of a layer (gate, up, down, input projection, output projection;
// quants + metadata each), the embedding and lm_head of the global image, and the
// embedded eight-row references the packer stored for self-checks.  The file
// layouts are the reference's (qwen38_m3_image.h:26-94, version 3, magic
// "Q38M3Q4\0"; qwen38_m3_attention_image.h:21-72, version 1, magic "Q38M3ATT";
// qwen38_m3_global_image.h:14-38, version 1, magic "Q38M3GLB"; qwen38_m3_mtp_image.h:
// 21-51, version 1, magic "Q38M3MTP", validated as qwen38_m3_model_mtp_open does,
// qwen38_m3_decode.m:2365-2380); they are restated here as field offsets, pinned by a test against the offsets the reference's own
// headers give.
//
// On unified memory the reference wraps the mapping in no-copy buffers; on a B200
// a matrix is uploaded and repacked into the tile stream (q4b_weight_upload), by
// row slice so that every rank of a column-parallel job reads only its rows.
// Host-only code: nothing here touches the GPU except through q4b_weight_upload.
#include "../../include/q4b200.h"

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <fcntl.h>
#include <new>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

namespace {

constexpr uint64_t kPage = 4096;
constexpr uint32_t kMtpLayerIndex = 64;  // qwen38_m3_mtp_image.h:18

struct SegmentFields {  // byte offsets of the four uint64 of one matrix: quants offset/bytes, metadata offset/bytes
    uint32_t quants_offset, quants_bytes, meta_offset, meta_bytes;
};
struct ShapeFields {  // byte offsets of the uint32 rows / groups-per-row of one matrix (0 = derived)
    uint32_t rows, groups;
};
struct Layout {
    unsigned char magic[8];
    uint32_t version;
    uint32_t matrices;          // 5 for a layer image, 2 for the global image (embedding, lm_head)
    uint32_t layer_index, hidden_size, intermediate_size, group_size, constants_count;
    SegmentFields segment[5];   // gate, up, down, input, output
    ShapeFields shape[5];
    uint32_t constants_offset, constants_bytes;
    uint32_t last_segment;      // the matrix whose metadata ends the file
    uint32_t source_sha256, mlp_source_sha256;            // 65-byte strings (0 = absent)
    uint32_t gate_up_reference, mlp_reference, layer_reference;              // float[8] (0 = absent)
    uint32_t gate_up_reference_count, mlp_reference_count, layer_reference_count;  // uint32 (0 = absent)
    uint32_t constants_index[3];  // uint64 indices into the constants (0 = absent)
};

// qwen38_m3_image.h:26-94
const Layout kDelta = {
    {'Q', '3', '8', 'M', '3', 'Q', '4', '\0'}, 3, 5,
    284, 16, 20, 24, 304,
    {{56, 64, 72, 80}, {88, 96, 104, 112}, {120, 128, 136, 144}, {384, 392, 400, 408}, {416, 424, 432, 440}},
    {{20, 0}, {20, 0}, {40, 44}, {288, 292}, {296, 300}},
    320, 328, 4,
    152, 480,
    220, 252, 448,
    32, 48, 308,
};
// qwen38_m3_attention_image.h:21-72
const Layout kAttention = {
    {'Q', '3', '8', 'M', '3', 'A', 'T', 'T'}, 1, 5,
    16, 20, 24, 28, 64,
    {{72, 80, 88, 96}, {104, 112, 120, 128}, {136, 144, 152, 160}, {216, 224, 232, 240}, {248, 256, 264, 272}},
    {{24, 0}, {24, 0}, {0, 0}, {48, 52}, {56, 60}},
    168, 176, 4,
    280, 0,
    0, 0, 0,
    0, 0, 0,
};

// qwen38_m3_global_image.h:14-38: embedding and lm_head, both [vocab, hidden]; the file ends with the constants
const Layout kGlobal = {
    {'Q', '3', '8', 'M', '3', 'G', 'L', 'B'}, 1, 2,
    0, 20, 16, 24, 28,
    {{40, 48, 56, 64}, {72, 80, 88, 96}, {0, 0, 0, 0}, {0, 0, 0, 0}, {0, 0, 0, 0}},
    {{16, 0}, {16, 0}, {0, 0}, {0, 0}, {0, 0}},
    104, 112, 0xffffffffu,
    120, 185,
    0, 0, 0,
    0, 0, 0,
};

// qwen38_m3_mtp_image.h:21-51: the fused fc projection [hidden, 2 x hidden] and three norm vectors; the file
// ends with the constants
const Layout kMtp = {
    {'Q', '3', '8', 'M', '3', 'M', 'T', 'P'}, 1, 1,
    0, 16, 20, 28, 32,
    {{40, 48, 56, 64}, {0, 0, 0, 0}, {0, 0, 0, 0}, {0, 0, 0, 0}, {0, 0, 0, 0}},
    {{20, 24}, {0, 0}, {0, 0}, {0, 0}, {0, 0}},
    72, 80, 0xffffffffu,
    112, 0,
    0, 0, 0,
    0, 0, 0,
    {88, 96, 104},
};

const Layout &layout_of(int kind) {
    return kind == Q4B_IMAGE_DELTA ? kDelta : kind == Q4B_IMAGE_ATTENTION ? kAttention
           : kind == Q4B_IMAGE_GLOBAL ? kGlobal : kMtp;
}
const char *name_of(int kind) {
    return kind == Q4B_IMAGE_DELTA ? "DeltaNet" : kind == Q4B_IMAGE_ATTENTION ? "attention"
           : kind == Q4B_IMAGE_GLOBAL ? "global" : "MTP extras";
}

void set_message(char *message, size_t capacity, const char *format, ...) {
    if (message == nullptr || capacity == 0) return;
    va_list arguments;
    va_start(arguments, format);
    vsnprintf(message, capacity, format, arguments);
    va_end(arguments);
}

uint32_t read_u32(const unsigned char *base, uint32_t offset) {
    uint32_t value;
    memcpy(&value, base + offset, sizeof(value));
    return value;
}
uint64_t read_u64(const unsigned char *base, uint32_t offset) {
    uint64_t value;
    memcpy(&value, base + offset, sizeof(value));
    return value;
}

}  // namespace

struct q4b_image {
    int file;
    unsigned char *mapping;
    size_t length;
    const Layout *layout;
    q4b_image_info info;
    uint64_t quants_offset[5], meta_offset[5];
    uint64_t constants_offset;
};

extern "C" {

int q4b_image_open(const char *path, int kind, uint32_t layer_index, int check_27b_shapes,
                   const char *const *allowed_sha256, int allowed_count, q4b_image **image,
                   char *error_message, size_t error_capacity) {
    if (path == nullptr || image == nullptr ||
        (kind != Q4B_IMAGE_DELTA && kind != Q4B_IMAGE_ATTENTION && kind != Q4B_IMAGE_GLOBAL &&
         kind != Q4B_IMAGE_MTP)) {
        set_message(error_message, error_capacity, "path, kind or result pointer missing");
        return Q4B_BAD_ARGUMENT;
    }
    *image = nullptr;
    const Layout &layout = layout_of(kind);
    // map_file (qwen38_m3_decode.m:374-396): a regular file of at least one page, mapped read-only
    const int file = open(path, O_RDONLY);
    struct stat status;
    if (file < 0 || fstat(file, &status) != 0 || (uint64_t)status.st_size < kPage) {
        if (file >= 0) close(file);
        set_message(error_message, error_capacity, "cannot open %s", path);
        return Q4B_LOAD_FAILURE;
    }
    const size_t length = (size_t)status.st_size;
    void *mapping = mmap(nullptr, length, PROT_READ, MAP_PRIVATE, file, 0);
    if (mapping == MAP_FAILED) {
        close(file);
        set_message(error_message, error_capacity, "cannot map %s", path);
        return Q4B_LOAD_FAILURE;
    }
    const unsigned char *h = static_cast<const unsigned char *>(mapping);
    q4b_image *result = new (std::nothrow) q4b_image();
    if (result == nullptr) {
        munmap(mapping, length);
        close(file);
        return Q4B_LOAD_FAILURE;
    }
    result->file = file;
    result->mapping = static_cast<unsigned char *>(mapping);
    result->length = length;
    result->layout = &layout;
    q4b_image_info &info = result->info;
    memset(&info, 0, sizeof(info));

    const char *problem = nullptr;
    // validate_delta_header / validate_attention_header (:409-446)
    info.kind = (uint32_t)kind;
    info.version = read_u32(h, 8);
    info.layer_index = layout.layer_index != 0 ? read_u32(h, layout.layer_index) : 0;
    info.hidden_size = read_u32(h, layout.hidden_size);
    info.intermediate_size = read_u32(h, layout.intermediate_size);
    info.group_size = read_u32(h, layout.group_size);
    info.constants_f32_count = read_u32(h, layout.constants_count);
    if (memcmp(h, layout.magic, 8) != 0) problem = "wrong magic";
    else if (info.version != layout.version) problem = "wrong version";
    else if (read_u32(h, 12) != kPage) problem = "header is not one page";
    else if (info.group_size != 64) problem = "group size is not 64";
    else if (layout.layer_index != 0 && info.layer_index != layer_index)
        problem = "layer index differs from the one asked for";
    else if (kind == Q4B_IMAGE_DELTA && layer_index % 4 == 3) problem = "layers 3 mod 4 are attention layers";
    else if (kind == Q4B_IMAGE_ATTENTION && layer_index % 4 != 3 && layer_index != kMtpLayerIndex)
        problem = "only layers 3 mod 4 (and the MTP layer) are attention layers";
    else if (info.hidden_size == 0 || info.hidden_size % 64 != 0 || info.intermediate_size == 0 ||
             ((kind == Q4B_IMAGE_DELTA || kind == Q4B_IMAGE_ATTENTION) && info.intermediate_size % 64 != 0))
        problem = "hidden or intermediate size is not a positive multiple of 64";

    for (int m = 0; m < (int)layout.matrices && problem == nullptr; ++m) {
        // rows and groups: gate/up are [intermediate, hidden/64]; down of the attention image [hidden, intermediate/64]
        uint32_t rows = layout.shape[m].rows != 0 ? read_u32(h, layout.shape[m].rows) : info.hidden_size;
        uint32_t groups = layout.shape[m].groups != 0 ? read_u32(h, layout.shape[m].groups)
                          : m == Q4B_MATRIX_DOWN      ? info.intermediate_size / 64
                                                      : info.hidden_size / 64;
        info.rows[m] = rows;
        info.groups[m] = groups;
        const uint64_t q_offset = read_u64(h, layout.segment[m].quants_offset);
        const uint64_t q_bytes = read_u64(h, layout.segment[m].quants_bytes);
        const uint64_t m_offset = read_u64(h, layout.segment[m].meta_offset);
        const uint64_t m_bytes = read_u64(h, layout.segment[m].meta_bytes);
        result->quants_offset[m] = q_offset;
        result->meta_offset[m] = m_offset;
        // mapped_buffer (:398-407): page-aligned offsets and sizes
        if (((q_offset | q_bytes | m_offset | m_bytes) & (kPage - 1)) != 0) problem = "a segment is not page-aligned";
        else if (rows == 0 || groups == 0) problem = "a matrix has no rows or groups";
        else if (q_offset < kPage || q_offset > length || q_bytes > length - q_offset || m_offset < kPage ||
                 m_offset > length || m_bytes > length - m_offset)
            problem = "a segment lies outside the file";
        else if (q_bytes < (uint64_t)rows * groups * 32 || m_bytes < (uint64_t)rows * groups * 4)
            problem = "a segment is smaller than its matrix";
    }
    if (problem == nullptr) {
        const uint64_t c_offset = read_u64(h, layout.constants_offset), c_bytes = read_u64(h, layout.constants_bytes);
        result->constants_offset = c_offset;
        if (c_offset > length || c_bytes > length - c_offset || c_bytes < (uint64_t)info.constants_f32_count * 4)
            problem = "the constants lie outside the file";
        const uint32_t last = layout.last_segment;
        const uint64_t end = last == 0xffffffffu ? c_offset + c_bytes
                                                 : read_u64(h, layout.segment[last].meta_offset) +
                                                       read_u64(h, layout.segment[last].meta_bytes);
        if (problem == nullptr && end != length)
            problem = last == 0xffffffffu ? "the file does not end with the constants"
                                          : "the file does not end with the output metadata";
    }
    for (int i = 0; i < 3 && problem == nullptr && layout.constants_index[0] != 0; ++i) {
        // the three norm vectors of the MTP image, hidden_size floats each, by index into the constants
        info.constants_index[i] = read_u64(h, layout.constants_index[i]);
        if (info.constants_index[i] > info.constants_f32_count ||
            info.hidden_size > info.constants_f32_count - info.constants_index[i])
            problem = "a norm vector lies outside the constants";
    }
    if (problem == nullptr && check_27b_shapes && kind == Q4B_IMAGE_MTP) {
        // qwen38_m3_model_mtp_open (:2365-2375)
        if (info.hidden_size != 5120 || info.rows[0] != 5120 || info.groups[0] != 160 ||
            info.constants_f32_count != 3 * 5120)
            problem = "not the 27B fc projection and norm vectors";
    } else if (problem == nullptr && check_27b_shapes && kind == Q4B_IMAGE_GLOBAL) {
        // validate_global_header (:447-460)
        if (info.intermediate_size != 248320 || info.hidden_size != 5120 || info.constants_f32_count != 5120)
            problem = "not the 27B vocabulary and hidden size";
    } else if (problem == nullptr && check_27b_shapes) {
        // the shapes the reference runtime insists on (:412-421, :433-443)
        const bool delta = kind == Q4B_IMAGE_DELTA;
        const bool ok = info.hidden_size == 5120 && info.intermediate_size == 17408 &&
                        info.rows[Q4B_MATRIX_INPUT] == (delta ? 16480u : 14336u) && info.groups[Q4B_MATRIX_INPUT] == 80 &&
                        info.rows[Q4B_MATRIX_OUTPUT] == 5120 && info.groups[Q4B_MATRIX_OUTPUT] == 96 &&
                        info.constants_f32_count == (delta ? 51424u : 10752u) &&
                        (delta || (read_u32(h, 32) == 24 && read_u32(h, 36) == 4 && read_u32(h, 40) == 256 &&
                                   read_u32(h, 44) == 64));
        if (!ok) problem = "not the 27B layer shapes";
    }
    if (problem == nullptr) {
        memcpy(info.source_sha256, h + layout.source_sha256, 64);
        if (layout.mlp_source_sha256 != 0) memcpy(info.mlp_source_sha256, h + layout.mlp_source_sha256, 64);
        if (allowed_sha256 != nullptr) {  // pinned_sha: the digests the caller accepts
            auto allowed = [&](const char *digest) {
                for (int i = 0; i < allowed_count; ++i) {
                    if (allowed_sha256[i] != nullptr && strncmp(allowed_sha256[i], digest, 64) == 0) return true;
                }
                return false;
            };
            if (!allowed(info.source_sha256) ||
                (info.mlp_source_sha256[0] != '\0' && !allowed(info.mlp_source_sha256)))
                problem = "source digest is not one of the accepted ones";
        }
    }
    if (problem != nullptr) {
        set_message(error_message, error_capacity, "invalid %s image at layer %u: %s",
                    name_of(kind), layer_index, problem);
        q4b_image_close(result);
        return Q4B_LOAD_FAILURE;
    }
    if (layout.gate_up_reference != 0) {
        memcpy(info.gate_up_reference_first_8, h + layout.gate_up_reference, 32);
        memcpy(info.mlp_reference_first_8, h + layout.mlp_reference, 32);
        memcpy(info.layer_reference_first_8, h + layout.layer_reference, 32);
        info.reference_counts[0] = read_u32(h, layout.gate_up_reference_count);
        info.reference_counts[1] = read_u32(h, layout.mlp_reference_count);
        info.reference_counts[2] = read_u32(h, layout.layer_reference_count);
    }
    *image = result;
    return Q4B_OK;
}

int q4b_image_describe(const q4b_image *image, q4b_image_info *info) {
    if (image == nullptr || info == nullptr) return Q4B_BAD_ARGUMENT;
    *info = image->info;
    return Q4B_OK;
}

const float *q4b_image_constants(const q4b_image *image, uint32_t *count) {
    if (image == nullptr) return nullptr;
    if (count != nullptr) *count = image->info.constants_f32_count;
    return reinterpret_cast<const float *>(image->mapping + image->constants_offset);
}

int q4b_image_segments(const q4b_image *image, int matrix, const void **quants, const void **metadata) {
    if (image == nullptr || matrix < 0 || matrix >= (int)image->layout->matrices || quants == nullptr ||
        metadata == nullptr) {
        return Q4B_BAD_ARGUMENT;
    }
    *quants = image->mapping + image->quants_offset[matrix];
    *metadata = image->mapping + image->meta_offset[matrix];
    return Q4B_OK;
}

int q4b_image_weight(q4b_context *context, const q4b_image *image, int matrix, uint32_t row_begin,
                     uint32_t row_count, q4b_weight **weight, char *error_message, size_t error_capacity) {
    if (image == nullptr || matrix < 0 || matrix >= (int)image->layout->matrices) {
        set_message(error_message, error_capacity, "no image or no such matrix");
        return Q4B_BAD_ARGUMENT;
    }
    return q4b_weight_upload(context, image->mapping + image->quants_offset[matrix],
                             image->mapping + image->meta_offset[matrix], image->info.rows[matrix],
                             image->info.groups[matrix], row_begin, row_count, weight, error_message, error_capacity);
}

void q4b_image_close(q4b_image *image) {
    if (image == nullptr) return;
    if (image->mapping != nullptr) munmap(image->mapping, image->length);
    if (image->file >= 0) close(image->file);
    delete image;
}

}  // extern "C"
