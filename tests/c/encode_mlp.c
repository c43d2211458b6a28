/* The binding a maintainer of the reference's C runtime would write for the decode MLP (encode_mlp,
 * models/qwen3.8-27b/targets/apple-m3-pro/qwen38_m3_decode.m:639-660): plain C11, q4b200.h, nothing else.
 * Loads a synthetic layer (seeded generator of the library, so that the Python test can regenerate the same
 * weights on the CPU), runs gate/up + SiLU and down + residual on `batch` activation rows and writes the two
 * results to a file as raw little-endian floats.
 *
 *   encode_mlp <hidden> <intermediate> <batch> <seed> <out-file>
 */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "q4b200.h"

typedef struct {
    q4b_context *gpu;
    q4b_weight *gate, *up, *down;
    unsigned hidden, intermediate;
} b200_layer;

static int b200_encode_mlp(b200_layer *layer, const void *normed_f16, const void *hidden_f32,
                           void *activated_f16, void *hidden_out_f32, unsigned batch, char *err, size_t cap) {
    /* qwen38_q4_gate_up_silu: silu(gate x) * (up x), one read of x */
    int status = q4b_gate_up_silu(layer->gpu, layer->gate, layer->up, normed_f16, Q4B_F16, batch, activated_f16,
                                  Q4B_F16, layer->intermediate, err, cap);
    if (status != Q4B_OK) return status;
    /* qwen38_q4_mlp_down_residual_f32: down(activated) + residual, fp32 out */
    return q4b_matmul(layer->gpu, layer->down, activated_f16, Q4B_F16, batch, hidden_out_f32, Q4B_F32,
                      layer->hidden, hidden_f32, Q4B_F32, layer->hidden, err, cap);
}

#define CHECK(call)                                                     \
    do {                                                                \
        int status_ = (call);                                           \
        if (status_ != Q4B_OK) {                                        \
            fprintf(stderr, "%s: status %d: %s\n", #call, status_, err); \
            return 1;                                                   \
        }                                                               \
    } while (0)

int main(int argc, char **argv) {
    if (argc != 6) {
        fprintf(stderr, "usage: %s hidden intermediate batch seed out-file\n", argv[0]);
        return 2;
    }
    const unsigned hidden = (unsigned)atoi(argv[1]), intermediate = (unsigned)atoi(argv[2]);
    const unsigned batch = (unsigned)atoi(argv[3]);
    const uint64_t seed = (uint64_t)atoll(argv[4]);
    char err[512] = "";
    b200_layer layer = {0};
    layer.hidden = hidden;
    layer.intermediate = intermediate;
    layer.gpu = q4b_context_open(0, err, sizeof err);
    if (layer.gpu == NULL) {
        fprintf(stderr, "no context: %s\n", err);
        return 1;
    }
    /* projections 0, 1, 2 of the seed: gate, up [intermediate, hidden]; down [hidden, intermediate] */
    CHECK(q4b_weight_synth(layer.gpu, seed, 0, intermediate, hidden / 64, 0, intermediate, &layer.gate, err, sizeof err));
    CHECK(q4b_weight_synth(layer.gpu, seed, 1, intermediate, hidden / 64, 0, intermediate, &layer.up, err, sizeof err));
    CHECK(q4b_weight_synth(layer.gpu, seed, 2, hidden, intermediate / 64, 0, hidden, &layer.down, err, sizeof err));

    void *normed = NULL, *residual_f16 = NULL, *residual = NULL, *activated = NULL, *out = NULL;
    CHECK(q4b_alloc(layer.gpu, (size_t)batch * hidden * 2, &normed, err, sizeof err));
    CHECK(q4b_alloc(layer.gpu, (size_t)batch * hidden * 2, &residual_f16, err, sizeof err));
    CHECK(q4b_alloc(layer.gpu, (size_t)batch * hidden * 4, &residual, err, sizeof err));
    CHECK(q4b_alloc(layer.gpu, (size_t)batch * intermediate * 2, &activated, err, sizeof err));
    CHECK(q4b_alloc(layer.gpu, (size_t)batch * hidden * 4, &out, err, sizeof err));
    CHECK(q4b_synth_x(layer.gpu, seed, 0, normed, 0, (uint64_t)batch * hidden, err, sizeof err));
    CHECK(q4b_synth_x(layer.gpu, seed, 1, residual_f16, 0, (uint64_t)batch * hidden, err, sizeof err));

    /* the residual stream is fp32 in the reference: widen the seeded fp16 values on the host */
    uint16_t *halves = malloc((size_t)batch * hidden * 2);
    float *wide = malloc((size_t)batch * hidden * 4);
    float *result = malloc((size_t)batch * hidden * 4);
    uint16_t *middle = malloc((size_t)batch * intermediate * 2);
    if (halves == NULL || wide == NULL || result == NULL || middle == NULL) return 1;
    CHECK(q4b_copy_to_host(layer.gpu, halves, residual_f16, (size_t)batch * hidden * 2, err, sizeof err));
    CHECK(q4b_sync(layer.gpu, NULL, err, sizeof err));
    for (size_t i = 0; i < (size_t)batch * hidden; ++i) {
        const uint32_t h = halves[i], sign = (h & 0x8000u) << 16, exponent = (h >> 10) & 31u, mantissa = h & 1023u;
        uint32_t bits;
        if (exponent == 0) {  /* zero or subnormal */
            float value = (float)mantissa * (1.0f / 16777216.0f);
            memcpy(&bits, &value, 4);
            bits |= sign;
        } else {
            bits = sign | ((exponent + 112u) << 23) | (mantissa << 13);
        }
        memcpy(&wide[i], &bits, 4);
    }
    CHECK(q4b_copy_to_device(layer.gpu, residual, wide, (size_t)batch * hidden * 4, err, sizeof err));

    CHECK(b200_encode_mlp(&layer, normed, residual, activated, out, batch, err, sizeof err));
    CHECK(q4b_copy_to_host(layer.gpu, middle, activated, (size_t)batch * intermediate * 2, err, sizeof err));
    CHECK(q4b_copy_to_host(layer.gpu, result, out, (size_t)batch * hidden * 4, err, sizeof err));
    CHECK(q4b_sync(layer.gpu, NULL, err, sizeof err));

    FILE *file = fopen(argv[5], "wb");
    if (file == NULL) return 1;
    fwrite(middle, 2, (size_t)batch * intermediate, file);
    fwrite(result, 4, (size_t)batch * hidden, file);
    fclose(file);
    printf("encode_mlp ok: hidden %u intermediate %u batch %u, %llu kernel launches\n", hidden, intermediate, batch,
           (unsigned long long)q4b_context_launch_count(layer.gpu));

    q4b_free(layer.gpu, normed);
    q4b_free(layer.gpu, residual_f16);
    q4b_free(layer.gpu, residual);
    q4b_free(layer.gpu, activated);
    q4b_free(layer.gpu, out);
    q4b_weight_free(layer.gpu, layer.gate);
    q4b_weight_free(layer.gpu, layer.up);
    q4b_weight_free(layer.gpu, layer.down);
    q4b_context_close(layer.gpu);
    free(halves);
    free(wide);
    free(result);
    free(middle);
    return 0;
}
