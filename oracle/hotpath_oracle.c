/* Plain-C restatement of the hot-path arithmetic (TEST INFRASTRUCTURE ONLY — never linked into the product).
 *
 *  oracle_wkv7      : the recurrence of the reference CUDA kernel, one (sequence, head, row) at a time
 *                     (reference/cuda/rwkv7_state_fwd_fp16.cu:12-55). Inputs are the fp16 tensors widened
 *                     to float by the caller; y is returned unrounded.
 *  oracle_gemv_int8 : y = W x for int8 rows with one fp32 scale per output row (build-defined format).
 *  oracle_gemv_nvfp4: y = W x for packed e2m1 pairs, one e4m3 scale per 16 inputs, fp32 tensor scale,
 *                     decoding both 8-bit and 4-bit codes bit by bit.
 *
 * Parity: the WKV loop is pinned indirectly (it must agree with the torch restatement, which is pinned
 * against the reference's single-token path); the two quantised products are unpinned: the reference
 * has no quantiser.
 */
#include <math.h>
#include <stdint.h>

void oracle_wkv7(int B, int T, int C, int H, float* state, const float* r, const float* w, const float* k,
                 const float* v, const float* a, const float* b, float* y) {
    const int N = 64;
    for (int bb = 0; bb < B; ++bb)
        for (int h = 0; h < H; ++h)
            for (int i = 0; i < N; ++i) {
                float* s = state + (long)bb * C * N + (long)h * N * N + (long)i * N;
                for (int t = 0; t < T; ++t) {
                    const long base = (long)bb * T * C + (long)t * C + h * N;
                    float sa = 0.f;
                    for (int j = 0; j < N; ++j) sa += a[base + j] * s[j];
                    const float vv = v[base + i];
                    float acc = 0.f;
                    for (int j = 0; j < N; ++j) {
                        const float dec = expf(-expf(w[base + j]));
                        s[j] = s[j] * dec + k[base + j] * vv + sa * b[base + j];
                        acc += s[j] * r[base + j];
                    }
                    y[base + i] = acc;
                }
            }
}

void oracle_gemv_int8(int n_out, int k, const int8_t* q, const float* row_scale, const float* x, double* y) {
    for (int o = 0; o < n_out; ++o) {
        double acc = 0.0;
        for (int i = 0; i < k; ++i) acc += (double)((float)q[(long)o * k + i] * row_scale[o]) * (double)x[i];
        y[o] = acc;
    }
}

static float e4m3_value(uint8_t c) {
    const int e = (c >> 3) & 15, m = c & 7;
    const float mag = e == 0 ? (float)m * 0.001953125f : (1.0f + (float)m / 8.0f) * ldexpf(1.0f, e - 7);
    return (c & 0x80) ? -mag : mag;
}
static float e2m1_value(uint8_t c) {
    static const float tab[8] = {0.f, 0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
    return (c & 8) ? -tab[c & 7] : tab[c & 7];
}

void oracle_dequant_nvfp4(int n_out, int k, const uint8_t* packed, const uint8_t* sb, float t, float* out) {
    for (int o = 0; o < n_out; ++o)
        for (int i = 0; i < k; ++i) {
            const uint8_t byte = packed[(long)o * (k / 2) + i / 2];
            const uint8_t code = (i & 1) ? (byte >> 4) : (byte & 15);
            const float s = e4m3_value(sb[(long)o * (k / 16) + i / 16]);
            out[(long)o * k + i] = (e2m1_value(code) * s) * t;
        }
}

void oracle_gemv_nvfp4(int n_out, int k, const uint8_t* packed, const uint8_t* sb, float t, const float* x, double* y) {
    for (int o = 0; o < n_out; ++o) {
        double acc = 0.0;
        for (int i = 0; i < k; ++i) {
            const uint8_t byte = packed[(long)o * (k / 2) + i / 2];
            const uint8_t code = (i & 1) ? (byte >> 4) : (byte & 15);
            const float s = e4m3_value(sb[(long)o * (k / 16) + i / 16]);
            acc += (double)((e2m1_value(code) * s) * t) * (double)x[i];
        }
        y[o] = acc;
    }
}
