/* CPU restatement, in plain C, of the arithmetic behind izwi-core's Linear /
 * QMatMul call sites.  TEST INFRASTRUCTURE ONLY: it is the checker and the
 * timed CPU baseline, never part of the shipped path.
 *
 * The reference delegates this arithmetic to un-vendored crates (candle-core
 * 0.10.2 with the `gemm` 0.18.2/0.19.0 CPU GEMM), so the functions follow the
 * reference call sites and the published GGML block formats:
 *   - orc_linear_f32:  Linear::forward, Y = X.W^T (+b), W is [N,K]
 *       (crates/izwi-core/src/models/architectures/qwen3/core.rs:794,975,1163)
 *   - orc_dequantize_q8_0 / orc_dequantize_q4_k: QTensor::dequantize
 *       (call sites qwen3/core.rs:853-858, models/shared/weights/gguf.rs:131)
 *   - orc_qlinear_f32:  QMatMul::forward stated as dequant(W).X
 *       (call site qwen3/core.rs:812)
 *   - orc_silu_mul_f32: try_fused_silu_mul (kernels/cuda.rs:51-62; formula
 *       kernels/metal.rs:39-40)
 * Pinned against gguf-py 0.19.0 dequantisation through the NumPy oracle's
 * golden vectors; GEMM numerics themselves are "parity unpinned".
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

static float half_to_float(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {
            int e = -1;
            do { e++; man <<= 1; } while ((man & 0x400u) == 0);
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3FFu) << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((exp + 112u) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

int orc_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* Size of the OpenMP team used by the functions below (a launcher may have exported
 * OMP_NUM_THREADS=1; the timed baseline sets the count it reports). */
void orc_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* One Q8_0 block: fp16 d then 32 int8; value = d*q. */
static void dequant_row_q8_0(const uint8_t *row, int64_t k, float *out) {
    for (int64_t b = 0; b < k / 32; ++b) {
        const uint8_t *blk = row + b * 34;
        uint16_t dh;
        memcpy(&dh, blk, 2);
        float d = half_to_float(dh);
        const int8_t *q = (const int8_t *)(blk + 2);
        for (int i = 0; i < 32; ++i) out[b * 32 + i] = d * (float)q[i];
    }
}

/* One Q4_K super-block: fp16 d, fp16 dmin, 12 scale bytes, 128 code bytes. */
static void dequant_row_q4_k(const uint8_t *row, int64_t k, float *out) {
    for (int64_t b = 0; b < k / 256; ++b) {
        const uint8_t *blk = row + b * 144;
        uint16_t dh, mh;
        memcpy(&dh, blk, 2);
        memcpy(&mh, blk + 2, 2);
        const float d = half_to_float(dh), dmin = half_to_float(mh);
        const uint8_t *s = blk + 4, *qs = blk + 16;
        float *y = out + b * 256;
        for (int j = 0; j < 8; ++j) {
            uint8_t sc, mn;
            if (j < 4) {
                sc = s[j] & 63;
                mn = s[j + 4] & 63;
            } else {
                sc = (uint8_t)((s[j + 4] & 0x0F) | ((s[j - 4] >> 6) << 4));
                mn = (uint8_t)((s[j + 4] >> 4) | ((s[j] >> 6) << 4));
            }
            volatile float dsc = d * (float)sc; /* volatile: keep the three */
            volatile float dm = dmin * (float)mn; /* roundings separate      */
            const uint8_t *g = qs + 32 * (j / 2);
            for (int i = 0; i < 32; ++i) {
                int q = (j & 1) ? (g[i] >> 4) : (g[i] & 0x0F);
                volatile float p = dsc * (float)q;
                y[j * 32 + i] = p - dm;
            }
        }
    }
}

void orc_dequantize_q8_0(const uint8_t *raw, int64_t n_elems, float *out) {
    dequant_row_q8_0(raw, n_elems, out);
}

void orc_dequantize_q4_k(const uint8_t *raw, int64_t n_elems, float *out) {
    dequant_row_q4_k(raw, n_elems, out);
}

static float dot_f32(const float *a, const float *b, int64_t k) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    int64_t i = 0;
    for (; i + 8 <= k; i += 8)
        for (int j = 0; j < 8; ++j) acc[j] += a[i + j] * b[i + j];
    float s = 0.f;
    for (; i < k; ++i) s += a[i] * b[i];
    for (int j = 0; j < 8; ++j) s += acc[j];
    return s;
}

/* Y[M,N] = X[M,K] . W[N,K]^T (+ b[N]); rows of W split over the host threads. */
void orc_linear_f32(const float *x, const float *w, const float *bias, float *y,
                    int64_t m, int64_t n, int64_t k) {
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < n; ++r) {
        const float *wr = w + r * k;
        for (int64_t t = 0; t < m; ++t) {
            float v = dot_f32(x + t * k, wr, k);
            y[t * n + r] = bias ? v + bias[r] : v;
        }
    }
}

/* fmt: 0 = Q8_0, 1 = Q4_K.  Each weight row is dequantised once into a
 * per-thread fp32 buffer and then dotted with every activation row. */
int orc_qlinear_f32(int fmt, const float *x, const uint8_t *raw, float *y,
                    int64_t m, int64_t n, int64_t k) {
    const int64_t row_bytes = fmt == 0 ? k / 32 * 34 : k / 256 * 144;
    if ((fmt == 0 && k % 32) || (fmt == 1 && k % 256) || fmt < 0 || fmt > 1) return -1;
#pragma omp parallel
    {
        float *buf = (float *)malloc((size_t)k * sizeof(float));
#pragma omp for schedule(static)
        for (int64_t r = 0; r < n; ++r) {
            if (fmt == 0) dequant_row_q8_0(raw + r * row_bytes, k, buf);
            else dequant_row_q4_k(raw + r * row_bytes, k, buf);
            for (int64_t t = 0; t < m; ++t) y[t * n + r] = dot_f32(x + t * k, buf, k);
        }
        free(buf);
    }
    return 0;
}

void orc_silu_mul_f32(const float *gate, const float *up, float *out, int64_t n) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) out[i] = gate[i] / (1.0f + expf(-gate[i])) * up[i];
}
