/*
 * CPU oracle for the quantized frozen-base LoRA linear — plain C restatement.
 *
 * TEST INFRASTRUCTURE ONLY: the checker the CUDA path is compared against and the timed CPU
 * baseline of bench.py.  Nothing in the shipped library links or calls it.
 *
 * Each function cites the loractl item it follows (paths relative to the loractl repository
 * root).  The quantize arithmetic itself is burn-ndarray 0.21.0's (not part of the loractl
 * tree): per block absmax, scale = 2*absmax/(b-a), q = clamp(round(w/scale)), dq = q*scale,
 * f32 throughout, `round` = Rust f32::round = C roundf (half away from zero).
 *
 * Pinned through tests/test_oracle_c.py against the numpy oracle, which is itself pinned to the
 * reference's golden vectors (quant_int4/int8_golden.json, fp8_*_golden.json, lora_toy.json).
 * Parity unpinned: exact .5 ties, all-zero groups (scale 0, q 0 here), block 64, backward.
 *
 * Build: gcc -O2 -fno-fast-math -ffp-contract=off -shared -fPIC (see oracle/build.py).
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* reference/quant_int4_reference.py:46-58, reference/quant_reference.py:40-52,
 * crates/loractl-core/src/quant.rs:61-82.  Returns 1 when d_in % group != 0 (the reference
 * asserts, quant.rs:76-80). */
int lqo_quantize(const float* w, int64_t m, int64_t k, int group, int bits, int8_t* codes, float* scales) {
    if (group <= 0 || k % group != 0 || (bits != 4 && bits != 8)) return 1;
    const float qmax = bits == 4 ? 7.0f : 127.0f;
    const int64_t ng = k / group;
    for (int64_t i = 0; i < m; ++i)
        for (int64_t g = 0; g < ng; ++g) {
            const float* blk = w + i * k + g * group;
            float absmax = 0.0f;
            for (int e = 0; e < group; ++e) {
                float a = fabsf(blk[e]);
                if (a > absmax) absmax = a;
            }
            float scale = absmax / qmax;
            scales[i * ng + g] = scale;
            for (int e = 0; e < group; ++e) {
                float q = 0.0f;
                if (scale > 0.0f) {
                    q = roundf(blk[e] / scale);
                    if (q > qmax) q = qmax;
                    if (q < -qmax) q = -qmax;
                }
                codes[i * k + g * group + e] = (int8_t)q;
            }
        }
    return 0;
}

/* burn-ndarray `dequantize_one`: q * scale. */
void lqo_dequantize(const int8_t* codes, const float* scales, int64_t m, int64_t k, int group, float* out) {
    const int64_t ng = k / group;
    for (int64_t i = 0; i < m; ++i)
        for (int64_t j = 0; j < k; ++j) out[i * k + j] = (float)codes[i * k + j] * scales[i * ng + j / group];
}

/* crates/loractl-core/src/quant.rs:102-117.  Returns the chunk count; writes at most cap rows. */
size_t lqo_dequant_chunk_rows(uint64_t d_out, uint64_t d_in, uint64_t chunk_bytes, uint64_t* rows, size_t cap) {
    uint64_t full = d_out * d_in * 4;
    if (chunk_bytes == 0 || full <= chunk_bytes || d_out <= 1) {
        if (cap > 0) rows[0] = d_out;
        return 1;
    }
    uint64_t row_bytes = d_in * 4, max_rows = chunk_bytes / row_bytes;
    if (max_rows < 1) max_rows = 1;
    uint64_t n = (d_out + max_rows - 1) / max_rows, base = d_out / n, rem = d_out % n;
    for (uint64_t i = 0; i < n && i < cap; ++i) rows[i] = i < rem ? base + 1 : base;
    return (size_t)n;
}

/* crates/loractl-core/src/fp8.rs:45-56. */
float lqo_decode_e4m3fn(uint8_t byte) {
    float sign = (byte & 0x80) ? -1.0f : 1.0f;
    int exp = (byte >> 3) & 0x0f;
    float man = (float)(byte & 0x07);
    if (exp == 0x0f && (byte & 0x07) == 0x07) return NAN;
    if (exp == 0) return sign * (man / 8.0f) * exp2f(-6.0f);
    return sign * (1.0f + man / 8.0f) * exp2f((float)exp - 7.0f);
}

/* crates/loractl-core/src/fp8.rs:305-317: LUT[byte] * scale, scalar (n_scale == 1) or per row. */
void lqo_fp8_dequant(const uint8_t* bytes, const float* scale, int64_t n_scale, int64_t m, int64_t k, float* out) {
    for (int64_t i = 0; i < m; ++i)
        for (int64_t j = 0; j < k; ++j)
            out[i * k + j] = lqo_decode_e4m3fn(bytes[i * k + j]) * (n_scale == 1 ? scale[0] : scale[i]);
}

/* out[i,j] (+)= alpha * sum_p a(i,p) * b(p,j) with arbitrary strides: the "stock matmul" every step
 * of the reference's sequence reduces to (ndarray -> matrixmultiply sgemm, single-threaded).
 * Cache-blocked i-p-j loops; j innermost is contiguous when sb_j == 1. */
static void gemm(int64_t I, int64_t J, int64_t P, float alpha, const float* a, int64_t sa_i, int64_t sa_p,
                 const float* b, int64_t sb_p, int64_t sb_j, float* c, int64_t ldc, int accumulate) {
    if (!accumulate)
        for (int64_t i = 0; i < I; ++i) memset(c + i * ldc, 0, sizeof(float) * (size_t)J);
    const int64_t BI = 64, BP = 256, BJ = 512;
    for (int64_t j0 = 0; j0 < J; j0 += BJ)
        for (int64_t p0 = 0; p0 < P; p0 += BP)
            for (int64_t i0 = 0; i0 < I; i0 += BI) {
                int64_t j1 = j0 + BJ < J ? j0 + BJ : J, p1 = p0 + BP < P ? p0 + BP : P, i1 = i0 + BI < I ? i0 + BI : I;
                for (int64_t i = i0; i < i1; ++i)
                    for (int64_t p = p0; p < p1; ++p) {
                        float av = alpha * a[i * sa_i + p * sa_p];
                        float* cr = c + i * ldc;
                        const float* br = b + p * sb_p;
                        if (sb_j == 1)
                            for (int64_t j = j0; j < j1; ++j) cr[j] += av * br[j];
                        else
                            for (int64_t j = j0; j < j1; ++j) cr[j] += av * br[j * sb_j];
                    }
            }
}

/* Forward of one LoRA'd quantized site, the reference's op sequence
 * (crates/loractl-core/src/quant.rs:250-251, mmdit.rs:512-514, lora.rs:199-203):
 *   dq = dequantize(wq)  [full f32 M x K, every call];  y = x . dq^T + bias;  h = x . a;
 *   y += s * (h . b).
 * `dq_scratch` is [M,K], `h` is [N,r]. */
void lqo_lora_linear_fwd(const float* x, int64_t n, const int8_t* codes, const float* scales, int group, int64_t m,
                         int64_t k, const float* bias, const float* a, const float* b, int r, float s, float* y,
                         float* h, float* dq_scratch) {
    lqo_dequantize(codes, scales, m, k, group, dq_scratch);
    gemm(n, m, k, 1.0f, x, k, 1, dq_scratch, 1, k, y, m, 0);
    if (bias)
        for (int64_t i = 0; i < n; ++i)
            for (int64_t j = 0; j < m; ++j) y[i * m + j] += bias[j];
    if (r > 0) {
        gemm(n, r, k, 1.0f, x, k, 1, a, r, 1, h, r, 0);
        gemm(n, m, r, s, h, r, 1, b, m, 1, y, m, 1);
    }
}

/* Backward (crates/loractl-core/src/quant.rs:229-234; reference/lora_reference.py:103-123):
 *   dq = dequantize(wq) again;  dx = dy . dq;  dh = s * dy . b^T;  db = s * h^T . dy;
 *   da = x^T . dh;  dx += dh . a^T.   `dh` is [N,r] scratch. */
void lqo_lora_linear_bwd(const float* dy, const float* x, const float* h, int64_t n, const int8_t* codes,
                         const float* scales, int group, int64_t m, int64_t k, const float* a, const float* b, int r,
                         float s, float* dx, float* da, float* db, float* dh, float* dq_scratch) {
    lqo_dequantize(codes, scales, m, k, group, dq_scratch);
    gemm(n, k, m, 1.0f, dy, m, 1, dq_scratch, k, 1, dx, k, 0);
    if (r > 0) {
        gemm(n, r, m, s, dy, m, 1, b, 1, m, dh, r, 0);
        gemm(r, m, n, s, h, 1, r, dy, m, 1, db, m, 0);
        gemm(k, r, n, 1.0f, x, 1, k, dh, r, 1, da, r, 0);
        gemm(n, k, r, 1.0f, dh, r, 1, a, 1, r, dx, k, 1);
    }
}
