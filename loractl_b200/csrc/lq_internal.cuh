// Internal declarations shared by the translation units of libloractl_b200.
//
// Packed layouts (device-resident, tile-contiguous so one bulk copy fetches a tile):
//
//   int4: tiles of 128 rows x 64 k.  Tile (mt, kt) starts at byte
//         (mt * k_tiles + kt) * 4096 and is a row-major [128][8] array of u32; each
//         u32 holds 8 consecutive k of one row as offset-binary nibbles (q + 8).
//         Element e (0..7) of the word sits at nibble (e >> 1) + 4 * (e & 1), so that
//         `(word >> 4j) & 0x000F000F` yields the register-adjacent pair (2j, 2j+1).
//   int8: same tiling, tile = row-major [128][64] int8 (8192 bytes).
//   scales (int4/int8): f32, [m_tiles][n_groups][128]: the 128 row scales of one
//         (m-tile, k-group) are contiguous.  Padding rows / k have code 0, scale 0.
//   fp8:  the file's row-major [M][K] e4m3fn bytes, untouched (TMA-tileable as is);
//         scales f32 [1] or [M].
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <stdexcept>
#include <string>

#include "../../include/loractl_b200.h"

#define LQ_TILE_M 128
#define LQ_TILE_K 64

struct lq_weight {
    int device = 0;
    int scheme = LQ_INT4;
    int group = 0;
    int scale_kind = LQ_SCALE_SCALAR;
    int64_t M = 0, K = 0;
    int64_t m_tiles = 0, k_tiles = 0, n_groups = 0;
    void* packed = nullptr;
    float* scales = nullptr;
    float* bias = nullptr;
    size_t packed_bytes = 0, scale_bytes = 0;
    void* packed_t = nullptr;  // fp8 only: the bytes transposed to [d_in, d_out], built on first use
    const void* bf16_copy = nullptr;  // optional caller-owned bf16 [d_out, d_in] copy of the dequantised weight
};

// Device-side view passed to kernels by value.
struct LqWView {
    const void* packed;
    const float* scales;
    int64_t M, K, k_tiles, n_groups;
    int scheme, group, scale_kind;
};

struct LqError : std::runtime_error {
    int status;
    LqError(int st, const std::string& m) : std::runtime_error(m), status(st) {}
};

#define LQ_CHECK_ARG(cond, msg)                                   \
    do {                                                          \
        if (!(cond)) throw LqError(LQ_ERR_INVALID, std::string(msg)); \
    } while (0)

#define LQ_CUDA(expr)                                                                         \
    do {                                                                                      \
        cudaError_t _e = (expr);                                                              \
        if (_e != cudaSuccess)                                                                \
            throw LqError(LQ_ERR_CUDA, std::string(#expr) + ": " + cudaGetErrorString(_e));   \
    } while (0)

inline LqWView lq_view(const lq_weight* w) {
    LqWView v;
    v.packed = w->packed;
    v.scales = w->scales;
    v.M = w->M;
    v.K = w->K;
    v.k_tiles = w->k_tiles;
    v.n_groups = w->n_groups;
    v.scheme = w->scheme;
    v.group = w->group;
    v.scale_kind = w->scale_kind;
    return v;
}

// ---- device helpers ------------------------------------------------------------

__host__ __device__ inline float lq_decode_e4m3fn(uint32_t b) {
    // crates/loractl-core/src/fp8.rs:45-56: bias 7, 3 mantissa bits, no inf, NaN at 0x7f/0xff.
    uint32_t sign = (b & 0x80u) << 24;
    uint32_t exp = (b >> 3) & 0xFu;
    uint32_t man = b & 0x7u;
    uint32_t bits;
    if (exp == 0xFu && man == 0x7u) {
        bits = 0x7FC00000u;
    } else if (exp == 0) {
        // subnormal: man / 8 * 2^-6 = man * 2^-9 (exact in f32)
        float v = (float)man * 0.001953125f;
#ifdef __CUDA_ARCH__
        bits = __float_as_uint(v);
#else
        union { float f; uint32_t u; } cv; cv.f = v; bits = cv.u;
#endif
    } else {
        bits = ((exp + 120u) << 23) | (man << 20);
    }
    bits |= sign;
#ifdef __CUDA_ARCH__
    return __uint_as_float(bits);
#else
    union { float f; uint32_t u; } cv; cv.u = bits; return cv.f;
#endif
}

// Dequantized value of logical element (m, k): `q * scale` in f32 (burn-ndarray
// `dequantize_one`) or `LUT[b] * scale` (crates/loractl-core/src/fp8.rs:305-317).
__device__ __forceinline__ float lq_dequant_elem(const LqWView& w, int64_t m, int64_t k) {
    if (w.scheme == LQ_FP8_E4M3) {
        uint32_t b = ((const uint8_t*)w.packed)[m * w.K + k];
        float s = w.scale_kind == LQ_SCALE_PER_CHANNEL ? w.scales[m] : w.scales[0];
        return lq_decode_e4m3fn(b) * s;
    }
    int64_t mt = m >> 7, r = m & 127, kt = k >> 6, kk = k & 63;
    float s = w.scales[(mt * w.n_groups + k / w.group) * 128 + r];
    int q;
    if (w.scheme == LQ_INT4) {
        const uint32_t* tile = (const uint32_t*)w.packed + (mt * w.k_tiles + kt) * 1024;
        uint32_t word = tile[r * 8 + (kk >> 3)];
        int e = (int)(kk & 7);
        int pos = (e >> 1) + 4 * (e & 1);
        q = (int)((word >> (4 * pos)) & 0xFu) - 8;
    } else {
        const int8_t* tile = (const int8_t*)w.packed + (mt * w.k_tiles + kt) * 8192;
        q = tile[r * 64 + kk];
    }
    return (float)q * s;
}

// ---- kernel launchers (defined in the .cu files) ---------------------------------

void lq_launch_quantize(const void* w, int w_dtype, const lq_weight* dst, int bits, cudaStream_t st);
void lq_launch_quantize_fp8(const uint8_t* bytes, const float* scale, int per_channel, const lq_weight* dst, int bits,
                            cudaStream_t st);
void lq_launch_pack_codes(const int8_t* codes, const float* scales, const lq_weight* dst, cudaStream_t st);
void lq_launch_unpack(const lq_weight* w, int8_t* codes, float* scales, cudaStream_t st);
// out[m * ld + k] (transpose = 0) or out[k * ld + m] (transpose = 1), dtype f32/bf16.
void lq_launch_dequant(const lq_weight* w, void* out, int out_dtype, int64_t ld, int transpose, cudaStream_t st);
void lq_launch_fp8_quantize(const float* w, int64_t M, int64_t K, int per_channel, uint8_t* bytes,
                            float* scales, cudaStream_t st);

// Generic SIMT f32 GEMM:  C[i,j] = alpha * sum_k A(i,k) * B(k,j) + (beta ? C[i,j] : 0) + bias[j]
//   A(i,k) = A[i * sa_i + k * sa_k]  (element type a_dtype)
//   B(k,j): b_mode 0 -> Bp[k * sb_k + j * sb_j] (element type b_dtype); 1 -> dequant(W)[m = j, k];
//           2 -> dequant(W)[m = k, j]
struct LqSimtArgs {
    const void* A; int a_dtype; int64_t sa_i, sa_k;
    int b_mode; const void* Bp; int b_dtype; int64_t sb_k, sb_j; LqWView W;
    void* C; int c_dtype; int64_t ldc;
    const float* bias;
    int64_t I, J, Kred;
    float alpha; int beta;
};
void lq_launch_simt_gemm(const LqSimtArgs& a, cudaStream_t st);

// Sets the calling thread's lq_last_error() text (empty string clears it).
void lq_set_last_error(const std::string& msg);
