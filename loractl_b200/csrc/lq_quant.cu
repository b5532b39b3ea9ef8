// Quantize / pack / unpack / dequantize kernels (HBM-bound, load-time and scratch paths).
//
// Arithmetic follows burn-ndarray 0.21's symmetric per-block scheme as pinned by
// reference/quant_int4_reference.py:46-58 and reference/quant_reference.py:40-52:
//   scale = absmax / qmax            (f32, IEEE division)
//   q     = clamp(round(w / scale))  (f32 division, round half away from zero)
// An all-zero block gets scale 0 and codes 0.
#include <cstdlib>
#include <cuda_fp8.h>

#include "lq_internal.cuh"
#include "lq_prof.cuh"

namespace {

__device__ __forceinline__ float ld_as_f32(const float* p, int64_t i) { return p[i]; }
__device__ __forceinline__ float ld_as_f32(const __nv_bfloat16* p, int64_t i) { return __bfloat162float(p[i]); }

// A scaled-fp8 weight as the quantizer's source: element (row, k) is LUT[byte] * scale in f32,
// exactly the value crates/loractl-core/src/fp8.rs:305-317 would have written to the f32 tensor
// that the reference then hands to quantize_linear_weight (diffusion_trainer.rs:1130-1175).
struct Fp8Src {
    const uint8_t* bytes;
    const float* scale;
    int per_channel;
};

// Two adjacent source elements (k0 even) of one row.
__device__ __forceinline__ void ld_pair(const float* p, int64_t row, int64_t K, int64_t k0, float& v0, float& v1) {
    const float2 v = *(const float2*)(p + row * K + k0);
    v0 = v.x;
    v1 = v.y;
}
__device__ __forceinline__ void ld_pair(const __nv_bfloat16* p, int64_t row, int64_t K, int64_t k0, float& v0, float& v1) {
    const __nv_bfloat162 v = *(const __nv_bfloat162*)(p + row * K + k0);
    v0 = __bfloat162float(v.x);
    v1 = __bfloat162float(v.y);
}
__device__ __forceinline__ void ld_pair(const Fp8Src& s, int64_t row, int64_t K, int64_t k0, float& v0, float& v1) {
    const uint16_t b = *(const uint16_t*)(s.bytes + row * K + k0);
    const float sc = s.per_channel ? s.scale[row] : s.scale[0];
    v0 = lq_decode_e4m3fn(b & 0xffu) * sc;
    v1 = lq_decode_e4m3fn(b >> 8) * sc;
}

__device__ __forceinline__ int quant_one(float v, float scale, float qmax) {
    if (!(scale > 0.f)) return 0;
    float r = roundf(__fdiv_rn(v, scale));  // roundf: ties away from zero (Rust f32::round)
    r = fminf(fmaxf(r, -qmax), qmax);
    return (int)r;
}

// One warp per (padded row, k-tile): lane owns k = kt*64 + 2*lane, +1.
template <typename Src>
__global__ void __launch_bounds__(256) quantize_kernel(const Src w, int64_t M, int64_t K, int G,
                                                       int bits, int64_t m_tiles, int64_t k_tiles,
                                                       int64_t n_groups, void* __restrict__ packed,
                                                       float* __restrict__ scales) {
    int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    int lane = threadIdx.x & 31;
    int64_t total = m_tiles * LQ_TILE_M * k_tiles;
    if (warp >= total) return;
    int64_t row = warp / k_tiles, kt = warp % k_tiles;
    int64_t k0 = kt * LQ_TILE_K + 2 * lane;
    float v0 = 0.f, v1 = 0.f;
    if (row < M && k0 < K) ld_pair(w, row, K, k0, v0, v1);  // K is even, so k0 + 1 < K too
    float a = fmaxf(fabsf(v0), fabsf(v1));
    int span = G / 2;  // lanes per group: 16 (G = 32) or 32 (G = 64)
    for (int off = span / 2; off >= 1; off >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, off));
    float qmax = bits == 4 ? 7.f : 127.f;
    float scale = __fdiv_rn(a, qmax);
    int q0 = quant_one(v0, scale, qmax), q1 = quant_one(v1, scale, qmax);

    int64_t mt = row >> 7, r = row & 127;
    int64_t g = k0 / G;
    if ((lane % span) == 0 && g < n_groups) scales[(mt * n_groups + g) * 128 + r] = scale;

    if (bits == 4) {
        int j = lane & 3;
        uint32_t part = ((uint32_t)(q0 + 8) << (4 * j)) | ((uint32_t)(q1 + 8) << (4 * j + 16));
        part |= __shfl_xor_sync(0xffffffffu, part, 1);
        part |= __shfl_xor_sync(0xffffffffu, part, 2);
        if (j == 0) {
            uint32_t* tile = (uint32_t*)packed + (mt * k_tiles + kt) * 1024;
            tile[r * 8 + (lane >> 2)] = part;
        }
    } else {
        uint16_t* tile = (uint16_t*)((int8_t*)packed + (mt * k_tiles + kt) * 8192);
        tile[r * 32 + lane] = (uint16_t)((uint32_t)(q0 & 0xff) | ((uint32_t)(q1 & 0xff) << 8));
    }
}

// Sixteen adjacent source elements (k0 a multiple of 16) of one row, as f32.
__device__ __forceinline__ void ld16(const float* p, int64_t row, int64_t K, int64_t k0, float (&v)[16]) {
    const float4* s = (const float4*)(p + row * K + k0);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float4 f = s[i];
        v[4 * i] = f.x; v[4 * i + 1] = f.y; v[4 * i + 2] = f.z; v[4 * i + 3] = f.w;
    }
}
__device__ __forceinline__ void ld16(const __nv_bfloat16* p, int64_t row, int64_t K, int64_t k0, float (&v)[16]) {
    const uint4* s = (const uint4*)(p + row * K + k0);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const uint4 u = s[i];
        const uint32_t w4[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            v[8 * i + 2 * j] = __uint_as_float(w4[j] << 16);
            v[8 * i + 2 * j + 1] = __uint_as_float(w4[j] & 0xFFFF0000u);
        }
    }
}
// e4m3 -> f16 is exact for every code (hardware conversion), f16 -> f32 is exact, so this is
// LUT[byte] * scale bit for bit.
__device__ __forceinline__ void ld16(const Fp8Src& s, int64_t row, int64_t K, int64_t k0, float (&v)[16]) {
    const uint4 u = *(const uint4*)(s.bytes + row * K + k0);
    const float sc = s.per_channel ? s.scale[row] : s.scale[0];
    const uint32_t w4[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const __half2_raw hr = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)((w4[j] >> (16 * h)) & 0xFFFFu), __NV_E4M3);
            const float2 f = __half22float2(*(const __half2*)&hr);
            v[4 * j + 2 * h] = f.x * sc;
            v[4 * j + 2 * h + 1] = f.y * sc;
        }
    }
}

// The load-time quantizer at HBM speed.  One warp per (8 consecutive rows, k-tile); lane =
// (row i = lane >> 2, quarter q = lane & 3) owns the 16 elements k = kt*64 + 16q .. +15: a
// 16/32/64-byte vector load per lane, 64 B per row and 8 rows per warp fully used; group absmax by
// one or two shuffles; the lane writes its two packed words (int4) or 16 bytes (int8), so a warp
// stores 256 (512) contiguous bytes of the tile and 8 consecutive scales.  Needs a 16-byte-aligned
// source and K % 16 == 0 (true whenever K % block == 0).
template <typename Src>
__global__ void __launch_bounds__(256) quantize16_kernel(const Src w, int64_t M, int64_t K, int G, int bits,
                                                         int64_t m_tiles, int64_t k_tiles, int64_t n_groups,
                                                         void* __restrict__ packed, float* __restrict__ scales) {
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (warp >= m_tiles * 16 * k_tiles) return;
    const int64_t unit = warp / k_tiles, kt = warp % k_tiles;
    const int64_t row = unit * 8 + (lane >> 2);
    const int q = lane & 3;
    const int64_t k0 = kt * LQ_TILE_K + 16 * q;
    float v[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = 0.f;
    if (row < M && k0 < K) ld16(w, row, K, k0, v);
    float a = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) a = fmaxf(a, fabsf(v[i]));
    a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 1));
    if (G == 64) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 2));
    const float qmax = bits == 4 ? 7.f : 127.f;
    const float scale = __fdiv_rn(a, qmax);
    const int64_t mt = row >> 7, r = row & 127;
    const int64_t g = k0 / G;
    if (g < n_groups && (G == 64 ? q == 0 : (q & 1) == 0)) scales[(mt * n_groups + g) * 128 + r] = scale;
    if (bits == 4) {
        uint32_t word[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            uint32_t acc = 0;
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const uint32_t u = (uint32_t)(quant_one(v[8 * h + e], scale, qmax) + 8);
                acc |= u << (4 * ((e >> 1) + 4 * (e & 1)));
            }
            word[h] = acc;
        }
        uint32_t* tile = (uint32_t*)packed + (mt * k_tiles + kt) * 1024;
        *(uint2*)(tile + r * 8 + 2 * q) = make_uint2(word[0], word[1]);
    } else {
        uint32_t word[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            uint32_t acc = 0;
#pragma unroll
            for (int e = 0; e < 4; ++e) acc |= ((uint32_t)quant_one(v[4 * j + e], scale, qmax) & 0xffu) << (8 * e);
            word[j] = acc;
        }
        uint8_t* tile = (uint8_t*)packed + (mt * k_tiles + kt) * 8192;
        *(uint4*)(tile + r * 64 + 16 * q) = make_uint4(word[0], word[1], word[2], word[3]);
    }
}

// Same tiling, from logical codes [M,K] + scales [M,K/G].
__global__ void __launch_bounds__(256) pack_codes_kernel(const int8_t* __restrict__ codes,
                                                         const float* __restrict__ sc_in, int64_t M, int64_t K,
                                                         int G, int bits, int64_t m_tiles, int64_t k_tiles,
                                                         int64_t n_groups, void* __restrict__ packed,
                                                         float* __restrict__ scales) {
    int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    int lane = threadIdx.x & 31;
    int64_t total = m_tiles * LQ_TILE_M * k_tiles;
    if (warp >= total) return;
    int64_t row = warp / k_tiles, kt = warp % k_tiles;
    int64_t k0 = kt * LQ_TILE_K + 2 * lane;
    int q0 = 0, q1 = 0;
    if (row < M && k0 < K) {
        q0 = codes[row * K + k0];
        q1 = codes[row * K + k0 + 1];
    }
    int64_t mt = row >> 7, r = row & 127;
    int span = G / 2;
    int64_t g = k0 / G;
    if ((lane % span) == 0 && g < n_groups)
        scales[(mt * n_groups + g) * 128 + r] = row < M ? sc_in[row * n_groups + g] : 0.f;
    if (bits == 4) {
        int j = lane & 3;
        uint32_t part = ((uint32_t)(q0 + 8) << (4 * j)) | ((uint32_t)(q1 + 8) << (4 * j + 16));
        part |= __shfl_xor_sync(0xffffffffu, part, 1);
        part |= __shfl_xor_sync(0xffffffffu, part, 2);
        if (j == 0) {
            uint32_t* tile = (uint32_t*)packed + (mt * k_tiles + kt) * 1024;
            tile[r * 8 + (lane >> 2)] = part;
        }
    } else {
        uint16_t* tile = (uint16_t*)((int8_t*)packed + (mt * k_tiles + kt) * 8192);
        tile[r * 32 + lane] = (uint16_t)((uint32_t)(q0 & 0xff) | ((uint32_t)(q1 & 0xff) << 8));
    }
}

__global__ void __launch_bounds__(256) unpack_kernel(LqWView w, int8_t* __restrict__ codes,
                                                     float* __restrict__ scales) {
    int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t total = w.M * w.K;
    if (idx < total) {
        int64_t m = idx / w.K, k = idx % w.K;
        if (w.scheme == LQ_FP8_E4M3) {
            codes[idx] = (int8_t)((const uint8_t*)w.packed)[idx];
        } else {
            int64_t mt = m >> 7, r = m & 127, kt = k >> 6, kk = k & 63;
            int q;
            if (w.scheme == LQ_INT4) {
                const uint32_t* tile = (const uint32_t*)w.packed + (mt * w.k_tiles + kt) * 1024;
                uint32_t word = tile[r * 8 + (kk >> 3)];
                int e = (int)(kk & 7);
                q = (int)((word >> (4 * ((e >> 1) + 4 * (e & 1)))) & 0xFu) - 8;
            } else {
                q = ((const int8_t*)w.packed + (mt * w.k_tiles + kt) * 8192)[r * 64 + kk];
            }
            codes[idx] = (int8_t)q;
        }
    }
    if (w.scheme == LQ_FP8_E4M3) {
        int64_t ns = w.scale_kind == LQ_SCALE_PER_CHANNEL ? w.M : 1;
        if (idx < ns) scales[idx] = w.scales[idx];
    } else {
        int64_t ns = w.M * w.n_groups;
        if (idx < ns) {
            int64_t m = idx / w.n_groups, g = idx % w.n_groups;
            scales[idx] = w.scales[((m >> 7) * w.n_groups + g) * 128 + (m & 127)];
        }
    }
}

// 64 x 64 tile through shared memory; writes are coalesced in either orientation.
template <typename OutT>
__global__ void __launch_bounds__(256) dequant_kernel(LqWView w, OutT* __restrict__ out, int64_t ld, int transpose) {
    __shared__ float tile[64][65];
    int64_t m0 = (int64_t)blockIdx.y * 64, k0 = (int64_t)blockIdx.x * 64;
    int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;  // 64 x 4
    for (int i = ty; i < 64; i += 4) {
        int64_t m = m0 + i, k = k0 + tx;
        tile[i][tx] = (m < w.M && k < w.K) ? lq_dequant_elem(w, m, k) : 0.f;
    }
    __syncthreads();
    if (!transpose) {
        for (int i = ty; i < 64; i += 4) {
            int64_t m = m0 + i, k = k0 + tx;
            if (m < w.M && k < w.K) out[m * ld + k] = (OutT)tile[i][tx];
        }
    } else {
        for (int i = ty; i < 64; i += 4) {
            int64_t k = k0 + i, m = m0 + tx;
            if (m < w.M && k < w.K) out[k * ld + m] = (OutT)tile[tx][i];
        }
    }
}

// Fast bf16 dequantisation for the GEMM scratch.  One block per 128 (m) x 64 (k) tile; every
// thread produces 32 consecutive k of one row: f32 `q * scale` (resp. `LUT[b] * scale`) rounded
// once to bf16.  transpose = 0 writes out[m * ld + k]; transpose = 1 stages the tile in shared
// memory and writes out[k * ld + m] in 256-byte runs.  Requires ld % 8 == 0, 16-byte aligned
// `out`, and for fp8 d_in % 16 == 0.
__device__ __forceinline__ uint32_t pack_bf16x2(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *(uint32_t*)&v;
}

__global__ void __launch_bounds__(256) dequant_tile_kernel(LqWView w, __nv_bfloat16* __restrict__ out, int64_t ld,
                                                           int transpose) {
    constexpr int TLD = 136;  // staged tile row stride (bf16), keeps 16-byte alignment
    __shared__ __align__(16) __nv_bfloat16 stage[64 * TLD];
    const int t = threadIdx.x;
    const int r = t >> 1, half = t & 1;
    const int64_t mt = blockIdx.y, kt = blockIdx.x;
    const int64_t m = mt * 128 + r, k0 = kt * 64 + half * 32;
    uint32_t o[16];  // 32 bf16
    const bool live = m < w.M && k0 < w.K;  // K % 32 == 0 on the int path, % 16 on fp8: handled below
    if (!live) {
#pragma unroll
        for (int i = 0; i < 16; ++i) o[i] = 0u;
    } else if (w.scheme == LQ_INT4) {
        const uint4 v = *((const uint4*)((const uint32_t*)w.packed + (mt * w.k_tiles + kt) * 1024) + t);
        const uint32_t words[4] = {v.x, v.y, v.z, v.w};
        // the 32 k of this thread never straddle a scale group (group is 32 or 64, k0 % 32 == 0)
        const float s = w.scales[(mt * w.n_groups + k0 / w.group) * 128 + r];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int q0 = (int)((words[c] >> (4 * j)) & 0xFu) - 8;
                const int q1 = (int)((words[c] >> (4 * j + 16)) & 0xFu) - 8;
                o[c * 4 + j] = pack_bf16x2((float)q0 * s, (float)q1 * s);
            }
        }
    } else if (w.scheme == LQ_INT8) {
        const uint4* src = (const uint4*)((const int8_t*)w.packed + (mt * w.k_tiles + kt) * 8192 + r * 64 + half * 32);
        const float s = w.scales[(mt * w.n_groups + k0 / w.group) * 128 + r];
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            const uint4 v = src[c];
            const uint32_t words[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int q0 = (int)(int8_t)(words[j] & 0xFF), q1 = (int)(int8_t)((words[j] >> 8) & 0xFF);
                const int q2 = (int)(int8_t)((words[j] >> 16) & 0xFF), q3 = (int)(int8_t)(words[j] >> 24);
                o[c * 8 + j * 2] = pack_bf16x2((float)q0 * s, (float)q1 * s);
                o[c * 8 + j * 2 + 1] = pack_bf16x2((float)q2 * s, (float)q3 * s);
            }
        }
    } else {  // fp8 e4m3fn, row-major [M, K]
        const float s = w.scale_kind == LQ_SCALE_PER_CHANNEL ? w.scales[m] : w.scales[0];
        const uint8_t* row = (const uint8_t*)w.packed + m * w.K + k0;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            if (k0 + c * 16 < w.K) {
                const uint4 v = *(const uint4*)(row + c * 16);
                const uint32_t words[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    // e4m3 -> f16 is exact (hardware cvt); NaN bytes stay NaN
                    const __half2_raw lo = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(words[j] & 0xFFFF), __NV_E4M3);
                    const __half2_raw hi = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(words[j] >> 16), __NV_E4M3);
                    const float2 fl = __half22float2(*(const __half2*)&lo), fh = __half22float2(*(const __half2*)&hi);
                    o[c * 8 + j * 2] = pack_bf16x2(fl.x * s, fl.y * s);
                    o[c * 8 + j * 2 + 1] = pack_bf16x2(fh.x * s, fh.y * s);
                }
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) o[c * 8 + j] = 0u;
            }
        }
    }
    if (!transpose) {
        if (live) {
            uint4* dst = (uint4*)(out + m * ld + k0);
#pragma unroll
            for (int c = 0; c < 4; ++c)
                if (k0 + c * 8 < w.K) dst[c] = make_uint4(o[c * 4], o[c * 4 + 1], o[c * 4 + 2], o[c * 4 + 3]);
        }
        return;
    }
    // transposed: stage[k][m] then 256-byte rows out
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const __nv_bfloat162 v = *(const __nv_bfloat162*)&o[i];
        stage[(half * 32 + 2 * i) * TLD + r] = v.x;
        stage[(half * 32 + 2 * i + 1) * TLD + r] = v.y;
    }
    __syncthreads();
    const int mc = (t & 15) * 8;  // 8 consecutive m per thread
#pragma unroll
    for (int pass = 0; pass < 4; ++pass) {
        const int kk = pass * 16 + (t >> 4);
        const int64_t k = kt * 64 + kk, mm = mt * 128 + mc;
        if (k < w.K && mm < w.M)  // M % 8 == 0: an 8-wide group is entirely in or out
            *(uint4*)(out + k * ld + mm) = *(const uint4*)&stage[kk * TLD + mc];
    }
}

// ---- fp8 repack: scale = amax / 448 (>= 1e-12), q = e4m3fn(w / scale), RNE ------------

__device__ __forceinline__ uint8_t encode_e4m3fn(float x) {
    // Round to nearest even on the e4m3fn grid; |x| that rounds past 448 -> NaN (torch cast).
    uint32_t u = __float_as_uint(x);
    uint8_t sign = (uint8_t)((u >> 24) & 0x80u);
    float ax = fabsf(x);
    if (!(ax == ax)) return sign | 0x7F;
    if (ax > 464.f) return sign | 0x7F;  // 464 itself ties to even (448)
    if (ax < 0.015625f) {  // below the smallest normal 2^-6: subnormal grid, spacing 2^-9
        float r = rintf(ax * 512.f);  // rintf: round half to even
        return sign | (uint8_t)r;     // r == 8 encodes the first normal (exp 1, man 0) correctly
    }
    uint32_t a = __float_as_uint(ax);
    // keep 3 mantissa bits, RNE on the dropped 20
    uint32_t lsb = (a >> 20) & 1u;
    a += 0x7FFFFu + lsb;
    a &= 0xFFF00000u;
    int e = (int)(a >> 23) - 127 + 7;
    uint32_t man = (a >> 20) & 7u;
    return sign | (uint8_t)((e << 3) | man);
}

__global__ void __launch_bounds__(256) fp8_rowmax_kernel(const float* __restrict__ w, int64_t M, int64_t K,
                                                         float* __restrict__ rowmax) {
    __shared__ float red[8];
    int64_t m = blockIdx.x;
    float a = 0.f;
    for (int64_t k = threadIdx.x; k < K; k += blockDim.x) a = fmaxf(a, fabsf(w[m * K + k]));
    for (int off = 16; off >= 1; off >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, off));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = a;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int i = 1; i < 8; ++i) a = fmaxf(a, red[i]);
        rowmax[m] = a;
    }
}

__global__ void fp8_scale_kernel(const float* __restrict__ rowmax, int64_t M, int per_channel,
                                 float* __restrict__ scales) {
    if (per_channel) {
        int64_t m = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
        if (m < M) scales[m] = fmaxf(__fdiv_rn(rowmax[m], 448.f), 1e-12f);
    } else if (blockIdx.x == 0 && threadIdx.x == 0) {
        float a = 0.f;
        for (int64_t m = 0; m < M; ++m) a = fmaxf(a, rowmax[m]);
        scales[0] = fmaxf(__fdiv_rn(a, 448.f), 1e-12f);
    }
}

__global__ void __launch_bounds__(256) fp8_encode_kernel(const float* __restrict__ w, int64_t M, int64_t K,
                                                         int per_channel, const float* __restrict__ scales,
                                                         uint8_t* __restrict__ bytes) {
    int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= M * K) return;
    float s = per_channel ? scales[idx / K] : scales[0];
    bytes[idx] = encode_e4m3fn(__fdiv_rn(w[idx], s));
}

inline unsigned blocks_for(int64_t n, int per) { return (unsigned)((n + per - 1) / per); }

}  // namespace

template <typename Src>
static void launch_quantize_src(const Src& src, const void* base, const lq_weight* d, int bits, cudaStream_t st) {
    if (((uintptr_t)base & 15) == 0 && d->K % 16 == 0) {
        const int64_t warps = d->m_tiles * 16 * d->k_tiles;
        quantize16_kernel<Src><<<blocks_for(warps, 8), 256, 0, st>>>(src, d->M, d->K, d->group, bits, d->m_tiles, d->k_tiles,
                                                                    d->n_groups, d->packed, d->scales);
    } else {  // unaligned source: the element-pair kernel
        const int64_t warps = d->m_tiles * LQ_TILE_M * d->k_tiles;
        quantize_kernel<Src><<<blocks_for(warps, 8), 256, 0, st>>>(src, d->M, d->K, d->group, bits, d->m_tiles, d->k_tiles,
                                                                  d->n_groups, d->packed, d->scales);
    }
    LQ_CUDA(cudaGetLastError());
}

void lq_launch_quantize(const void* w, int w_dtype, const lq_weight* d, int bits, cudaStream_t st) {
    LqProf prof(LQ_K_QUANT, st);
    if (w_dtype == LQ_F32) launch_quantize_src<const float*>((const float*)w, w, d, bits, st);
    else launch_quantize_src<const __nv_bfloat16*>((const __nv_bfloat16*)w, w, d, bits, st);
}

void lq_launch_quantize_fp8(const uint8_t* bytes, const float* scale, int per_channel, const lq_weight* d, int bits,
                            cudaStream_t st) {
    LqProf prof(LQ_K_QUANT, st);
    Fp8Src src{bytes, scale, per_channel};
    launch_quantize_src<Fp8Src>(src, bytes, d, bits, st);
}

void lq_launch_pack_codes(const int8_t* codes, const float* scales, const lq_weight* d, cudaStream_t st) {
    LqProf prof(LQ_K_QUANT, st);
    int64_t warps = d->m_tiles * LQ_TILE_M * d->k_tiles;
    int bits = d->scheme == LQ_INT4 ? 4 : 8;
    pack_codes_kernel<<<blocks_for(warps, 8), 256, 0, st>>>(codes, scales, d->M, d->K, d->group, bits, d->m_tiles,
                                                            d->k_tiles, d->n_groups, d->packed, d->scales);
    LQ_CUDA(cudaGetLastError());
}

void lq_launch_unpack(const lq_weight* w, int8_t* codes, float* scales, cudaStream_t st) {
    LqProf prof(LQ_K_QUANT, st);
    unpack_kernel<<<blocks_for(w->M * w->K, 256), 256, 0, st>>>(lq_view(w), codes, scales);
    LQ_CUDA(cudaGetLastError());
}

void lq_launch_dequant(const lq_weight* w, void* out, int out_dtype, int64_t ld, int transpose, cudaStream_t st) {
    LqProf prof(LQ_K_DEQUANT, st);
    const bool aligned = (ld % 8 == 0) && (((uintptr_t)out & 15) == 0) && (w->M % 8 == 0) &&
                         (w->scheme != LQ_FP8_E4M3 || w->K % 16 == 0);
    if (out_dtype == LQ_BF16 && aligned) {
        dim3 grid((unsigned)((w->K + 63) / 64), (unsigned)((w->M + 127) / 128));
        dequant_tile_kernel<<<grid, 256, 0, st>>>(lq_view(w), (__nv_bfloat16*)out, ld, transpose);
        LQ_CUDA(cudaGetLastError());
        return;
    }
    dim3 grid((unsigned)((w->K + 63) / 64), (unsigned)((w->M + 63) / 64));
    if (out_dtype == LQ_F32)
        dequant_kernel<float><<<grid, 256, 0, st>>>(lq_view(w), (float*)out, ld, transpose);
    else
        dequant_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(lq_view(w), (__nv_bfloat16*)out, ld, transpose);
    LQ_CUDA(cudaGetLastError());
}

void lq_launch_fp8_quantize(const float* w, int64_t M, int64_t K, int per_channel, uint8_t* bytes, float* scales,
                            cudaStream_t st) {
    LqProf prof(LQ_K_QUANT, st);
    float* rowmax = nullptr;
    LQ_CUDA(cudaMallocAsync((void**)&rowmax, sizeof(float) * (size_t)M, st));
    fp8_rowmax_kernel<<<(unsigned)M, 256, 0, st>>>(w, M, K, rowmax);
    fp8_scale_kernel<<<per_channel ? blocks_for(M, 256) : 1, 256, 0, st>>>(rowmax, M, per_channel, scales);
    fp8_encode_kernel<<<blocks_for(M * K, 256), 256, 0, st>>>(w, M, K, per_channel, scales, bytes);
    cudaError_t e = cudaGetLastError();
    cudaFreeAsync(rowmax, st);
    LQ_CUDA(e);
}
