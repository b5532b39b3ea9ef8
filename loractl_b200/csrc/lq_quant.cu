// Quantize / pack / unpack / dequantize kernels (HBM-bound, load-time and scratch paths).
//
// Arithmetic follows burn-ndarray 0.21's symmetric per-block scheme as pinned by
// reference/quant_int4_reference.py:46-58 and reference/quant_reference.py:40-52:
//   scale = absmax / qmax            (f32, IEEE division)
//   q     = clamp(round(w / scale))  (f32 division, round half away from zero)
// An all-zero block gets scale 0 and codes 0.
#include "lq_internal.cuh"
#include "lq_prof.cuh"

namespace {

__device__ __forceinline__ float ld_as_f32(const float* p, int64_t i) { return p[i]; }
__device__ __forceinline__ float ld_as_f32(const __nv_bfloat16* p, int64_t i) { return __bfloat162float(p[i]); }

__device__ __forceinline__ int quant_one(float v, float scale, float qmax) {
    if (!(scale > 0.f)) return 0;
    float r = roundf(__fdiv_rn(v, scale));  // roundf: ties away from zero (Rust f32::round)
    r = fminf(fmaxf(r, -qmax), qmax);
    return (int)r;
}

// One warp per (padded row, k-tile): lane owns k = kt*64 + 2*lane, +1.
template <typename T>
__global__ void __launch_bounds__(256) quantize_kernel(const T* __restrict__ w, int64_t M, int64_t K, int G,
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
    if (row < M && k0 < K) {  // K is even, so k0 + 1 < K too
        v0 = ld_as_f32(w, row * K + k0);
        v1 = ld_as_f32(w, row * K + k0 + 1);
    }
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

void lq_launch_quantize(const void* w, int w_dtype, const lq_weight* d, int bits, cudaStream_t st) {
    LqProf prof(LQ_K_QUANT, st);
    int64_t warps = d->m_tiles * LQ_TILE_M * d->k_tiles;
    unsigned grid = blocks_for(warps, 8);
    if (w_dtype == LQ_F32)
        quantize_kernel<float><<<grid, 256, 0, st>>>((const float*)w, d->M, d->K, d->group, bits, d->m_tiles,
                                                     d->k_tiles, d->n_groups, d->packed, d->scales);
    else
        quantize_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)w, d->M, d->K, d->group, bits,
                                                             d->m_tiles, d->k_tiles, d->n_groups, d->packed,
                                                             d->scales);
    LQ_CUDA(cudaGetLastError());
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
