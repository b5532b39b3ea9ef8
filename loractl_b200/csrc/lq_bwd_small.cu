// Backward of the quantized LoRA linear at N <= 16 tokens over the PACKED int4 stream.
//
//   dX[n, k] = sum_m dY[n, m] * W[m, k]  +  sum_j dH[n, j] * A[k, j]        dH = s * dY . B^T
//   dA[k, j] (+)= sum_n X[n, k] * dH[n, j]                                  dB[j, m] (+)= s * sum_n H[n, j] * dY[n, m]
//
// The reference's backward dequantises the whole weight to f32 and multiplies
// (crates/loractl-core/src/quant.rs:232-233,250-251); the tensor-regime path here writes a bf16 image
// of W^T first.  For a one-token site (an adaLN modulation projection, 3072 -> 18432: 56.6 M weights)
// that image is a 113 MB round trip for 0.1 GFLOP.  Here the 28 MB of packed nibbles are read from
// HBM once and converted in registers, as in the <= 16-token forward (`stream_small_fwd_kernel`),
// and the whole call is two launches (weight stream + finalize) instead of about twelve.
//
// Weight stream kernel, 160 threads, 3 CTAs per SM.  A work item is (chunk of 4 adjacent k-tiles,
// split z of the m-tiles); a pipeline stage holds one m-tile of the chunk: the 4 packed tiles (one
// bulk copy of 16 KB: tiles of one m-tile are adjacent in k), their 4 (or 8) x 128 group scales, and the
// [16 tokens x 128 m] slice of dY as two 128-byte-swizzled tensor boxes (rows past N and columns
// past d_out read as zero).  Consumer warp c owns k-tile c of the chunk = 64 output columns.
//
// mma.sync.m16n8k16 with the weight as the 16-row operand: rows = output columns k, reduction = m,
// columns = tokens.  A register of the row operand pairs two values that are adjacent along the
// REDUCTION, i.e. the same nibble of the packed words of two different weight rows, so each register
// is one byte permute of two masked words plus one and-or (`0x4300 | u` = bf16 128 + u = 136 + q).
// The assignment of fragment slots to (m, k) is free as long as both operands agree; it is chosen so
// that a lane uses all 8 nibbles of every word it loads and no two lanes of a load share a bank:
//   fragment row g   of MMA j  <->  k = 8g + j        (word g of the row, element j)
//   fragment row g+8 of MMA j  <->  k = 8g + j + 4    (word g, element j + 4)
//   reduction slots 2t, 2t+1, 2t+8, 2t+9  <->  m = m0 + t, m0 + 4 + t, m0 + 8 + t, m0 + 12 + t
// The group scale varies along the reduction (one per weight row), so it is folded into the token
// operand instead: b'[m, n] = bf16(dY[n, m] * scale[m, tile]).  The +136 offset is removed with one
// extra MMA against an all-ones row operand per 16 m (sum of b' per token).  With quant block 32 a
// k-tile holds two scale groups (words 0-3 and 4-7 of a row) and an MMA must stay inside one: lanes g
// and g + 4 then share word 4h + (g & 3) and split its elements by parity, two token operands and two
// offset sums per 16 m (the reference's own block size, crates/loractl-core/src/quant.rs:52).
//
// The first CTAs of the grid compute partial rows of dH = s * dY . B^T (and of H = X . A when the
// caller did not keep it) in f32; the finalize kernel sums the splits in a fixed order, adds the
// LoRA term, and forms dA and dB.  Every wait is bounded and reports through the device status word.
#include <algorithm>
#include <cstdint>
#include <string>

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "lq_internal.cuh"
#include "lq_prof.cuh"
#include "lq_stream.cuh"
#include "lq_tc.cuh"
#include "lq_umma.cuh"

namespace {

using namespace umma;
using namespace lqstream;

constexpr int kThreads = 32 + 128;
constexpr int KC = 4;                      // k-tiles per chunk = consumer warps
constexpr int NT = 16;                     // token rows of the dY boxes
constexpr uint32_t DY_BYTES = 2 * NT * 128;  // two boxes [16 tokens][64 m] bf16
constexpr uint32_t P_OFF = DY_BYTES, S_OFF = P_OFF + KC * 4096;
constexpr uint32_t STAGE_BYTES = S_OFF + KC * 1024;  // 24 KB (scales: up to two groups per k-tile), a multiple of 1024
constexpr int STAGES = 2;  // three stages (a whole item in flight) measured no faster
constexpr size_t SMEM = (size_t)STAGES * STAGE_BYTES + 1024 + 128;
constexpr int CTAS_PER_SM = 3;
constexpr int kMaxSplits = 48;
constexpr int kRowChunk = 2048;  // reduction elements per CTA of the dH / H partial rows

struct BwdParams {
    const uint8_t* packed;
    const float* scales;
    int M, K, N;
    int k_tiles, m_tiles, n_groups;
    int kchunks, splits;
    float* part;  // [splits][N][K]
    int* status;
    // partial LoRA rows, computed by the first h_blocks CTAs
    int h_blocks, dh_chunks, h_chunks, r;
    const __nv_bfloat16* dY;  // [N, M]
    const __nv_bfloat16* X;   // [N, K]
    const float* A;           // [K, r]
    const float* B;           // [r, M]
    float* dHpart;            // [dh_chunks][N][r]   (unscaled)
    float* Hpart;             // [h_chunks][N][r]    (only when the caller passed no H)
};

// (nibble of x, nibble of y) as the bf16 pair (128 + u_x, 128 + u_y): `sel` picks one byte of each masked word
__device__ __forceinline__ uint32_t nib_pair(uint32_t x, uint32_t y, uint32_t sel) {
    return (__byte_perm(x, y, sel) & 0x00FF00FFu) | 0x43004300u;
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *(uint32_t*)&v;
}

// out[j] = sum over l in [l0, l1) of x[l] * Mat[l * sl + j * sj], j < r: one CTA, f32, 16 columns at a
// time, fixed shuffle tree then a fixed-order pass over the warps (deterministic).
__device__ __forceinline__ void row_partial(const __nv_bfloat16* __restrict__ x, const float* __restrict__ Mat, long long sl,
                                            long long sj, int l0, int l1, int r, float* __restrict__ out, float* red) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (int j0 = 0; j0 < r; j0 += 16) {
        float acc[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) acc[j] = 0.f;
#pragma unroll 2
        for (int l = l0 + tid; l < l1; l += kThreads) {
            const float xv = __bfloat162float(x[l]);
            const float* src = Mat + (long long)l * sl + (long long)j0 * sj;
#pragma unroll
            for (int j = 0; j < 16; ++j)
                if (j0 + j < r) acc[j] = fmaf(xv, __ldg(src + (long long)j * sj), acc[j]);
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            float v = acc[j];
#pragma unroll
            for (int off = 16; off >= 1; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
            if (lane == 0) red[warp * 16 + j] = v;
        }
        __syncthreads();
        if (tid < 16 && j0 + tid < r) {
            float h = 0.f;
#pragma unroll
            for (int w5 = 0; w5 < kThreads / 32; ++w5) h += red[w5 * 16 + tid];
            out[j0 + tid] = h;
        }
        __syncthreads();
    }
}

// GPT = scale groups per 64-wide k-tile: 1 (quant block 64) or 2 (block 32).
template <int NB, int GPT>
__global__ void __launch_bounds__(kThreads, CTAS_PER_SM)
stream_small_bwd_kernel(const __grid_constant__ CUtensorMap tmDY, const __grid_constant__ BwdParams p) {
    extern __shared__ uint8_t smem_raw_[];
    uint8_t* raw = (uint8_t*)(((uintptr_t)smem_raw_ + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = (uint64_t*)(raw + (size_t)STAGES * STAGE_BYTES);
    uint64_t* full = bars;
    uint64_t* empty = bars + STAGES;
    volatile int* abort_flag = (volatile int*)(bars + 2 * STAGES);

    pdl_launch_dependents();
    pdl_wait();
    if ((int)blockIdx.x < p.h_blocks) {  // uniform per CTA: one chunk of one token's dH (or H) row
        int b = (int)blockIdx.x;
        const int n_dh = p.dh_chunks * p.N;
        if (b < n_dh) {
            const int q = b / p.N, n = b - q * p.N;
            row_partial(p.dY + (size_t)n * p.M, p.B, 1, p.M, q * kRowChunk, min(p.M, (q + 1) * kRowChunk), p.r,
                        p.dHpart + ((size_t)q * p.N + n) * p.r, (float*)raw);
        } else {
            b -= n_dh;
            const int q = b / p.N, n = b - q * p.N;
            row_partial(p.X + (size_t)n * p.K, p.A, p.r, 1, q * kRowChunk, min(p.K, (q + 1) * kRowChunk), p.r,
                        p.Hpart + ((size_t)q * p.N + n) * p.r, (float*)raw);
        }
        return;
    }
    const int first = (int)blockIdx.x - p.h_blocks, stride = (int)gridDim.x - p.h_blocks;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&full[s]), 1);
            mbar_init(smem_u32(&empty[s]), KC);  // one arrival per consumer warp
        }
        *abort_flag = 0;
        fence_barrier_init();
        prefetch_tmap(&tmDY);
    }
    __syncthreads();
    const int num_items = p.kchunks * p.splits;

    if (warp == 0) {
        if (lane == 0) {
            int s = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int item = first; ok && item < num_items; item += stride) {
                const int kc = item / p.splits, z = item - kc * p.splits;
                const int mt0 = (int)(((long long)z * p.m_tiles) / p.splits);
                const int mt1 = (int)(((long long)(z + 1) * p.m_tiles) / p.splits);
                const int tiles = min(KC, p.k_tiles - kc * KC);
                for (int mt = mt0; mt < mt1; ++mt) {
                    if (!mbar_wait(smem_u32(&empty[s]), phase ^ 1u, abort_flag, p.status, 35)) { ok = false; break; }
                    const uint32_t bar = smem_u32(&full[s]);
                    const uint32_t base = smem_u32(raw + (size_t)s * STAGE_BYTES);
                    mbar_expect_tx(bar, DY_BYTES + (uint32_t)tiles * (4096u + GPT * 512u));  // the dY boxes are always whole
                    tma_load_2d(base, &tmDY, bar, mt * 128, 0);
                    tma_load_2d(base + NT * 128, &tmDY, bar, mt * 128 + 64, 0);
                    bulk_load(base + P_OFF, p.packed + ((size_t)mt * p.k_tiles + (size_t)kc * KC) * 4096,
                              (uint32_t)tiles * 4096u, bar);
                    bulk_load(base + S_OFF, p.scales + ((size_t)mt * p.n_groups + (size_t)kc * KC * GPT) * 128,
                              (uint32_t)tiles * GPT * 512u, bar);
                    if (++s == STAGES) { s = 0; phase ^= 1u; }
                }
            }
            if (!ok)
                for (int i = 0; i < 64; ++i) __nanosleep(1000);
        }
        return;
    }

    // ---------------- consumers: warp cw owns k-tile cw of the chunk ----------------
    const int cw = warp - 1, g = lane >> 2, t = lane & 3;
    constexpr uint32_t ONES = 0x3F803F80u;  // bf16 (1, 1)
    int s = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int item = first; ok && item < num_items; item += stride) {
        const int kc = item / p.splits, z = item - kc * p.splits;
        const int mt0 = (int)(((long long)z * p.m_tiles) / p.splits);
        const int mt1 = (int)(((long long)(z + 1) * p.m_tiles) / p.splits);
        const bool live = kc * KC + cw < p.k_tiles;  // the last chunk may hold fewer than KC tiles
        // GPT 1: acc[j] = MMA j of the tile, one[0] its offset sums.  GPT 2: acc[2h + jj] = MMA jj of scale
        // group h (k = 32h .. 32h + 31), one[h] that group's offset sums.
        float acc[4][NB][4], one[GPT][NB][4];
#pragma unroll
        for (int nb = 0; nb < NB; ++nb)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
#pragma unroll
                for (int h = 0; h < GPT; ++h) one[h][nb][e] = 0.f;
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[j][nb][e] = 0.f;
            }
        for (int mt = mt0; ok && mt < mt1; ++mt) {
            if (!mbar_wait(smem_u32(&full[s]), phase, abort_flag, p.status, 36)) { ok = false; break; }
            if (live) {
                const uint8_t* stage = raw + (size_t)s * STAGE_BYTES;
                const uint32_t* pk = (const uint32_t*)(stage + P_OFF + cw * 4096);
                const float* sc = (const float*)(stage + S_OFF) + cw * GPT * 128;
                const int mrem = p.M - mt * 128;
#pragma unroll 2
                for (int c = 0; c < 8; ++c) {
                    const int m0 = c * 16 + t;  // this lane's four reduction rows: m0, m0 + 4, m0 + 8, m0 + 12
                    float dy[NB][4];
#pragma unroll
                    for (int nb = 0; nb < NB; ++nb) {
                        const int n = nb * 8 + g;
                        // [16 tokens][64 m] boxes, 128-byte swizzle: 16-byte chunk index ^ (token & 7)
                        const uint8_t* row = stage + (c >> 2) * (NT * 128) + n * 128;
                        const int ml = (c & 3) * 16 + t;  // m0 within its box; m0 + 4i stays inside the same 16
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const uint32_t mm = (uint32_t)(ml + 4 * i);
                            const uint32_t off = (((mm >> 3) ^ ((uint32_t)n & 7u)) << 4) + ((mm & 7u) << 1);
                            dy[nb][i] = __bfloat162float(*(const __nv_bfloat16*)(row + off));
                        }
                    }
                    // rows past d_out (last m-tile): dY reads as zero there, and the scale must not turn it into NaN
                    const bool in0 = m0 < mrem, in1 = m0 + 4 < mrem, in2 = m0 + 8 < mrem, in3 = m0 + 12 < mrem;
                    if constexpr (GPT == 1) {
                        const uint32_t* pw = pk + g;  // word g of each row: 8 consecutive k
                        const uint32_t wA = pw[m0 * 8], wB = pw[(m0 + 4) * 8], wC = pw[(m0 + 8) * 8], wD = pw[(m0 + 12) * 8];
                        const float sA = in0 ? sc[m0] : 0.f, sB = in1 ? sc[m0 + 4] : 0.f;
                        const float sC = in2 ? sc[m0 + 8] : 0.f, sD = in3 ? sc[m0 + 12] : 0.f;
                        const uint32_t eA = wA & 0x0F0F0F0Fu, oA = (wA >> 4) & 0x0F0F0F0Fu;
                        const uint32_t eB = wB & 0x0F0F0F0Fu, oB = (wB >> 4) & 0x0F0F0F0Fu;
                        const uint32_t eC = wC & 0x0F0F0F0Fu, oC = (wC >> 4) & 0x0F0F0F0Fu;
                        const uint32_t eD = wD & 0x0F0F0F0Fu, oD = (wD >> 4) & 0x0F0F0F0Fu;
                        // element e of a word sits in nibble (e >> 1) + 4 (e & 1): elements 0, 4, 1, 5 are bytes
                        // 0..3 of the even-nibble word, elements 2, 6, 3, 7 those of the odd-nibble word
#pragma unroll
                        for (int nb = 0; nb < NB; ++nb) {
                            const uint32_t b0 = pack_bf16x2(dy[nb][0] * sA, dy[nb][1] * sB);
                            const uint32_t b1 = pack_bf16x2(dy[nb][2] * sC, dy[nb][3] * sD);
                            // MMA j: fragment rows g / g + 8 = elements j / j + 4 of word g
                            mma_16816(acc[0][nb], nib_pair(eA, eB, 0x0400u), nib_pair(eA, eB, 0x0501u),
                                      nib_pair(eC, eD, 0x0400u), nib_pair(eC, eD, 0x0501u), b0, b1);
                            mma_16816(acc[1][nb], nib_pair(eA, eB, 0x0602u), nib_pair(eA, eB, 0x0703u),
                                      nib_pair(eC, eD, 0x0602u), nib_pair(eC, eD, 0x0703u), b0, b1);
                            mma_16816(acc[2][nb], nib_pair(oA, oB, 0x0400u), nib_pair(oA, oB, 0x0501u),
                                      nib_pair(oC, oD, 0x0400u), nib_pair(oC, oD, 0x0501u), b0, b1);
                            mma_16816(acc[3][nb], nib_pair(oA, oB, 0x0602u), nib_pair(oA, oB, 0x0703u),
                                      nib_pair(oC, oD, 0x0602u), nib_pair(oC, oD, 0x0703u), b0, b1);
                            mma_16816(one[0][nb], ONES, ONES, ONES, ONES, b0, b1);
                        }
                    } else {
                        // Two scale groups per tile (words 0-3, words 4-7): an MMA must stay inside one group,
                        // so lanes g and g + 4 share word 4h + (g & 3) and take its elements of parity g >> 2:
                        //   MMA (h, jj): fragment row g <-> element (g >> 2) + 2 jj, row g + 8 <-> that + 4
                        const uint32_t sel0 = (g & 4) ? 0x0602u : 0x0400u, sel1 = (g & 4) ? 0x0703u : 0x0501u;
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            const uint32_t* pw = pk + 4 * h + (g & 3);
                            const uint32_t wA = pw[m0 * 8], wB = pw[(m0 + 4) * 8], wC = pw[(m0 + 8) * 8], wD = pw[(m0 + 12) * 8];
                            const float* sh_ = sc + h * 128;
                            const float sA = in0 ? sh_[m0] : 0.f, sB = in1 ? sh_[m0 + 4] : 0.f;
                            const float sC = in2 ? sh_[m0 + 8] : 0.f, sD = in3 ? sh_[m0 + 12] : 0.f;
                            const uint32_t eA = wA & 0x0F0F0F0Fu, oA = (wA >> 4) & 0x0F0F0F0Fu;
                            const uint32_t eB = wB & 0x0F0F0F0Fu, oB = (wB >> 4) & 0x0F0F0F0Fu;
                            const uint32_t eC = wC & 0x0F0F0F0Fu, oC = (wC >> 4) & 0x0F0F0F0Fu;
                            const uint32_t eD = wD & 0x0F0F0F0Fu, oD = (wD >> 4) & 0x0F0F0F0Fu;
#pragma unroll
                            for (int nb = 0; nb < NB; ++nb) {
                                const uint32_t b0 = pack_bf16x2(dy[nb][0] * sA, dy[nb][1] * sB);
                                const uint32_t b1 = pack_bf16x2(dy[nb][2] * sC, dy[nb][3] * sD);
                                mma_16816(acc[2 * h][nb], nib_pair(eA, eB, sel0), nib_pair(eA, eB, sel1),
                                          nib_pair(eC, eD, sel0), nib_pair(eC, eD, sel1), b0, b1);
                                mma_16816(acc[2 * h + 1][nb], nib_pair(oA, oB, sel0), nib_pair(oA, oB, sel1),
                                          nib_pair(oC, oD, sel0), nib_pair(oC, oD, sel1), b0, b1);
                                mma_16816(one[h][nb], ONES, ONES, ONES, ONES, b0, b1);
                            }
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&empty[s]));
            if (++s == STAGES) { s = 0; phase ^= 1u; }
        }
        if (!ok) break;
        if (live) {
            float* pz = p.part + (size_t)z * p.N * p.K;
            const int kt0 = (kc * KC + cw) * 64;
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) {
#pragma unroll
                for (int col = 0; col < 2; ++col) {
                    const int n = nb * 8 + 2 * t + col;
                    if (n >= p.N) continue;
                    float* dst = pz + (size_t)n * p.K + kt0;
                    if constexpr (GPT == 1) {
                        // fragment (row g, columns 2t / 2t+1) of MMA j = dX partial of k = 8g + j for tokens 2t,
                        // 2t + 1; row g + 8 the same for k = 8g + j + 4: eight consecutive k per lane and token
                        const float off = 136.f * one[0][nb][col];
                        float4 lo, hi;
                        lo.x = acc[0][nb][col] - off; lo.y = acc[1][nb][col] - off;
                        lo.z = acc[2][nb][col] - off; lo.w = acc[3][nb][col] - off;
                        hi.x = acc[0][nb][2 + col] - off; hi.y = acc[1][nb][2 + col] - off;
                        hi.z = acc[2][nb][2 + col] - off; hi.w = acc[3][nb][2 + col] - off;
                        *(float4*)(dst + g * 8) = lo;
                        *(float4*)(dst + g * 8 + 4) = hi;
                    } else {
                        // MMA (h, jj), row g: k = 32h + 8 (g & 3) + (g >> 2) + 2 jj; row g + 8: that + 4
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            const float off = 136.f * one[h][nb][col];
                            float* d = dst + 32 * h + 8 * (g & 3) + (g >> 2);
                            d[0] = acc[2 * h][nb][col] - off;
                            d[2] = acc[2 * h + 1][nb][col] - off;
                            d[4] = acc[2 * h][nb][2 + col] - off;
                            d[6] = acc[2 * h + 1][nb][2 + col] - off;
                        }
                    }
                }
            }
        }
    }
}

// Sums the splits and the partial LoRA rows in a fixed order and writes every output of the call.
// blockIdx.x ranges: [0, dx_blocks) dX (256 columns of one token each), then dB (256 columns of d_out),
// then dA (256 rows of d_in).
struct FinParams {
    int N, K, M, r, splits, dh_chunks, h_chunks;
    int dx_blocks, db_blocks, da_blocks, accumulate;
    float s;
    const float* part;
    const float* dHpart;
    const float* Hpart;  // used when H == nullptr
    const float* H;      // [N, r] kept by the caller, or nullptr
    const float* A;
    const __nv_bfloat16* dY;
    const __nv_bfloat16* X;
    __nv_bfloat16* dX;
    float* dA;
    float* dB;
};

__global__ void __launch_bounds__(256) small_bwd_finalize_kernel(const __grid_constant__ FinParams f) {
    __shared__ float sh[16 * 64];  // dH (dX, dA blocks) or s * H (dB blocks): [N][r]
    pdl_launch_dependents();
    pdl_wait();
    const int b = (int)blockIdx.x, tid = (int)threadIdx.x;
    const bool is_db = b >= f.dx_blocks && b < f.dx_blocks + f.db_blocks;
    if (f.r > 0) {
        for (int i = tid; i < f.N * f.r; i += 256) {
            float v = 0.f;
            if (!is_db) {
                for (int q = 0; q < f.dh_chunks; ++q) v += f.dHpart[(size_t)q * f.N * f.r + i];
            } else if (f.H) {
                v = f.H[i];
            } else {
                for (int q = 0; q < f.h_chunks; ++q) v += f.Hpart[(size_t)q * f.N * f.r + i];
            }
            sh[i] = f.s * v;
        }
        __syncthreads();
    }
    if (b < f.dx_blocks) {
        const int kb = (f.K + 255) / 256;
        const int n = b / kb, k = (b - n * kb) * 256 + tid;
        if (k >= f.K) return;
        float v = 0.f;
        for (int z = 0; z < f.splits; ++z) v += f.part[((size_t)z * f.N + n) * f.K + k];
        if (f.r > 0) {
            float d = 0.f;
            const float* a = f.A + (size_t)k * f.r;
            for (int j = 0; j < f.r; ++j) d = fmaf(sh[n * f.r + j], a[j], d);
            v += d;
        }
        f.dX[(size_t)n * f.K + k] = __float2bfloat16(v);
    } else if (is_db) {
        const int m = (b - f.dx_blocks) * 256 + tid;
        if (m >= f.M) return;
        float dy[16];
#pragma unroll
        for (int n = 0; n < 16; ++n) dy[n] = n < f.N ? __bfloat162float(f.dY[(size_t)n * f.M + m]) : 0.f;
        for (int j = 0; j < f.r; ++j) {
            float d = 0.f;
#pragma unroll
            for (int n = 0; n < 16; ++n)
                if (n < f.N) d = fmaf(sh[n * f.r + j], dy[n], d);
            float* o = f.dB + (size_t)j * f.M + m;
            *o = f.accumulate ? *o + d : d;
        }
    } else {
        const int k = (b - f.dx_blocks - f.db_blocks) * 256 + tid;
        if (k >= f.K) return;
        float x[16];
#pragma unroll
        for (int n = 0; n < 16; ++n) x[n] = n < f.N ? __bfloat162float(f.X[(size_t)n * f.K + k]) : 0.f;
        for (int j = 0; j < f.r; ++j) {
            float d = 0.f;
#pragma unroll
            for (int n = 0; n < 16; ++n)
                if (n < f.N) d = fmaf(x[n], sh[n * f.r + j], d);
            float* o = f.dA + (size_t)k * f.r + j;
            *o = f.accumulate ? *o + d : d;
        }
    }
}

inline size_t al256(size_t x) { return (x + 255) & ~size_t(255); }

struct Carve {
    float *part, *dHpart, *Hpart;
    size_t bytes;
};
Carve carve(const lq_weight* w, int64_t N, int r, void* base) {
    size_t off = 0;
    auto take = [&](size_t bytes) {
        size_t o = al256(off);
        off = o + bytes;
        return base ? (float*)((char*)base + o) : nullptr;
    };
    const size_t rr = (size_t)(r > 0 ? r : 1);
    Carve c;
    c.part = take((size_t)kMaxSplits * (size_t)N * (size_t)w->K * 4);
    c.dHpart = take((size_t)((w->M + kRowChunk - 1) / kRowChunk) * (size_t)N * rr * 4);
    c.Hpart = take((size_t)((w->K + kRowChunk - 1) / kRowChunk) * (size_t)N * rr * 4);
    c.bytes = al256(off);
    return c;
}

}  // namespace

bool lq_small_bwd_supported(const lq_weight* w, int64_t n_tokens, int rank) {
    static const bool off = [] {
        const char* e = getenv("LQ_NO_SMALL_BWD");
        return e && e[0] == '1';
    }();
    if (off) return false;
    return w->scheme == LQ_INT4 && (w->group == 64 || w->group == 32) && n_tokens >= 1 && n_tokens <= NT && rank <= 64 && w->K % 64 == 0 &&
           w->M % 8 == 0 && w->device >= 0;
}

size_t lq_small_bwd_workspace_bytes(const lq_weight* w, int64_t n_tokens, int rank) {
    return carve(w, n_tokens, rank, nullptr).bytes + 256;
}

void lq_small_bwd(const lq_weight* w, const void* dY, const void* X, const float* H, int64_t N, const float* A,
                  const float* B, int r, float s, void* dX, float* dA, float* dB, int accumulate, void* ws,
                  size_t ws_bytes, cudaStream_t st) {
    LQ_CHECK_ARG(ws != nullptr && ((uintptr_t)ws & 255) == 0, "workspace must be non-NULL and 256-byte aligned");
    const Carve c = carve(w, N, r, ws);
    if (c.bytes > ws_bytes)
        throw LqError(LQ_ERR_WORKSPACE, "workspace too small for the small-batch backward: need " +
                                            std::to_string(c.bytes) + " bytes, got " + std::to_string(ws_bytes));
    LQ_CHECK_ARG(((uintptr_t)dY & 15) == 0, "dY must be 16-byte aligned");
    const bool lora = r > 0 && (dX || dA || dB);
    const bool want_dh = r > 0 && (dX || dA);
    const bool want_h = r > 0 && dB && !H;
    const int sms = lq_tc_sm_count(w->device);
    BwdParams p;
    p.packed = (const uint8_t*)w->packed;
    p.scales = w->scales;
    p.M = (int)w->M;
    p.K = (int)w->K;
    p.N = (int)N;
    p.k_tiles = (int)w->k_tiles;
    p.m_tiles = (int)w->m_tiles;
    p.n_groups = (int)w->n_groups;
    p.kchunks = dX ? (p.k_tiles + KC - 1) / KC : 0;
    p.part = c.part;
    p.status = lq_tc_status_word(w->device);
    p.r = r;
    p.dh_chunks = want_dh ? (p.M + kRowChunk - 1) / kRowChunk : 0;
    p.h_chunks = want_h ? (p.K + kRowChunk - 1) / kRowChunk : 0;
    p.h_blocks = (p.dh_chunks + p.h_chunks) * (int)N;
    p.dY = (const __nv_bfloat16*)dY;
    p.X = (const __nv_bfloat16*)X;
    p.A = A;
    p.B = B;
    p.dHpart = c.dHpart;
    p.Hpart = c.Hpart;
    const int slots = std::max(sms * CTAS_PER_SM - p.h_blocks, sms);
    p.splits = 1;
    if (p.kchunks > 0) p.splits = std::max(1, std::min({slots / p.kchunks, p.m_tiles, kMaxSplits}));
    const int grid = std::min(p.kchunks * p.splits, slots) + p.h_blocks;
    if (grid > 0) {
        CUtensorMap tmDY = lq_tc_make_map(dY, w->M, N, w->M, NT);
        const bool g32 = w->group == 32;
        auto kern = N <= 8 ? (g32 ? stream_small_bwd_kernel<1, 2> : stream_small_bwd_kernel<1, 1>)
                           : (g32 ? stream_small_bwd_kernel<2, 2> : stream_small_bwd_kernel<2, 1>);
        LQ_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM));
        LqProf prof(LQ_K_GEMM_MAIN, st);
        launch_pdl(kern, dim3(grid), dim3(kThreads), SMEM, st, tmDY, p);
        LQ_CUDA(cudaGetLastError());
    }
    FinParams f;
    f.N = (int)N;
    f.K = p.K;
    f.M = p.M;
    f.r = lora ? r : 0;
    f.splits = p.splits;
    f.dh_chunks = p.dh_chunks;
    f.h_chunks = p.h_chunks;
    f.dx_blocks = dX ? (int)N * ((p.K + 255) / 256) : 0;
    f.db_blocks = (r > 0 && dB) ? (p.M + 255) / 256 : 0;
    f.da_blocks = (r > 0 && dA) ? (p.K + 255) / 256 : 0;
    f.accumulate = accumulate;
    f.s = s;
    f.part = c.part;
    f.dHpart = c.dHpart;
    f.Hpart = c.Hpart;
    f.H = H;
    f.A = A;
    f.dY = (const __nv_bfloat16*)dY;
    f.X = (const __nv_bfloat16*)X;
    f.dX = (__nv_bfloat16*)dX;
    f.dA = dA;
    f.dB = dB;
    const int fin_grid = f.dx_blocks + f.db_blocks + f.da_blocks;
    if (fin_grid > 0) {
        LqProf prof(LQ_K_REDUCE, st);
        launch_pdl(small_bwd_finalize_kernel, dim3(fin_grid), dim3(256), 0, st, f);
        LQ_CUDA(cudaGetLastError());
    }
}
