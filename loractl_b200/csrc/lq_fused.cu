// Small-batch forward: the packed-weight-stream regime (N <= 64 tokens).
//
// At N <= 64 the frozen GEMM is bound by the HBM stream of the packed weight (int4: half a byte
// per element; scaled fp8: one), so the weight is read from HBM exactly once, as stored, and
// converted on chip — no bf16 copy of the weight ever exists in HBM.  Three kernels share the work
// decomposition (128-row weight tile x k-split -> f32 partial tile; `fused_finalize_kernel` sums the
// splits in a fixed order and adds bias and s * (X.A) . B, so results are deterministic):
//
//   stream_small_fwd_kernel   int4, N <= 16: packed words -> registers -> mma.sync (see its header)
//   stream_small_fp8_kernel   scaled fp8, N <= 16: e4m3 bytes -> registers -> mma.sync
//   fused_small_fwd_kernel    int4, 17 <= N <= 64: dequantise into a shared-memory operand tile,
//                             tcgen05.mma with the weight tile as the 128-row operand (below)
//
// fused_small_fwd_kernel:  D[128 features, NT tokens] += Wt[128, 64] . Xt[NT, 64]^T
//
//   warp 0      producer: cp.async.bulk of KS packed tiles (16 KB) + their scales, one 3-D TMA box of X
//   warp 1      MMA issuer (tcgen05.mma 128 x NT x 16, f32 accumulator in TMEM)
//   warps 2-17  dequant, two groups of 8 warps on alternate k-tiles: nibbles -> exact bf16 integers
//               (0x4300 | u is 128 + u; minus 136) times the group scale, written straight into the
//               128-byte-swizzled K-major operand layout (generic-proxy stores + fence.proxy.async);
//               group 0 afterwards drains TMEM and stores the item's partial tile
//
// Scale handling there: w = bf16(q * bf16(scale)); q is exact, the scale is rounded to bf16 once per
// group (relative 2^-9), inside the bf16 path's stated tolerance.  The two register kernels apply
// the f32 scale to f32 sums instead and round no weight at all.
#include <algorithm>
#include <cstdlib>
#include <utility>

#include <cuda_fp8.h>

#include "lq_prof.cuh"
#include "lq_stream.cuh"
#include "lq_tc.cuh"
#include "lq_umma.cuh"

namespace {

using namespace umma;
using namespace lqstream;

constexpr int kFusedThreads = 64 + 512;  // producer warp, MMA warp, two dequant groups of 8 warps
constexpr int A_STAGES = 3;
constexpr uint32_t A_BYTES = 128 * 64 * 2;  // dequantised operand tile

struct FusedParams {
    const uint8_t* packed;
    const float* scales;
    int M, N;
    int k_tiles, n_groups, group;
    int m_tiles, splits;
    float* part;  // [splits][N][M]
    int* status;
    // stream kernel only: the first `h_blocks` CTAs compute H = X . A (one token each) instead of
    // weight items, so that the LoRA down-projection costs no launch of its own
    int h_blocks, r, K;
    const __nv_bfloat16* X;
    const float* A;
    float* H;
};

// Up to kMaxGroup sites that share one activation X (the reference runs `site()` on the same x for
// wq / wk / wv and for gate / up, crates/loractl-core/src/mmdit.rs:599-610,701-706) as ONE launch of
// the <= 16-token stream kernel: the work list is the concatenation of the sites' (weight tile,
// k-split) items, so launch ramp and tail are paid once per group instead of once per site.
constexpr int kMaxGroup = 4;
struct StreamGroup {
    int n_sites, n_items, n_hblocks;
    int item_end[kMaxGroup];  // running total of (m-tile, split) items up to and including site i
    int h_end[kMaxGroup];     // running total of H blocks (one per token of a site with rank > 0)
    FusedParams site[kMaxGroup];
};

constexpr int KS = 4;  // k-tiles per pipeline stage: one bulk copy moves 4 packed tiles (16 KB)

template <int NT>
struct FCfg {
    static constexpr uint32_t X_BYTES = NT * 128;                // one X tile [NT tokens][64 k] bf16
    static constexpr uint32_t RAW_BYTES = KS * (X_BYTES + 4096 + 1024);  // X tiles | packed tiles | scales
    static constexpr int RAW_STAGES = (208 * 1024 - A_STAGES * (int)A_BYTES) / (int)RAW_BYTES;
    // 2 accumulator stages x 4 independent accumulators (one per 16-wide k-step of a tile): MMAs
    // that accumulate into the same TMEM tile serialise on its latency (~200 cycles each, measured),
    // which at 128 x NT x 16 per instruction is far longer than the math; the epilogue adds the four.
    static constexpr uint32_t TMEM_COLS = NT * 8;
    static constexpr size_t SMEM = (size_t)RAW_STAGES * RAW_BYTES + A_STAGES * A_BYTES + 1024 + 512;
};

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* m, uint32_t bar, int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(dst),
        "l"((uint64_t)m), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}

// Requests to the copy engine, not bytes, bound this kernel when every k-tile is fetched by its own
// copies (three requests per 4.6 KB); a stage therefore carries KS k-tiles with three requests in
// all: one bulk copy of KS packed tiles (contiguous in the tile-major layout), one of their scales,
// and one 3-D tensor copy that lands the KS X tiles as KS separate swizzled [NT][64] tiles.
template <int NT>
__global__ void __launch_bounds__(kFusedThreads, 1)
fused_small_fwd_kernel(const __grid_constant__ CUtensorMap tmX, FusedParams p) {
    using C = FCfg<NT>;
    constexpr int RS = C::RAW_STAGES;
    extern __shared__ uint8_t smem_raw_[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw_ + 1023) & ~(uintptr_t)1023);
    uint8_t* raw = smem;                               // RS x RAW_BYTES (each 1024-aligned)
    uint8_t* abuf = smem + (size_t)RS * C::RAW_BYTES;  // A_STAGES x 16 KB
    uint64_t* bars = (uint64_t*)(abuf + A_STAGES * A_BYTES);
    uint64_t* full_raw = bars;
    uint64_t* empty_raw = bars + RS;
    uint64_t* full_a = bars + 2 * RS;
    uint64_t* empty_a = full_a + A_STAGES;
    uint64_t* tfull = empty_a + A_STAGES;
    uint64_t* tempty = tfull + 2;
    uint32_t* tmem_slot = (uint32_t*)(tempty + 2);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < RS; ++s) {
            mbar_init(smem_u32(&full_raw[s]), 1);
            mbar_init(smem_u32(&empty_raw[s]), 1);
        }
        for (int a = 0; a < A_STAGES; ++a) {
            mbar_init(smem_u32(&full_a[a]), 8);  // one arrival per dequant warp of the group that owns the tile
            mbar_init(smem_u32(&empty_a[a]), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(smem_u32(&tfull[a]), 1);
            mbar_init(smem_u32(&tempty[a]), 256);
        }
        *abort_flag = 0;
        fence_barrier_init();
        prefetch_tmap(&tmX);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), C::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int num_items = p.m_tiles * p.splits;
    const int gpt = 64 / p.group;  // scale groups per k-tile: 1 (G = 64) or 2 (G = 32)
    constexpr uint32_t X_OFF = 0, P_OFF = KS * C::X_BYTES, S_OFF = P_OFF + KS * 4096;

    if (warp == 0) {
        if (lane == 0) {
            // ---------------- producer ----------------
            int s = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int item = blockIdx.x; ok && item < num_items; item += gridDim.x) {
                const int mt = item / p.splits, z = item - mt * p.splits;
                const int kt0 = (int)(((long long)z * p.k_tiles) / p.splits);
                const int kt1 = (int)(((long long)(z + 1) * p.k_tiles) / p.splits);
                for (int kt = kt0; kt < kt1; kt += KS) {
                    if (!mbar_wait(smem_u32(&empty_raw[s]), phase ^ 1u, abort_flag, p.status, 21)) { ok = false; break; }
                    const uint32_t bar = smem_u32(&full_raw[s]);
                    const uint32_t base = smem_u32(raw + (size_t)s * C::RAW_BYTES);
                    const int tiles = min(KS, kt1 - kt);
                    const uint32_t pk_bytes = (uint32_t)tiles * 4096u, sc_bytes = (uint32_t)(tiles * gpt) * 512u;
                    mbar_expect_tx(bar, KS * C::X_BYTES + pk_bytes + sc_bytes);  // the X box is always whole
                    tma_load_3d(base + X_OFF, &tmX, bar, 0, 0, kt);
                    bulk_load(base + P_OFF, p.packed + ((size_t)mt * p.k_tiles + kt) * 4096, pk_bytes, bar);
                    bulk_load(base + S_OFF, p.scales + ((size_t)mt * p.n_groups + (size_t)kt * gpt) * 128, sc_bytes, bar);
                    if (++s == RS) { s = 0; phase ^= 1u; }
                }
            }
            if (!ok)
                for (int i = 0; i < 64; ++i) __nanosleep(1000);
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---------------- MMA issuer ----------------
            constexpr uint32_t idesc = make_idesc(1, 1, false, false, 128, NT);
            const uint32_t d_hi = desc_hi(1024);
            const uint32_t a_lo0 = desc_lo(smem_u32(abuf), 16), x_lo0 = desc_lo(smem_u32(raw + X_OFF), 16);
            int s = 0, a = 0, acc = 0;
            uint32_t phase = 0, aphase = 0, acc_phase = 0;
            bool ok = true;
            for (int item = blockIdx.x; ok && item < num_items; item += gridDim.x) {
                const int mt = item / p.splits, z = item - mt * p.splits;
                const int kt0 = (int)(((long long)z * p.k_tiles) / p.splits);
                const int kt1 = (int)(((long long)(z + 1) * p.k_tiles) / p.splits);
                if (!mbar_wait(smem_u32(&tempty[acc]), acc_phase ^ 1u, abort_flag, p.status, 22)) { ok = false; break; }
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + (uint32_t)(acc * 4 * NT);
                for (int kt = kt0; ok && kt < kt1; kt += KS) {
                    if (!mbar_wait(smem_u32(&full_raw[s]), phase, abort_flag, p.status, 24)) { ok = false; break; }
                    const int tiles = min(KS, kt1 - kt);
                    const uint32_t x_lo = x_lo0 + (uint32_t)s * (C::RAW_BYTES >> 4);
                    for (int j = 0; j < tiles; ++j) {
                        if (!mbar_wait(smem_u32(&full_a[a]), aphase, abort_flag, p.status, 23)) { ok = false; break; }
                        tc_fence_after();
                        const uint32_t a_lo = a_lo0 + (uint32_t)a * (A_BYTES >> 4);
                        const uint32_t xj_lo = x_lo + (uint32_t)j * (C::X_BYTES >> 4);
                        const uint32_t accum = (kt > kt0 || j > 0) ? 1u : 0u;
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            mma_f16(tmem_d + (uint32_t)(k * NT), desc_join(a_lo + k * 2u, d_hi), desc_join(xj_lo + k * 2u, d_hi),
                                    idesc, accum);
                        mma_commit(smem_u32(&empty_a[a]));
                        if (++a == A_STAGES) { a = 0; aphase ^= 1u; }
                    }
                    if (!ok) break;
                    mma_commit(smem_u32(&empty_raw[s]));  // the stage (packed tiles, scales, X tiles) is free again
                    if (++s == RS) { s = 0; phase ^= 1u; }
                }
                if (!ok) break;
                mma_commit(smem_u32(&tfull[acc]));
                if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
            }
        }
    } else {
        // ---------------- dequant (warps 2..17: two groups of 256 threads) + epilogue (group 0) --------
        // The groups take alternate k-tiles, so two tiles are converted concurrently; ring positions
        // are derived from running counts that both groups advance identically.
        const int grp = (warp - 2) >> 3;
        const int dt = (threadIdx.x - 64) & 255;
        const int r = dt >> 1, half = dt & 1;      // row of the tile, 32-k half of it
        const int quarter = warp & 3;              // TMEM lane quarter of this warp
        const int chalf = ((warp - 2) >> 2) & 1;   // which half of the NT columns this warp drains
        int acc = 0;
        uint32_t acc_phase = 0, tix = 0, six = 0;  // running k-tile / stage counts
        bool ok = true;
        const __nv_bfloat162 off = __float2bfloat162_rn(136.f);
        for (int item = blockIdx.x; ok && item < num_items; item += gridDim.x) {
            const int mt = item / p.splits, z = item - mt * p.splits;
            const int kt0 = (int)(((long long)z * p.k_tiles) / p.splits);
            const int kt1 = (int)(((long long)(z + 1) * p.k_tiles) / p.splits);
            for (int kt = kt0; ok && kt < kt1; kt += KS, ++six) {
                const int s = (int)(six % RS);
                if (!mbar_wait(smem_u32(&full_raw[s]), (six / RS) & 1u, abort_flag, p.status, 25)) { ok = false; break; }
                const int tiles = min(KS, kt1 - kt);
                const uint8_t* stage = raw + (size_t)s * C::RAW_BYTES;
                for (int j = 0; j < tiles; ++j, ++tix) {
                    if ((int)(tix & 1u) != grp) continue;
                    const int a = (int)(tix % A_STAGES);
                    if (!mbar_wait(smem_u32(&empty_a[a]), ((tix / A_STAGES) & 1u) ^ 1u, abort_flag, p.status, 26)) { ok = false; break; }
                    const uint4 v = *((const uint4*)(stage + P_OFF + j * 4096) + dt);  // row r, chunks half*4..+3
                    const int gi = gpt == 2 ? half : 0;
                    const float sc = *((const float*)(stage + S_OFF) + (j * gpt + gi) * 128 + r);
                    const __nv_bfloat162 s2 = __float2bfloat162_rn(sc);
                    const uint32_t words[4] = {v.x, v.y, v.z, v.w};
                    uint8_t* arow = abuf + (size_t)a * A_BYTES + r * 128;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        uint32_t o[4];
#pragma unroll
                        for (int jj = 0; jj < 4; ++jj) {
                            uint32_t t = ((words[i] >> (4 * jj)) & 0x000F000Fu) | 0x43004300u;  // (128+u_lo, 128+u_hi)
                            __nv_bfloat162 q = __hsub2(*(__nv_bfloat162*)&t, off);             // exact integers -7..7
                            __nv_bfloat162 wv = __hmul2(q, s2);
                            o[jj] = *(uint32_t*)&wv;
                        }
                        const int chunk = (half * 4 + i) ^ (r & 7);  // 128-byte swizzle of the operand layout
                        *(uint4*)(arow + chunk * 16) = make_uint4(o[0], o[1], o[2], o[3]);
                    }
                    // every lane publishes its stores to the async proxy; the warp then arrives once
                    // (256 per-thread arrivals on one barrier serialise and cost more than the tile)
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(&full_a[a]));
                }
            }
            if (!ok) break;
            if (grp != 0) continue;
            // ---- epilogue of this item (group 0): D[m, n] -> part[z][n][m] ----
            if (!mbar_wait(smem_u32(&tfull[acc]), acc_phase, abort_flag, p.status, 27)) { ok = false; break; }
            tc_fence_after();
            const int m = mt * 128 + quarter * 32 + lane;
            float* pz = p.part + (size_t)z * p.N * p.M;
#pragma unroll 1
            for (int c = 0; c < NT / 2; c += 8) {
                uint32_t r0[8], r1[8], r2[8], r3[8];
                const int col0 = chalf * (NT / 2) + c;
                const uint32_t ta = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * 4 * NT + col0);
                tmem_ld_x8(ta, r0);
                tmem_ld_x8(ta + NT, r1);
                tmem_ld_x8(ta + 2 * NT, r2);
                tmem_ld_x8(ta + 3 * NT, r3);
                tmem_ld_wait();
                if (m < p.M) {
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        const int n = col0 + e;
                        const float v = (__uint_as_float(r0[e]) + __uint_as_float(r1[e])) +
                                        (__uint_as_float(r2[e]) + __uint_as_float(r3[e]));
                        if (n < p.N) pz[(size_t)n * p.M + m] = v;
                    }
                }
            }
            tc_fence_before();
            mbar_arrive(smem_u32(&tempty[acc]));
            if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, C::TMEM_COLS);
    }
}

// ---------------------------------------------------------------------------------------------
// N <= 16 tokens: register-dequant stream kernel.
//
// With so few tokens the tensor work per weight byte is tiny and the tcgen05 route above pays a
// shared-memory round trip (packed -> bf16 operand tile) plus a fixed cost per MMA instruction.
// Here the packed words go shared memory -> registers -> legacy warp MMA (mma.sync m16n8k16,
// weights as the 16-row operand, 8 tokens as the narrow one) with nothing written back to shared
// memory.  The instruction count per weight is what bounds this kernel, so the conversion is as
// lean as the format allows: `(word >> 4j) & 0x000F000F | 0x43004300` is the bf16 pair
// (128 + u, 128 + u') with u = q + 8, and it goes into the MMA as it is.  The excess
// 136 * sum_k x[n, k] is the same for every weight row: one MMA with an all-ones operand yields
// the token sums of the k-tile, and the accumulator of every row block starts from -136 times
// them.  The group scale multiplies the f32 partial sum of its group instead of the weights, so
// no weight is ever rounded (q exact, scale f32).
//
//   warp 0     producer, as above (one bulk copy of KS packed tiles, one of their scales, one
//              3-D tensor copy of the KS X tiles [16 tokens][64 k], 128-byte swizzled)
//   warps 1-4  consumers; warp w owns rows 32w .. 32w+31 of the 128-row tile (two m16 blocks)
//
// Fragment mapping.  The contraction index may be permuted freely as long as both operands use
// the same permutation.  Lane (g = lane >> 2, t = lane & 3) reads, for rows g and g + 8 of a
// block, word t (k = 8t .. 8t+7) and word 4 + t (k = 32 + 8t ..) of the row: each word feeds two
// k16 steps, the pairs (e0,e1) | (e2,e3) then (e4,e5) | (e6,e7).  The matching X fragment is the
// 16-byte chunk t (resp. 4 + t) of a token row, one LDS.128.  Steps 0-1 lie in k < 32 and steps
// 2-3 in k >= 32, so a group of 32 never mixes with its neighbour.  Fragment column g holds token
// (g >> 1) + 4 (g & 1) of its block of 8, which makes the swizzled X reads conflict-free.
//
// Partial tiles go to part[z][n][m] like the tcgen05 kernel's; fused_finalize_kernel sums the splits.
// (Letting the CTA that arrives last at a tile finish Y in-kernel was measured: the counter reset plus
// the serial tail cost more than the second launch saves at these sizes.)
constexpr int kStreamThreads = 32 + 128;
constexpr int STREAM_NT = 16;  // token rows of the X box
constexpr uint32_t STREAM_X_BYTES = STREAM_NT * 128;
constexpr uint32_t STREAM_RAW_BYTES = KS * (STREAM_X_BYTES + 4096 + 1024);
constexpr int STREAM_STAGES = 2;
constexpr size_t STREAM_SMEM = (size_t)STREAM_STAGES * STREAM_RAW_BYTES + 1024 + 128;
constexpr int STREAM_CTAS_PER_SM = 3;

__device__ __forceinline__ uint32_t dq_pair(uint32_t w, int sh) {
    return ((w >> sh) & 0x000F000Fu) | 0x43004300u;  // (128 + u_lo, 128 + u_hi) as bf16
}

// Two k16 steps: word `wg` of row g and `wh` of row g + 8 against the X chunk(s) `x`.
template <int NB>
__device__ __forceinline__ void half_mma(uint32_t wg, uint32_t wh, const uint4 (&x)[NB], float (&acc)[NB][4]) {
    const uint32_t a0 = dq_pair(wg, 0), a1 = dq_pair(wh, 0), a2 = dq_pair(wg, 4), a3 = dq_pair(wh, 4);
    const uint32_t c0 = dq_pair(wg, 8), c1 = dq_pair(wh, 8), c2 = dq_pair(wg, 12), c3 = dq_pair(wh, 12);
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
        mma_16816(acc[nb], a0, a1, a2, a3, x[nb].x, x[nb].y);
        mma_16816(acc[nb], c0, c1, c2, c3, x[nb].z, x[nb].w);
    }
}

// -136 * (sum of the 32 k of one X chunk pair), per token column of the fragment.
template <int NB>
__device__ __forceinline__ void half_offset(const uint4 (&x)[NB], float (&o)[NB][2], bool accumulate) {
    constexpr uint32_t ONES = 0x3F803F80u;  // bf16 (1, 1)
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
        float one[4] = {0.f, 0.f, 0.f, 0.f};
        mma_16816(one, ONES, ONES, ONES, ONES, x[nb].x, x[nb].y);
        mma_16816(one, ONES, ONES, ONES, ONES, x[nb].z, x[nb].w);
        o[nb][0] = accumulate ? fmaf(-136.f, one[0], o[nb][0]) : -136.f * one[0];
        o[nb][1] = accumulate ? fmaf(-136.f, one[1], o[nb][1]) : -136.f * one[1];
    }
}

// H[n, :] = X[n, :] . A for one token by one CTA of kStreamThreads threads, f32 accumulation; 16
// rank columns at a time, fixed shuffle tree then a fixed-order pass over the warps (deterministic).
__device__ __forceinline__ void stream_h_block(const FusedParams& p, int n, float* red /* [5][16] */) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const __nv_bfloat16* x = p.X + (size_t)n * p.K;
    for (int j0 = 0; j0 < p.r; j0 += 16) {
        float acc[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) acc[j] = 0.f;
        const bool vec = (p.r - j0 >= 16) && (p.r % 4 == 0) && (((uintptr_t)p.A & 15) == 0);
#pragma unroll 2
        for (int k = tid; k < p.K; k += kStreamThreads) {
            const float xv = __bfloat162float(x[k]);
            const float* arow = p.A + (size_t)k * p.r + j0;
            if (vec) {
#pragma unroll
                for (int j = 0; j < 16; j += 4) {
                    const float4 a4 = *(const float4*)(arow + j);
                    acc[j] = fmaf(xv, a4.x, acc[j]);
                    acc[j + 1] = fmaf(xv, a4.y, acc[j + 1]);
                    acc[j + 2] = fmaf(xv, a4.z, acc[j + 2]);
                    acc[j + 3] = fmaf(xv, a4.w, acc[j + 3]);
                }
            } else {
#pragma unroll
                for (int j = 0; j < 16; ++j)
                    if (j0 + j < p.r) acc[j] = fmaf(xv, arow[j], acc[j]);
            }
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            float v = acc[j];
#pragma unroll
            for (int off = 16; off >= 1; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
            if (lane == 0) red[warp * 16 + j] = v;
        }
        __syncthreads();
        if (tid < 16 && j0 + tid < p.r) {
            float h = 0.f;
#pragma unroll
            for (int w5 = 0; w5 < kStreamThreads / 32; ++w5) h += red[w5 * 16 + tid];
            p.H[(size_t)n * p.r + j0 + tid] = h;
        }
        __syncthreads();
    }
}

// The kernel is instantiated for one site (parameters are plain kernel arguments, i.e. instruction
// operands) and for a group (parameters indexed by site, i.e. loads from parameter space: a
// single-site launch through the group form measured 12.7 us per 3072 x 3072 site against 8.6 us).
struct SiteRegs {
    const uint8_t* packed;
    const float* scales;
    float* part;
    int k_tiles, n_groups, splits, N, M;
};
__device__ __forceinline__ int sg_items(const FusedParams& p) { return p.m_tiles * p.splits; }
__device__ __forceinline__ int sg_items(const StreamGroup& g) { return g.n_items; }
__device__ __forceinline__ int sg_hblocks(const FusedParams& p) { return p.h_blocks; }
__device__ __forceinline__ int sg_hblocks(const StreamGroup& g) { return g.n_hblocks; }
__device__ __forceinline__ int sg_group(const FusedParams& p) { return p.group; }
__device__ __forceinline__ int sg_group(const StreamGroup& g) { return g.site[0].group; }
__device__ __forceinline__ int* sg_status(const FusedParams& p) { return p.status; }
__device__ __forceinline__ int* sg_status(const StreamGroup& g) { return g.site[0].status; }
__device__ __forceinline__ void sg_fill(const FusedParams& p, SiteRegs& r) {
    r.packed = p.packed; r.scales = p.scales; r.part = p.part;
    r.k_tiles = p.k_tiles; r.n_groups = p.n_groups; r.splits = p.splits; r.N = p.N; r.M = p.M;
}
// item -> (site registers, item index within the site); `si` persists across calls (items only grow)
__device__ __forceinline__ int sg_site(const FusedParams& p, int item, int&, SiteRegs& r) {
    sg_fill(p, r);
    return item;
}
// Every index into the group is a literal, so that the fields stay instruction operands (unused
// slots of item_end / h_end hold INT_MAX).
__device__ __forceinline__ int sg_site(const StreamGroup& g, int item, int& si, SiteRegs& r) {
    static_assert(kMaxGroup == 4, "the selects below are written out for four sites");
    si = (item >= g.item_end[0]) + (item >= g.item_end[1]) + (item >= g.item_end[2]);
    switch (si) {
        case 0: sg_fill(g.site[0], r); return item;
        case 1: sg_fill(g.site[1], r); return item - g.item_end[0];
        case 2: sg_fill(g.site[2], r); return item - g.item_end[1];
        default: sg_fill(g.site[3], r); return item - g.item_end[2];
    }
}
__device__ __forceinline__ void sg_hblock(const FusedParams& p, int blk, float* red) { stream_h_block(p, blk, red); }
__device__ __forceinline__ void sg_hblock(const StreamGroup& g, int blk, float* red) {
    const int si = (blk >= g.h_end[0]) + (blk >= g.h_end[1]) + (blk >= g.h_end[2]);
    switch (si) {
        case 0: stream_h_block(g.site[0], blk, red); break;
        case 1: stream_h_block(g.site[1], blk - g.h_end[0], red); break;
        case 2: stream_h_block(g.site[2], blk - g.h_end[1], red); break;
        default: stream_h_block(g.site[3], blk - g.h_end[2], red); break;
    }
}

template <int NB, typename G>
__global__ void __launch_bounds__(kStreamThreads, STREAM_CTAS_PER_SM)
stream_small_fwd_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ G gp) {
    constexpr int RS = STREAM_STAGES;
    extern __shared__ uint8_t smem_raw_[];
    uint8_t* raw = (uint8_t*)(((uintptr_t)smem_raw_ + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = (uint64_t*)(raw + (size_t)RS * STREAM_RAW_BYTES);
    uint64_t* full_raw = bars;
    uint64_t* empty_raw = bars + RS;
    volatile int* abort_flag = (volatile int*)(bars + 2 * RS);

    pdl_launch_dependents();
    pdl_wait();
    const int h_blocks = sg_hblocks(gp);
    if ((int)blockIdx.x < h_blocks) {  // uniform per CTA: one token of one site's H = X . A
        sg_hblock(gp, (int)blockIdx.x, (float*)raw);
        return;
    }
    const int first = (int)blockIdx.x - h_blocks, stride = (int)gridDim.x - h_blocks;
    int* status = sg_status(gp);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < RS; ++s) {
            mbar_init(smem_u32(&full_raw[s]), 1);
            mbar_init(smem_u32(&empty_raw[s]), 4);  // one arrival per consumer warp
        }
        *abort_flag = 0;
        fence_barrier_init();
        prefetch_tmap(&tmX);
    }
    __syncthreads();

    const int num_items = sg_items(gp);
    const int gpt = 64 / sg_group(gp);  // the sites of a group share d_in and the quant block
    constexpr uint32_t X_OFF = 0, P_OFF = KS * STREAM_X_BYTES, S_OFF = P_OFF + KS * 4096;

    if (warp == 0) {
        if (lane == 0) {
            int s = 0;
            uint32_t phase = 0;
            bool ok = true;
            int si = 0;
            for (int item = first; ok && item < num_items; item += stride) {
                SiteRegs p;  // the site's fields, in registers once per item
                const int li = sg_site(gp, item, si, p);
                const int splits = p.splits;
                const int mt = li / splits, z = li - mt * splits;
                const int kt0 = (int)(((long long)z * p.k_tiles) / splits);
                const int kt1 = (int)(((long long)(z + 1) * p.k_tiles) / splits);
                for (int kt = kt0; kt < kt1; kt += KS) {
                    if (!mbar_wait(smem_u32(&empty_raw[s]), phase ^ 1u, abort_flag, status, 31)) { ok = false; break; }
                    const uint32_t bar = smem_u32(&full_raw[s]);
                    const uint32_t base = smem_u32(raw + (size_t)s * STREAM_RAW_BYTES);
                    const int tiles = min(KS, kt1 - kt);
                    const uint32_t pk_bytes = (uint32_t)tiles * 4096u, sc_bytes = (uint32_t)(tiles * gpt) * 512u;
                    mbar_expect_tx(bar, KS * STREAM_X_BYTES + pk_bytes + sc_bytes);  // the X box is always whole
                    tma_load_3d(base + X_OFF, &tmX, bar, 0, 0, kt);
                    bulk_load(base + P_OFF, p.packed + ((size_t)mt * p.k_tiles + kt) * 4096, pk_bytes, bar);
                    bulk_load(base + S_OFF, p.scales + ((size_t)mt * p.n_groups + (size_t)kt * gpt) * 128, sc_bytes, bar);
                    if (++s == RS) { s = 0; phase ^= 1u; }
                }
            }
            if (!ok)
                for (int i = 0; i < 64; ++i) __nanosleep(1000);
        }
        return;
    }

    // ---------------- consumers ----------------
    const int cw = warp - 1, g = lane >> 2, t = lane & 3;
    const int tok = (g >> 1) + 4 * (g & 1);  // token (within a block of 8) held by fragment column g
    const uint32_t x_lo_off = (uint32_t)tok * 128u + (((uint32_t)t ^ (uint32_t)tok) << 4);
    const uint32_t x_hi_off = (uint32_t)tok * 128u + (((uint32_t)(4 + t) ^ (uint32_t)tok) << 4);
    const uint32_t w_off = (uint32_t)((cw * 32 + g) * 8 + t);  // word index of (row g of block 0, word t)

    int s = 0;
    uint32_t phase = 0;
    bool ok = true;
    int si = 0;
    for (int item = first; ok && item < num_items; item += stride) {
        SiteRegs p;
        const int li = sg_site(gp, item, si, p);
        const int splits = p.splits, k_tiles = p.k_tiles;
        const int mt = li / splits, z = li - mt * splits;
        const int kt0 = (int)(((long long)z * k_tiles) / splits);
        const int kt1 = (int)(((long long)(z + 1) * k_tiles) / splits);
        float tot[2][NB][4];
#pragma unroll
        for (int mb = 0; mb < 2; ++mb)
#pragma unroll
            for (int nb = 0; nb < NB; ++nb)
#pragma unroll
                for (int e = 0; e < 4; ++e) tot[mb][nb][e] = 0.f;
        for (int kt = kt0; ok && kt < kt1; kt += KS) {
            if (!mbar_wait(smem_u32(&full_raw[s]), phase, abort_flag, status, 32)) { ok = false; break; }
            const int tiles = min(KS, kt1 - kt);
            const uint8_t* stage = raw + (size_t)s * STREAM_RAW_BYTES;
#pragma unroll 2
            for (int j = 0; j < tiles; ++j) {
                const uint8_t* xs = stage + X_OFF + j * STREAM_X_BYTES;
                uint4 xlo[NB], xhi[NB];
#pragma unroll
                for (int nb = 0; nb < NB; ++nb) {
                    xlo[nb] = *(const uint4*)(xs + nb * 1024 + x_lo_off);
                    xhi[nb] = *(const uint4*)(xs + nb * 1024 + x_hi_off);
                }
                const uint32_t* pk = (const uint32_t*)(stage + P_OFF + j * 4096) + w_off;
                const float* sc = (const float*)(stage + S_OFF) + (size_t)(j * gpt) * 128 + cw * 32 + g;
                float o_lo[NB][2], o_hi[NB][2];
                half_offset<NB>(xlo, o_lo, false);
                if (gpt == 2) {
                    half_offset<NB>(xhi, o_hi, false);
                } else {
                    half_offset<NB>(xhi, o_lo, true);
                }
#pragma unroll
                for (int mb = 0; mb < 2; ++mb) {
                    const uint32_t wg0 = pk[mb * 128], wg1 = pk[mb * 128 + 4];
                    const uint32_t wh0 = pk[mb * 128 + 64], wh1 = pk[mb * 128 + 68];
                    float acc[NB][4];
#pragma unroll
                    for (int nb = 0; nb < NB; ++nb) {
                        acc[nb][0] = acc[nb][2] = o_lo[nb][0];
                        acc[nb][1] = acc[nb][3] = o_lo[nb][1];
                    }
                    half_mma<NB>(wg0, wh0, xlo, acc);
                    if (gpt == 2) {
                        const float s0 = sc[mb * 16], s1 = sc[mb * 16 + 8];
#pragma unroll
                        for (int nb = 0; nb < NB; ++nb) {
                            tot[mb][nb][0] = fmaf(s0, acc[nb][0], tot[mb][nb][0]);
                            tot[mb][nb][1] = fmaf(s0, acc[nb][1], tot[mb][nb][1]);
                            tot[mb][nb][2] = fmaf(s1, acc[nb][2], tot[mb][nb][2]);
                            tot[mb][nb][3] = fmaf(s1, acc[nb][3], tot[mb][nb][3]);
                            acc[nb][0] = acc[nb][2] = o_hi[nb][0];
                            acc[nb][1] = acc[nb][3] = o_hi[nb][1];
                        }
                    }
                    half_mma<NB>(wg1, wh1, xhi, acc);
                    const float* sc1 = sc + (gpt == 2 ? 128 : 0);
                    const float s0 = sc1[mb * 16], s1 = sc1[mb * 16 + 8];
#pragma unroll
                    for (int nb = 0; nb < NB; ++nb) {
                        tot[mb][nb][0] = fmaf(s0, acc[nb][0], tot[mb][nb][0]);
                        tot[mb][nb][1] = fmaf(s0, acc[nb][1], tot[mb][nb][1]);
                        tot[mb][nb][2] = fmaf(s1, acc[nb][2], tot[mb][nb][2]);
                        tot[mb][nb][3] = fmaf(s1, acc[nb][3], tot[mb][nb][3]);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&empty_raw[s]));
            if (++s == RS) { s = 0; phase ^= 1u; }
        }
        if (!ok) break;
        // partial tile of this item: fragment columns 2t, 2t+1 hold tokens t and t + 4 of the block
        float* pz = p.part + (size_t)z * p.N * p.M;
#pragma unroll
        for (int mb = 0; mb < 2; ++mb) {
            const int m0 = mt * 128 + cw * 32 + mb * 16 + g;
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) {
                const int n0 = nb * 8 + t, n1 = n0 + 4;
                if (m0 < p.M) {
                    if (n0 < p.N) pz[(size_t)n0 * p.M + m0] = tot[mb][nb][0];
                    if (n1 < p.N) pz[(size_t)n1 * p.M + m0] = tot[mb][nb][1];
                }
                if (m0 + 8 < p.M) {
                    if (n0 < p.N) pz[(size_t)n0 * p.M + m0 + 8] = tot[mb][nb][2];
                    if (n1 < p.N) pz[(size_t)n1 * p.M + m0 + 8] = tot[mb][nb][3];
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// N <= 16 tokens, scaled-fp8 weights: the same register route over the file's row-major e4m3 bytes.
//
// A stage is one 2-D tensor copy of [128 weight rows][128 bytes of k] (two k-tiles, 128-byte
// swizzled) plus the matching two X tiles.  Lane (g, t) reads the 16-byte chunk t (+4 for the second
// k-tile) of fragment rows g and g + 8: four 32-bit words = four k16 steps, each word giving the
// pairs (b0,b1) | (b2,b3); e4m3 pairs become bf16 pairs through the hardware e4m3x2 -> f16x2
// conversion (exact) and an f16 -> f32 -> bf16 round trip (exact as well: 3 mantissa bits).  The X
// fragment is the 32 bytes k = 16t .. 16t+15 of a token row.  Fragment row g stands for tile row
// (g >> 1) + 4 (g & 1) of its group of 8 so that the swizzled reads of two rows never share a bank
// group.  The per-channel (or scalar) f32 scale multiplies the finished row sums, so no weight is
// rounded.  Partials and the H rows are handled as in the int4 kernel.
constexpr int KS_F8 = 2;
constexpr uint32_t F8_W_BYTES = 128 * 128;
constexpr uint32_t F8_RAW_BYTES = KS_F8 * STREAM_X_BYTES + F8_W_BYTES;
constexpr int F8_STAGES = 3;
constexpr size_t F8_SMEM = (size_t)F8_STAGES * F8_RAW_BYTES + 1024 + 128;

__device__ __forceinline__ uint32_t e4m3x2_to_bf16x2(uint32_t two_bytes) {
    const __half2_raw hr = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(two_bytes & 0xFFFFu), __NV_E4M3);
    const float2 f = __half22float2(*(const __half2*)&hr);
    const __nv_bfloat162 b = __floats2bfloat162_rn(f.x, f.y);
    return *(const uint32_t*)&b;
}

struct StreamF8Params {
    FusedParams base;       // packed / scales / group unused
    const float* wscale;    // [M] or [1]
    int per_channel;
};

template <int NB>
__global__ void __launch_bounds__(kStreamThreads, STREAM_CTAS_PER_SM)
stream_small_fp8_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW, StreamF8Params q) {
    const FusedParams& p = q.base;
    constexpr int RS = F8_STAGES;
    extern __shared__ uint8_t smem_raw_[];
    uint8_t* raw = (uint8_t*)(((uintptr_t)smem_raw_ + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = (uint64_t*)(raw + (size_t)RS * F8_RAW_BYTES);
    uint64_t* full_raw = bars;
    uint64_t* empty_raw = bars + RS;
    volatile int* abort_flag = (volatile int*)(bars + 2 * RS);

    pdl_launch_dependents();
    pdl_wait();
    if ((int)blockIdx.x < p.h_blocks) {  // uniform per CTA
        stream_h_block(p, (int)blockIdx.x, (float*)raw);
        return;
    }
    const int first = (int)blockIdx.x - p.h_blocks, stride = (int)gridDim.x - p.h_blocks;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < RS; ++s) {
            mbar_init(smem_u32(&full_raw[s]), 1);
            mbar_init(smem_u32(&empty_raw[s]), 4);
        }
        *abort_flag = 0;
        fence_barrier_init();
        prefetch_tmap(&tmX);
        prefetch_tmap(&tmW);
    }
    __syncthreads();

    const int num_items = p.m_tiles * p.splits;
    constexpr uint32_t W_OFF = 0, X_OFF = F8_W_BYTES;  // the weight box wants 1024-byte alignment; so do the X tiles

    if (warp == 0) {
        if (lane == 0) {
            int s = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int item = first; ok && item < num_items; item += stride) {
                const int mt = item / p.splits, z = item - mt * p.splits;
                const int kt0 = (int)(((long long)z * p.k_tiles) / p.splits) & ~1;  // splits start on a 128-byte box
                const int kt1 = z + 1 == p.splits ? p.k_tiles : ((int)(((long long)(z + 1) * p.k_tiles) / p.splits) & ~1);
                for (int kt = kt0; kt < kt1; kt += KS_F8) {
                    if (!mbar_wait(smem_u32(&empty_raw[s]), phase ^ 1u, abort_flag, p.status, 33)) { ok = false; break; }
                    const uint32_t bar = smem_u32(&full_raw[s]);
                    const uint32_t base = smem_u32(raw + (size_t)s * F8_RAW_BYTES);
                    mbar_expect_tx(bar, F8_RAW_BYTES);  // both boxes are always whole (out-of-range parts are zero-filled)
                    tma_load_2d(base + W_OFF, &tmW, bar, kt * 64, mt * 128);
                    tma_load_3d(base + X_OFF, &tmX, bar, 0, 0, kt);
                    if (++s == RS) { s = 0; phase ^= 1u; }
                }
            }
            if (!ok)
                for (int i = 0; i < 64; ++i) __nanosleep(1000);
        }
        return;
    }

    // ---------------- consumers ----------------
    const int cw = warp - 1, g = lane >> 2, t = lane & 3;
    const int rho = (g >> 1) + 4 * (g & 1);  // tile row (within a group of 8) held by fragment row g
    const uint32_t x_off = (uint32_t)g * 128u;  // token g of a block of 8; chunks 2t, 2t+1 swizzled by (g & 7)
    const uint32_t xc0 = ((uint32_t)(2 * t) ^ (uint32_t)g) << 4, xc1 = ((uint32_t)(2 * t + 1) ^ (uint32_t)g) << 4;
    int s = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int item = first; ok && item < num_items; item += stride) {
        const int mt = item / p.splits, z = item - mt * p.splits;
        const int kt0 = (int)(((long long)z * p.k_tiles) / p.splits) & ~1;
        const int kt1 = z + 1 == p.splits ? p.k_tiles : ((int)(((long long)(z + 1) * p.k_tiles) / p.splits) & ~1);
        float tot[2][NB][4];
#pragma unroll
        for (int mb = 0; mb < 2; ++mb)
#pragma unroll
            for (int nb = 0; nb < NB; ++nb)
#pragma unroll
                for (int e = 0; e < 4; ++e) tot[mb][nb][e] = 0.f;
        for (int kt = kt0; ok && kt < kt1; kt += KS_F8) {
            if (!mbar_wait(smem_u32(&full_raw[s]), phase, abort_flag, p.status, 34)) { ok = false; break; }
            const uint8_t* stage = raw + (size_t)s * F8_RAW_BYTES;
#pragma unroll
            for (int j = 0; j < KS_F8; ++j) {
                const uint8_t* xs = stage + X_OFF + j * STREAM_X_BYTES;
                uint4 xa[NB], xb[NB];
#pragma unroll
                for (int nb = 0; nb < NB; ++nb) {
                    xa[nb] = *(const uint4*)(xs + nb * 1024 + x_off + xc0);
                    xb[nb] = *(const uint4*)(xs + nb * 1024 + x_off + xc1);
                }
#pragma unroll
                for (int mb = 0; mb < 2; ++mb) {
                    const int r0 = cw * 32 + mb * 16 + rho;  // rows r0 and r0 + 8 of the tile; (r0 & 7) == rho
                    const uint32_t c = ((uint32_t)(4 * j + t) ^ (uint32_t)rho) << 4;
                    const uint4 wg = *(const uint4*)(stage + W_OFF + (uint32_t)r0 * 128u + c);
                    const uint4 wh = *(const uint4*)(stage + W_OFF + (uint32_t)(r0 + 8) * 128u + c);
                    const uint32_t g4[4] = {wg.x, wg.y, wg.z, wg.w}, h4[4] = {wh.x, wh.y, wh.z, wh.w};
#pragma unroll
                    for (int st = 0; st < 4; ++st) {
                        const uint32_t a0 = e4m3x2_to_bf16x2(g4[st]), a2 = e4m3x2_to_bf16x2(g4[st] >> 16);
                        const uint32_t a1 = e4m3x2_to_bf16x2(h4[st]), a3 = e4m3x2_to_bf16x2(h4[st] >> 16);
#pragma unroll
                        for (int nb = 0; nb < NB; ++nb) {
                            const uint4& xv = st < 2 ? xa[nb] : xb[nb];
                            const uint32_t b0 = (st & 1) ? xv.z : xv.x, b1 = (st & 1) ? xv.w : xv.y;
                            mma_16816(tot[mb][nb], a0, a1, a2, a3, b0, b1);
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&empty_raw[s]));
            if (++s == RS) { s = 0; phase ^= 1u; }
        }
        if (!ok) break;
        float* pz = p.part + (size_t)z * p.N * p.M;
#pragma unroll
        for (int mb = 0; mb < 2; ++mb) {
            const int m0 = mt * 128 + cw * 32 + mb * 16 + rho;
            const float s0 = m0 < p.M ? (q.per_channel ? q.wscale[m0] : q.wscale[0]) : 0.f;
            const float s1 = m0 + 8 < p.M ? (q.per_channel ? q.wscale[m0 + 8] : q.wscale[0]) : 0.f;
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) {
                const int n0 = nb * 8 + 2 * t, n1 = n0 + 1;  // fragment columns 2t, 2t+1 are tokens 2t, 2t+1
                if (m0 < p.M) {
                    if (n0 < p.N) pz[(size_t)n0 * p.M + m0] = s0 * tot[mb][nb][0];
                    if (n1 < p.N) pz[(size_t)n1 * p.M + m0] = s0 * tot[mb][nb][1];
                }
                if (m0 + 8 < p.M) {
                    if (n0 < p.N) pz[(size_t)n0 * p.M + m0 + 8] = s1 * tot[mb][nb][2];
                    if (n1 < p.N) pz[(size_t)n1 * p.M + m0 + 8] = s1 * tot[mb][nb][3];
                }
            }
        }
    }
}

// Second stage: Y[n, m] = bf16( sum_z part[z][n][m] + bias[m] + s * sum_j H[n, j] * B[j, m] ).
// One thread per output: at these sizes the kernel is bound by the latency of its few dependent
// loads, so the widest possible grid wins (a variant that kept B[j, m] in registers across eight
// tokens per thread loaded an eighth of the data and ran 1.5 to 2 times slower).
__global__ void __launch_bounds__(256) fused_finalize_kernel(const float* __restrict__ part, int splits, int N, int M,
                                                             const float* __restrict__ bias,
                                                             const float* __restrict__ H, const float* __restrict__ B,
                                                             int r, float s, __nv_bfloat16* __restrict__ Y) {
    pdl_launch_dependents();
    pdl_wait();
    const int m = blockIdx.x * blockDim.x + threadIdx.x;
    const int n = blockIdx.y;
    if (m >= M) return;
    float v = 0.f;
    for (int z = 0; z < splits; ++z) v += part[((size_t)z * N + n) * M + m];
    if (bias) v += bias[m];
    if (r > 0) {
        float d = 0.f;
        for (int j = 0; j < r; ++j) d = fmaf(H[(size_t)n * r + j], B[(size_t)j * M + m], d);
        v += s * d;
    }
    Y[(size_t)n * M + m] = __float2bfloat16(v);
}

// The same for a group of sites in one launch: blockIdx.x runs over the concatenated 256-column
// blocks of the sites' outputs.
struct FinalizeSite {
    const float* part;
    const float* bias;
    const float* H;
    const float* B;
    __nv_bfloat16* Y;
    int splits, M, r;
    float s;
};
struct FinalizeGroup {
    int n_sites, N;
    int block_end[kMaxGroup];
    FinalizeSite site[kMaxGroup];
};
__global__ void __launch_bounds__(256) fused_finalize_group_kernel(const __grid_constant__ FinalizeGroup g) {
    pdl_launch_dependents();
    pdl_wait();
    const int bx = (int)blockIdx.x;
    const int si = (bx >= g.block_end[0]) + (bx >= g.block_end[1]) + (bx >= g.block_end[2]);
    FinalizeSite f;  // literal indices keep the fields instruction operands
    int b0;
    switch (si) {
        case 0: f = g.site[0]; b0 = 0; break;
        case 1: f = g.site[1]; b0 = g.block_end[0]; break;
        case 2: f = g.site[2]; b0 = g.block_end[1]; break;
        default: f = g.site[3]; b0 = g.block_end[2]; break;
    }
    const int m = (bx - b0) * blockDim.x + threadIdx.x;
    const int n = blockIdx.y;
    if (m >= f.M) return;
    float v = 0.f;
    for (int z = 0; z < f.splits; ++z) v += f.part[((size_t)z * g.N + n) * f.M + m];
    if (f.bias) v += f.bias[m];
    if (f.r > 0) {
        float d = 0.f;
        for (int j = 0; j < f.r; ++j) d = fmaf(f.H[(size_t)n * f.r + j], f.B[(size_t)j * f.M + m], d);
        v += f.s * d;
    }
    f.Y[(size_t)n * f.M + m] = __float2bfloat16(v);
}

// H[n, j] = sum_k X[n, k] * A[k, j], one token per block, f32 accumulation (X bf16, A and H f32).
// Thread t owns k = t, t + 256, ... and keeps RP partial sums in registers (rows of A are read as
// float4, consecutive threads read consecutive rows); the 256 partial vectors are then combined by
// a fixed shuffle tree and a fixed-order pass over the 8 warps, so the result is deterministic.
template <int RP>
__global__ void __launch_bounds__(256) small_h_kernel(const __nv_bfloat16* __restrict__ X, const float* __restrict__ A,
                                                      int K, int r, float* __restrict__ H) {
    __shared__ float red[8][RP];
    const int n = blockIdx.x, t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const __nv_bfloat16* x = X + (size_t)n * K;
    float acc[RP];
#pragma unroll
    for (int j = 0; j < RP; ++j) acc[j] = 0.f;
    const bool vec = (r == RP);  // rows of A are RP floats: 16-byte aligned float4 loads
#pragma unroll 4
    for (int k = t; k < K; k += 256) {
        const float xv = __bfloat162float(x[k]);
        const float* arow = A + (size_t)k * r;
        if (vec) {
#pragma unroll
            for (int j = 0; j < RP; j += 4) {
                const float4 a4 = *(const float4*)(arow + j);
                acc[j] = fmaf(xv, a4.x, acc[j]);
                acc[j + 1] = fmaf(xv, a4.y, acc[j + 1]);
                acc[j + 2] = fmaf(xv, a4.z, acc[j + 2]);
                acc[j + 3] = fmaf(xv, a4.w, acc[j + 3]);
            }
        } else {
#pragma unroll
            for (int j = 0; j < RP; ++j)
                if (j < r) acc[j] = fmaf(xv, arow[j], acc[j]);
        }
    }
#pragma unroll
    for (int j = 0; j < RP; ++j) {
        float v = acc[j];
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
        if (lane == 0) red[warp][j] = v;
    }
    __syncthreads();
    if (t < r) {
        float h = 0.f;
#pragma unroll
        for (int w8 = 0; w8 < 8; ++w8) h += red[w8][t];
        H[(size_t)n * r + t] = h;
    }
}

int pick_splits(int m_tiles, int k_tiles, int sms) {
    int best = 1;
    long long best_cost = -1;
    for (int s = 1; s <= 16 && s <= k_tiles; ++s) {
        long long waves = ((long long)m_tiles * s + sms - 1) / sms;
        long long cost = waves * ((k_tiles + s - 1) / s) * 16 + s;  // tie-break: fewer splits (less partial traffic)
        if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = s; }
    }
    return best;
}

inline size_t al256(size_t x) { return (x + 255) & ~size_t(255); }

// X [N, K] bf16 viewed as [k-tile][token][64]: dim0 = 64 k of one tile (contiguous), dim1 = tokens
// (stride K), dim2 = k-tiles (stride 64 elements).  A box {64, NT, KS} then lands KS k-tiles as KS
// separate 128-byte-swizzled [NT][64] tiles.  Needs K % 64 == 0.
CUtensorMap make_x_map3d(const void* X, int64_t N, int64_t K, int nt, int ks = KS) {
    typedef CUresult (*Fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                           const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                           CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static Fn fn = nullptr;
    if (!fn) {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            throw LqError(LQ_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
        fn = (Fn)f;
    }
    if (((uintptr_t)X & 15) != 0) throw LqError(LQ_ERR_INVALID, "X must be 16-byte aligned");
    CUtensorMap m;
    cuuint64_t dims[3] = {64, (cuuint64_t)N, (cuuint64_t)(K / 64)};
    cuuint64_t strides[2] = {(cuuint64_t)K * 2, 128};
    cuuint32_t box[3] = {64, (cuuint32_t)nt, (cuuint32_t)ks};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult rc = fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(X), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS)
        throw LqError(LQ_ERR_CUDA, "cuTensorMapEncodeTiled (3-D X view) failed with CUresult " + std::to_string((int)rc));
    return m;
}

template <int NT>
void launch_fused(const CUtensorMap& tmX, const FusedParams& p, int grid, cudaStream_t st) {
    auto kern = fused_small_fwd_kernel<NT>;
    LQ_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FCfg<NT>::SMEM));
    LqProf prof(LQ_K_GEMM_MAIN, st);
    kern<<<grid, kFusedThreads, FCfg<NT>::SMEM, st>>>(tmX, p);
    LQ_CUDA(cudaGetLastError());
}

template <int NB, typename G>
void launch_stream(const CUtensorMap& tmX, const G& gp, int grid, cudaStream_t st) {  // G: FusedParams or StreamGroup
    auto kern = stream_small_fwd_kernel<NB, G>;
    LQ_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)STREAM_SMEM));
    LqProf prof(LQ_K_GEMM_MAIN, st);
    launch_pdl(kern, dim3(grid), dim3(kStreamThreads), STREAM_SMEM, st, tmX, gp);
    LQ_CUDA(cudaGetLastError());
}

template <int NB>
void launch_stream_f8(const CUtensorMap& tmX, const CUtensorMap& tmW, const StreamF8Params& q, int grid, cudaStream_t st) {
    auto kern = stream_small_fp8_kernel<NB>;
    LQ_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)F8_SMEM));
    LqProf prof(LQ_K_GEMM_MAIN, st);
    launch_pdl(kern, dim3(grid), dim3(kStreamThreads), F8_SMEM, st, tmX, tmW, q);
    LQ_CUDA(cudaGetLastError());
}

}  // namespace

bool lq_fused_supported(const lq_weight* w, int64_t n_tokens, int rank) {
    if (rank > 64 || n_tokens < 1 || w->K % 64 != 0 || w->M % 8 != 0) return false;
    if (w->scheme == LQ_INT4) return n_tokens <= 64;
    if (w->scheme == LQ_FP8_E4M3) return n_tokens <= STREAM_NT && ((uintptr_t)w->packed & 15) == 0;
    return false;
}

size_t lq_fused_workspace_bytes(const lq_weight* w, int64_t n_tokens, int rank) {
    size_t h = al256((size_t)n_tokens * (size_t)(rank > 0 ? rank : 1) * 4);
    size_t tok = (size_t)std::max<int64_t>(n_tokens, STREAM_NT);
    size_t m_tiles = (size_t)((w->M + 127) / 128);
    size_t part = al256((size_t)16 * tok * m_tiles * 128 * 4);
    size_t counters = al256(m_tiles * 4);
    return h + part + counters + 256;
}

void lq_fused_fwd(const lq_weight* w, const void* X, int64_t N, const float* A, const float* B, int r, float s,
                  void* Y, float* H_out, void* ws, size_t ws_bytes, cudaStream_t st) {
    LQ_CHECK_ARG(ws != nullptr && ((uintptr_t)ws & 255) == 0, "workspace must be non-NULL and 256-byte aligned");
    if (lq_fused_workspace_bytes(w, N, r) > ws_bytes + 256)
        throw LqError(LQ_ERR_WORKSPACE, "workspace too small for the fused small-batch path");
    const int64_t M = w->M, K = w->K;
    float* Hf = (float*)ws;
    float* part = (float*)((char*)ws + al256((size_t)N * (size_t)(r > 0 ? r : 1) * 4));
    if (r > 0 && H_out) Hf = H_out;
    const bool stream = N <= STREAM_NT;
    bool forked = false;
    if (r > 0 && !stream) {  // H = X . A in f32: one block per token, on the side stream beside the weight kernel
        cudaStream_t hs = lq_tc_fork(w->device, st);
        forked = true;
        LqProf prof(LQ_K_GEMM_DOWN, hs);
        const __nv_bfloat16* Xb = (const __nv_bfloat16*)X;
        if (r <= 16) small_h_kernel<16><<<(unsigned)N, 256, 0, hs>>>(Xb, A, (int)K, r, Hf);
        else if (r <= 32) small_h_kernel<32><<<(unsigned)N, 256, 0, hs>>>(Xb, A, (int)K, r, Hf);
        else small_h_kernel<64><<<(unsigned)N, 256, 0, hs>>>(Xb, A, (int)K, r, Hf);
        LQ_CUDA(cudaGetLastError());
    }
    const int sms = lq_tc_sm_count(w->device);
    FusedParams p;
    p.packed = (const uint8_t*)w->packed;
    p.scales = w->scales;
    p.M = (int)M;
    p.N = (int)N;
    p.k_tiles = (int)w->k_tiles;
    p.n_groups = (int)w->n_groups;
    p.group = w->group;
    p.m_tiles = (int)w->m_tiles;
    p.part = part;
    p.status = lq_tc_status_word(w->device);
    p.h_blocks = (stream && r > 0) ? (int)N : 0;
    p.r = r;
    p.K = (int)K;
    p.X = (const __nv_bfloat16*)X;
    p.A = A;
    p.H = Hf;
    if (stream && w->scheme == LQ_FP8_E4M3) {
        const int slots = sms * STREAM_CTAS_PER_SM - p.h_blocks;
        p.k_tiles = (int)((K + 63) / 64);
        p.m_tiles = (int)((M + 127) / 128);
        p.splits = pick_splits(p.m_tiles, (p.k_tiles + 1) / 2, slots);
        const int grid = std::min(p.m_tiles * p.splits, slots) + p.h_blocks;
        StreamF8Params q;
        q.base = p;
        q.wscale = w->scales;
        q.per_channel = w->scale_kind == LQ_SCALE_PER_CHANNEL;
        CUtensorMap tmX = make_x_map3d(X, N, K, STREAM_NT, KS_F8);
        CUtensorMap tmW = lq_tc_make_map_u8(w->packed, K, M, K, 128);
        if (N <= 8) launch_stream_f8<1>(tmX, tmW, q, grid, st);
        else launch_stream_f8<2>(tmX, tmW, q, grid, st);
    } else if (stream) {  // register-dequant stream kernel, several small CTAs per SM
        const int slots = sms * STREAM_CTAS_PER_SM - p.h_blocks;
        p.splits = pick_splits(p.m_tiles, p.k_tiles, slots);
        const int grid = std::min(p.m_tiles * p.splits, slots) + p.h_blocks;
        CUtensorMap tmX = make_x_map3d(X, N, K, STREAM_NT);
        if (N <= 8) launch_stream<1>(tmX, p, grid, st);
        else launch_stream<2>(tmX, p, grid, st);
    } else {
        p.splits = pick_splits(p.m_tiles, p.k_tiles, sms);
        const int grid = std::min(p.m_tiles * p.splits, sms);
        const int nt = N <= 32 ? 32 : 64;
        CUtensorMap tmX = make_x_map3d(X, N, K, nt);
        if (nt == 32) launch_fused<32>(tmX, p, grid, st);
        else launch_fused<64>(tmX, p, grid, st);
    }
    if (forked) lq_tc_join(w->device, st);
    {
        LqProf prof(LQ_K_REDUCE, st);
        dim3 g((unsigned)((M + 255) / 256), (unsigned)N);
        if (stream)
            launch_pdl(fused_finalize_kernel, g, dim3(256), 0, st, (const float*)part, p.splits, (int)N, (int)M,
                       (const float*)w->bias, (const float*)Hf, B, r, s, (__nv_bfloat16*)Y);
        else
            fused_finalize_kernel<<<g, 256, 0, st>>>(part, p.splits, (int)N, (int)M, w->bias, Hf, B, r, s, (__nv_bfloat16*)Y);
        LQ_CUDA(cudaGetLastError());
    }
}

// ---- a group of sites that share X, as one launch pair ------------------------------------------
bool lq_fused_group_supported(const lq_group_site* sites, int n_sites, int64_t n_tokens) {
    if (n_sites < 1 || n_sites > kMaxGroup || n_tokens < 1 || n_tokens > STREAM_NT) return false;
    const lq_weight* w0 = sites[0].w;
    for (int i = 0; i < n_sites; ++i) {
        const lq_weight* w = sites[i].w;
        if (!w || w->scheme != LQ_INT4 || w->K != w0->K || w->group != w0->group || w->device != w0->device) return false;
        if (!lq_fused_supported(w, n_tokens, sites[i].rank)) return false;
    }
    return true;
}

size_t lq_fused_group_workspace_bytes(const lq_group_site* sites, int n_sites, int64_t n_tokens) {
    size_t total = 256;
    for (int i = 0; i < n_sites; ++i) total += lq_fused_workspace_bytes(sites[i].w, n_tokens, sites[i].rank);
    return total;
}

void lq_fused_fwd_grouped(const lq_group_site* sites, int n_sites, const void* X, int64_t N, void* ws, size_t ws_bytes,
                          cudaStream_t st) {
    LQ_CHECK_ARG(ws != nullptr && ((uintptr_t)ws & 255) == 0, "workspace must be non-NULL and 256-byte aligned");
    if (lq_fused_group_workspace_bytes(sites, n_sites, N) > ws_bytes + 256)
        throw LqError(LQ_ERR_WORKSPACE, "workspace too small for the grouped small-batch path");
    const lq_weight* w0 = sites[0].w;
    const int sms = lq_tc_sm_count(w0->device);
    StreamGroup gp{};
    FinalizeGroup fg{};
    gp.n_sites = fg.n_sites = n_sites;
    fg.N = (int)N;
    int h_total = 0, m_tiles_total = 0;
    for (int i = 0; i < n_sites; ++i) {
        if (sites[i].rank > 0) h_total += (int)N;
        m_tiles_total += (int)sites[i].w->m_tiles;
    }
    const int slots = sms * STREAM_CTAS_PER_SM - h_total;
    const int splits = pick_splits(m_tiles_total, (int)w0->k_tiles, slots);  // one split count: the sites share d_in
    char* cur = (char*)ws;
    int items = 0, hb = 0, blocks = 0;
    for (int i = 0; i < n_sites; ++i) {
        const lq_weight* w = sites[i].w;
        const int r = sites[i].rank;
        LQ_CHECK_ARG(r == 0 || (sites[i].A && sites[i].B), "rank > 0 needs LoRA factors A and B");
        LQ_CHECK_ARG(sites[i].Y != nullptr, "Y pointer is NULL");
        float* Hf = (float*)cur;
        float* part = (float*)(cur + al256((size_t)N * (size_t)(r > 0 ? r : 1) * 4));
        cur += lq_fused_workspace_bytes(w, N, r);
        if (r > 0 && sites[i].H_out) Hf = sites[i].H_out;
        FusedParams& q = gp.site[i];
        q.packed = (const uint8_t*)w->packed;
        q.scales = w->scales;
        q.M = (int)w->M;
        q.N = (int)N;
        q.k_tiles = (int)w->k_tiles;
        q.n_groups = (int)w->n_groups;
        q.group = w->group;
        q.m_tiles = (int)w->m_tiles;
        q.splits = splits;
        q.part = part;
        q.status = lq_tc_status_word(w->device);
        q.h_blocks = r > 0 ? (int)N : 0;
        q.r = r;
        q.K = (int)w->K;
        q.X = (const __nv_bfloat16*)X;
        q.A = sites[i].A;
        q.H = Hf;
        items += q.m_tiles * splits;
        hb += q.h_blocks;
        gp.item_end[i] = items;
        gp.h_end[i] = hb;
        FinalizeSite& f = fg.site[i];
        f.part = part;
        f.bias = w->bias;
        f.H = Hf;
        f.B = sites[i].B;
        f.Y = (__nv_bfloat16*)sites[i].Y;
        f.splits = splits;
        f.M = (int)w->M;
        f.r = r;
        f.s = sites[i].scaling;
        blocks += (int)((w->M + 255) / 256);
        fg.block_end[i] = blocks;
    }
    gp.n_items = items;
    gp.n_hblocks = hb;
    for (int i = n_sites; i < kMaxGroup; ++i) gp.item_end[i] = gp.h_end[i] = 0x7fffffff;
    for (int i = n_sites; i < kMaxGroup; ++i) fg.block_end[i] = 0x7fffffff;
    const int grid = std::min(items, slots) + hb;
    CUtensorMap tmX = make_x_map3d(X, N, w0->K, STREAM_NT);
    if (N <= 8) launch_stream<1>(tmX, gp, grid, st);
    else launch_stream<2>(tmX, gp, grid, st);
    {
        LqProf prof(LQ_K_REDUCE, st);
        launch_pdl(fused_finalize_group_kernel, dim3((unsigned)blocks, (unsigned)N), dim3(256), 0, st, fg);
        LQ_CUDA(cudaGetLastError());
    }
}
