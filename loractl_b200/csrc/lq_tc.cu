// tcgen05 GEMM kernel + the host orchestration of the bf16 LoRA-linear path.
//
// One persistent, warp-specialised kernel serves every contraction on the path:
//
//   C[Mg, Ng] = A[Mg, Kg] . B[Ng, Kg]^T          (bf16 operands, f32 accumulation in TMEM)
//
//   warp 0 : TMA producer   (cp.async.bulk.tensor 2-D tiles, 128-byte swizzle, no multicast)
//   warp 1 : MMA issuer     (tcgen05.mma cta_group::1, 128 x BLOCK_N x 16 per instruction;
//                            kind::f16 on bf16 operands, kind::f8f6f4 on e4m3 operands)
//   warps 2-9 : epilogue    (tcgen05.ld from TMEM -> registers; two warps per TMEM lane quarter,
//                            each draining half of the columns; scales and bias applied here;
//                            bf16 output is staged in shared memory, 64-byte swizzled, and leaves
//                            through TMA tensor stores, f32 partial tiles through plain stores)
//
// The K loop may continue into a second pair of tensor maps ("K extension").  That is how
// the rank-r LoRA product is fused into the frozen GEMM: with A1 = s*H (N x r, zero padded to
// 64) and B1 = B^T (M x r), the extra k-block adds s * H . B to the same TMEM accumulator
// before the single epilogue; X is therefore read once by the frozen GEMM.
//
// Work items are (output tile, k-split); with splits > 1 the kernel writes f32 partial tiles
// that a fixed-order second stage reduces (deterministic: no atomics anywhere).
#include <atomic>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <vector>

#include <cuda_fp8.h>

#include "lq_gemm.cuh"
#include "lq_prof.cuh"
#include "lq_tc.cuh"
#include "lq_umma.cuh"

namespace {

using namespace umma;

using namespace lqgemm;

constexpr int kThreads = 320;  // TMA warp, MMA warp, 8 epilogue warps (two per TMEM lane quarter)

template <typename OutT>
__device__ __forceinline__ void store8(OutT* dst, const float* v);
template <>
__device__ __forceinline__ void store8<float>(float* dst, const float* v) {
    *(float4*)dst = make_float4(v[0], v[1], v[2], v[3]);
    *(float4*)(dst + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
template <>
__device__ __forceinline__ void store8<__nv_bfloat16>(__nv_bfloat16* dst, const float* v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
    __nv_bfloat162 c = __floats2bfloat162_rn(v[4], v[5]), d = __floats2bfloat162_rn(v[6], v[7]);
    uint4 u;
    u.x = *(uint32_t*)&a; u.y = *(uint32_t*)&b; u.z = *(uint32_t*)&c; u.w = *(uint32_t*)&d;
    *(uint4*)dst = u;
}

// F8: the operands of the first tensor-map pair are e4m3 bytes (128 per k-block row) multiplied
// with tcgen05.mma kind::f8f6f4; the K-extension pair stays bf16 (kind::f16) and accumulates into
// the same f32 TMEM tile.  Both pairs must be K-major in that mode.
template <int BLOCK_N, bool A_MN, bool B_MN, typename OutT, bool F8 = false>
__global__ void __launch_bounds__(kThreads, 1)
umma_gemm_kernel(const __grid_constant__ CUtensorMap tmA0, const __grid_constant__ CUtensorMap tmB0,
                 const __grid_constant__ CUtensorMap tmA1, const __grid_constant__ CUtensorMap tmB1,
                 const __grid_constant__ CUtensorMap tmC, GemmParams p) {
    using C = Cfg<BLOCK_N>;
    constexpr int STAGES = C::STAGES;
    static_assert(!(F8 && (A_MN || B_MN)), "fp8 operands are K-major only");
    constexpr int BK0 = F8 ? 128 : BK;  // elements per k-block of the first pair (128 bytes per row)
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* smem_a = smem;
    uint8_t* smem_b = smem + (size_t)STAGES * C::A_BYTES;
    uint8_t* stage_out = smem + (size_t)STAGES * (C::A_BYTES + C::B_BYTES);  // 1024-aligned
    uint64_t* bars = (uint64_t*)(stage_out + C::STAGE_OUT);
    uint64_t* full = bars;
    uint64_t* empty = bars + STAGES;
    uint64_t* tfull = bars + 2 * STAGES;
    uint64_t* tempty = bars + 2 * STAGES + 2;
    uint32_t* tmem_slot = (uint32_t*)(bars + 2 * STAGES + 4);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&full[s]), 1);
            mbar_init(smem_u32(&empty[s]), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(smem_u32(&tfull[a]), 1);
            mbar_init(smem_u32(&tempty[a]), 256);
        }
        *abort_flag = 0;
        fence_barrier_init();
        prefetch_tmap(&tmA0);
        prefetch_tmap(&tmB0);
        prefetch_tmap(&tmA1);
        prefetch_tmap(&tmB1);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), C::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int kb_total = p.kb0 + p.kb1;
    const int num_items = p.m_tiles * p.n_tiles * p.splits;

    if (warp == 0) {
        if (lane == 0) {
            // ---------------- TMA producer ----------------
            int s = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int item = blockIdx.x; ok && item < num_items; item += gridDim.x) {
                int m_tile, n_tile, z;
                item_coords(p, item, m_tile, n_tile, z);
                const int kb_begin = (int)(((long long)z * kb_total) / p.splits);
                const int kb_end = (int)(((long long)(z + 1) * kb_total) / p.splits);
                for (int kb = kb_begin; kb < kb_end; ++kb) {
                    if (!mbar_wait(smem_u32(&empty[s]), phase ^ 1u, abort_flag, p.status, 11)) { ok = false; break; }
                    const uint32_t bar = smem_u32(&full[s]);
                    mbar_expect_tx(bar, C::A_BYTES + C::B_BYTES);
                    const bool ext = kb >= p.kb0;
                    const CUtensorMap* ma = ext ? &tmA1 : &tmA0;
                    const CUtensorMap* mb = ext ? &tmB1 : &tmB0;
                    const int kc = ext ? (kb - p.kb0) * BK : kb * BK0;
                    const uint32_t sa = smem_u32(smem_a + (size_t)s * C::A_BYTES);
                    const uint32_t sb = smem_u32(smem_b + (size_t)s * C::B_BYTES);
                    if (!A_MN) {
                        tma_load_2d(sa, ma, bar, kc, m_tile * BM);
                    } else {
#pragma unroll
                        for (int i = 0; i < BM / 64; ++i) tma_load_2d(sa + i * 8192, ma, bar, m_tile * BM + i * 64, kc);
                    }
                    if (!B_MN) {
                        tma_load_2d(sb, mb, bar, kc, n_tile * BLOCK_N);
                    } else {
#pragma unroll
                        for (int i = 0; i < BLOCK_N / 64; ++i)
                            tma_load_2d(sb + i * 8192, mb, bar, n_tile * BLOCK_N + i * 64, kc);
                    }
                    if (++s == STAGES) { s = 0; phase ^= 1u; }
                }
            }
            if (!ok) {
                // Give copies already in flight time to land before the CTA's shared memory is released.
                for (int i = 0; i < 64; ++i) __nanosleep(1000);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---------------- MMA issuer ----------------
            constexpr uint32_t idesc = make_idesc(1, 1, A_MN, B_MN, BM, BLOCK_N);
            constexpr uint32_t idesc8 = make_idesc(0, 0, false, false, BM, BLOCK_N);  // e4m3 x e4m3
            const uint32_t d_hi = desc_hi(1024);
            const uint32_t a_lo0 = desc_lo(smem_u32(smem_a), A_MN ? 8192 : 16);
            const uint32_t b_lo0 = desc_lo(smem_u32(smem_b), B_MN ? 8192 : 16);
            int s = 0, acc = 0;
            uint32_t phase = 0, acc_phase = 0;
            bool ok = true;
            for (int item = blockIdx.x; ok && item < num_items; item += gridDim.x) {
                int m_tile, n_tile, z;
                item_coords(p, item, m_tile, n_tile, z);
                const int kb_begin = (int)(((long long)z * kb_total) / p.splits);
                const int kb_end = (int)(((long long)(z + 1) * kb_total) / p.splits);
                if (!mbar_wait(smem_u32(&tempty[acc]), acc_phase ^ 1u, abort_flag, p.status, 12)) { ok = false; break; }
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + (uint32_t)(acc * BLOCK_N);
                for (int kb = kb_begin; kb < kb_end; ++kb) {
                    if (!mbar_wait(smem_u32(&full[s]), phase, abort_flag, p.status, 13)) { ok = false; break; }
                    tc_fence_after();
                    // descriptors: constant high word, low word = stage base + 16-element k-step
                    // (K-major: 32 bytes along the row; MN-major: 16 k-rows of 128 bytes), in 16-byte units
                    const uint32_t a_lo = a_lo0 + (uint32_t)s * (C::A_BYTES >> 4);
                    const uint32_t b_lo = b_lo0 + (uint32_t)s * (C::B_BYTES >> 4);
                    if (F8 && kb < p.kb0) {
#pragma unroll
                        for (int k = 0; k < 4; ++k)  // 32 e4m3 per instruction = 32 bytes along the row
                            mma_f8(tmem_d, desc_join(a_lo + k * 2u, d_hi), desc_join(b_lo + k * 2u, d_hi), idesc8,
                                   (kb > kb_begin || k > 0) ? 1u : 0u);
                    } else {
#pragma unroll
                        for (int k = 0; k < BK / 16; ++k)
                            mma_f16(tmem_d, desc_join(a_lo + k * (A_MN ? 128u : 2u), d_hi),
                                    desc_join(b_lo + k * (B_MN ? 128u : 2u), d_hi), idesc,
                                    (kb > kb_begin || k > 0) ? 1u : 0u);
                    }
                    mma_commit(smem_u32(&empty[s]));  // frees the smem stage once these MMAs retire
                    if (++s == STAGES) { s = 0; phase ^= 1u; }
                }
                if (!ok) break;
                mma_commit(smem_u32(&tfull[acc]));  // accumulator complete -> epilogue
                if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
            }
        }
    } else {
        // ---------------- epilogue (warps 2..5) ----------------
        const int quarter = warp & 3;       // TMEM lane quarter this warp may access
        const int chalf = (warp - 2) >> 2;  // which half of the tile's columns this warp drains
        int acc = 0;
        uint32_t acc_phase = 0;
        bool ok = true;
        OutT* Cbase = (OutT*)p.C;
        for (int item = blockIdx.x; ok && item < num_items; item += gridDim.x) {
            int m_tile, n_tile, z;
            item_coords(p, item, m_tile, n_tile, z);
            if (!mbar_wait(smem_u32(&tfull[acc]), acc_phase, abort_flag, p.status, 14)) { ok = false; break; }
            tc_fence_after();
            const int row = m_tile * BM + quarter * 32 + lane;
            OutT* crow = Cbase + (long long)z * p.split_stride + (long long)row * p.ldc;
            const float rs = (p.row_scale && row < p.Mg) ? p.row_scale[row] : 1.f;
#pragma unroll 1
            for (int c = 0; c < BLOCK_N / 64; ++c) {
                uint32_t r[32];
                const int cc = chalf * (BLOCK_N / 2) + c * 32;  // column of the tile this load starts at
                tmem_ld_x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * BLOCK_N + cc), r);
                tmem_ld_wait();
                const int col0 = n_tile * BLOCK_N + cc;
                if (sizeof(OutT) == 2 && p.tma_store) {
                    // scale / bias, round to bf16, stage the warp's 32 x 32 piece in shared memory in
                    // the 64-byte-swizzled layout and hand it to a TMA tensor store: every row piece
                    // leaves as one full 64-byte write instead of four 16-byte partial-sector writes
                    // scattered over 32 rows (which measured 1.9 TB/s for an output-bound GEMM).
                    uint32_t wds[16];
#pragma unroll
                    for (int j = 0; j < 32; j += 8) {
                        const int col = col0 + j;
                        float v[8];
#pragma unroll
                        for (int e = 0; e < 8; ++e) v[e] = __uint_as_float(r[j + e]);
                        if (col < p.Ng) {
                            if (p.col_scale && !p.col_scale_bcast) {
                                const float4 c0 = *(const float4*)(p.col_scale + col);
                                const float4 c1 = *(const float4*)(p.col_scale + col + 4);
                                const float cs[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
#pragma unroll
                                for (int e = 0; e < 8; ++e) v[e] *= rs * cs[e];
                            } else if (p.row_scale || p.col_scale) {
                                const float sc = p.col_scale ? rs * p.col_scale[0] : rs;
#pragma unroll
                                for (int e = 0; e < 8; ++e) v[e] *= sc;
                            }
                            if (p.bias) {
                                const float4 b0 = *(const float4*)(p.bias + col);
                                const float4 b1 = *(const float4*)(p.bias + col + 4);
                                const float bs[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
                                for (int e = 0; e < 8; ++e) v[e] += bs[e];
                            }
                        }
#pragma unroll
                        for (int e = 0; e < 8; e += 2) {
                            __nv_bfloat162 h2 = __floats2bfloat162_rn(v[e], v[e + 1]);
                            wds[(j + e) >> 1] = *(uint32_t*)&h2;
                        }
                    }
                    uint8_t* my_stage = stage_out + (warp - 2) * 2048;
                    if (lane == 0) bulk_wait_read0();  // the previous store has finished reading this buffer
                    __syncwarp();
#pragma unroll
                    for (int q = 0; q < 4; ++q)  // 16-byte chunk q of this lane's row, 64-byte swizzle
                        *(uint4*)(my_stage + lane * 64 + ((q ^ ((lane >> 1) & 3)) << 4)) =
                            make_uint4(wds[4 * q], wds[4 * q + 1], wds[4 * q + 2], wds[4 * q + 3]);
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        tma_store_2d(&tmC, smem_u32(my_stage), col0, m_tile * BM + quarter * 32);
                        bulk_commit();
                    }
                    continue;
                }
                if (row < p.Mg) {
#pragma unroll
                    for (int j = 0; j < 32; j += 8) {
                        const int col = col0 + j;
                        if (col < p.Ng) {  // Ng % 8 == 0: an 8-column group is entirely in or out
                            float v[8];
#pragma unroll
                            for (int e = 0; e < 8; ++e) v[e] = __uint_as_float(r[j + e]);
                            if (p.col_scale && !p.col_scale_bcast) {  // col % 8 == 0: two aligned float4 loads
                                const float4 c0 = *(const float4*)(p.col_scale + col);
                                const float4 c1 = *(const float4*)(p.col_scale + col + 4);
                                const float cs[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
#pragma unroll
                                for (int e = 0; e < 8; ++e) v[e] *= rs * cs[e];
                            } else if (p.row_scale || p.col_scale) {
                                const float sc = p.col_scale ? rs * p.col_scale[0] : rs;
#pragma unroll
                                for (int e = 0; e < 8; ++e) v[e] *= sc;
                            }
                            if (p.bias) {
                                const float4 b0 = *(const float4*)(p.bias + col);
                                const float4 b1 = *(const float4*)(p.bias + col + 4);
                                const float bs[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
                                for (int e = 0; e < 8; ++e) v[e] += bs[e];
                            }
                            store8<OutT>(crow + col, v);
                        }
                    }
                }
            }
            tc_fence_before();
            mbar_arrive(smem_u32(&tempty[acc]));
            if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
        }
        if (sizeof(OutT) == 2 && p.tma_store && lane == 0) bulk_wait0();  // stores complete before the CTA exits
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, C::TMEM_COLS);
    }
}

// ---- CTA-pair variant of the frozen GEMM -------------------------------------------------
//
// Two CTAs of a cluster (an SM pair) share one 256 x BLOCK_N output tile: each CTA loads its own
// 128 rows of A and HALF of the B tile (BLOCK_N / 2 rows), one thread of the even CTA issues
// tcgen05.mma.cta_group::2 with M = 256, and each CTA's TMEM receives the 128 accumulator rows of
// its own A half.  Per FLOP every SM therefore stages and reads half of the B operand it does in
// the single-CTA kernel (64 B instead of 96 B of shared memory per clock at 256 columns), which is
// what the tensor pipe waits on and what the power budget goes into.
//
// Barrier protocol (every CTA holds the same barrier objects at the same offsets):
//   full[s]    used in the leader only: the leader's producer arms it with the bytes of BOTH CTAs'
//              copies; each CTA's copies signal it (the peer's through the pair-relative address)
//   empty[s]   one arrival per use in BOTH CTAs, from the leader's multicast tcgen05.commit
//   tfull[a]   same, accumulator complete
//   tempty[a]  used in the leader only: 512 arrivals, the epilogue threads of both CTAs
// K-major bf16 (or e4m3) operands, bf16 output through TMA stores, no split: the two frozen GEMMs.
template <int BLOCK_N>
struct Cfg2 {
    static constexpr uint32_t A_BYTES = BM * BK * 2;
    static constexpr uint32_t B_BYTES = (BLOCK_N / 2) * BK * 2;  // this CTA's half of the B tile
    static constexpr int STAGES = (208 * 1024 - 16 * 1024) / (A_BYTES + B_BYTES);
    static constexpr uint32_t TMEM_COLS = BLOCK_N * 2 <= 256 ? 256 : 512;
    static constexpr uint32_t STAGE_OUT = 8 * 2048;
    static constexpr size_t SMEM = (size_t)STAGES * (A_BYTES + B_BYTES) + STAGE_OUT + 1024 + 256;
};

// B_MN: the B operand of the first tensor-map pair is MN-major ([Kg, Ng] in memory, Ng contiguous) —
// the frozen weight's bf16 copy [d_out, d_in] read as the B operand of dX = dY . W, whose reduction
// runs over d_out: each CTA loads its 128 columns as two 64-column boxes of 64 reduction rows.  The
// K-extension pair stays K-major.  bf16 only, BLOCK_N = 256 only.
template <int BLOCK_N, bool F8, bool B_MN = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
umma_gemm2_kernel(const __grid_constant__ CUtensorMap tmA0, const __grid_constant__ CUtensorMap tmB0,
                  const __grid_constant__ CUtensorMap tmA1, const __grid_constant__ CUtensorMap tmB1,
                  const __grid_constant__ CUtensorMap tmC, GemmParams p) {
    using C = Cfg2<BLOCK_N>;
    constexpr int STAGES = C::STAGES;
    constexpr int BK0 = F8 ? 128 : BK;
    static_assert(!B_MN || (!F8 && BLOCK_N == 256), "MN-major B: bf16, 256-column tiles");
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* smem_a = smem;
    uint8_t* smem_b = smem + (size_t)STAGES * C::A_BYTES;
    uint8_t* stage_out = smem + (size_t)STAGES * (C::A_BYTES + C::B_BYTES);
    uint64_t* bars = (uint64_t*)(stage_out + C::STAGE_OUT);
    uint64_t* full = bars;
    uint64_t* empty = bars + STAGES;
    uint64_t* tfull = bars + 2 * STAGES;
    uint64_t* tempty = bars + 2 * STAGES + 2;
    uint32_t* tmem_slot = (uint32_t*)(bars + 2 * STAGES + 4);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();  // 0: leader (issues the MMAs), 1: peer
    const bool leader = rank == 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&full[s]), 1);
            mbar_init(smem_u32(&empty[s]), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(smem_u32(&tfull[a]), 1);
            mbar_init(smem_u32(&tempty[a]), 512);
        }
        *abort_flag = 0;
        fence_barrier_init();
        prefetch_tmap(&tmA0);
        prefetch_tmap(&tmB0);
        prefetch_tmap(&tmA1);
        prefetch_tmap(&tmB1);
    }
    if (warp == 1) {  // the same warp of both CTAs, the same slot offset
        tmem_alloc2(smem_u32(tmem_slot), C::TMEM_COLS);
        tmem_relinquish2();
    }
    tc_fence_before();
    cluster_sync_all();  // barriers of both CTAs are initialised before either signals the other's
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int kb_total = p.kb0 + p.kb1;
    const int num_items = pair_num_items(p);  // m_tiles counts 256-row pair tiles here; the last tiles may be cut along k
    const int cid = (int)(blockIdx.x >> 1), ncl = (int)(gridDim.x >> 1);

    if (warp == 0) {
        if (lane == 0) {
            // ---------------- TMA producer (both CTAs) ----------------
            int s = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int item = cid; ok && item < num_items; item += ncl) {
                int m_tile, n_tile, z, tile, kb_begin, kb_end, slot;
                pair_item(p, item, kb_total, tile, kb_begin, kb_end, slot);
                item_coords(p, tile, m_tile, n_tile, z);
                for (int kb = kb_begin; kb < kb_end; ++kb) {
                    if (!mbar_wait(smem_u32(&empty[s]), phase ^ 1u, abort_flag, p.status, 51)) { ok = false; break; }
                    const uint32_t bar = smem_u32(&full[s]);
                    if (leader) mbar_expect_tx(bar, 2 * (C::A_BYTES + C::B_BYTES));
                    const bool ext = kb >= p.kb0;
                    const CUtensorMap* ma = ext ? &tmA1 : &tmA0;
                    const CUtensorMap* mb = ext ? &tmB1 : &tmB0;
                    const int kc = ext ? (kb - p.kb0) * BK : kb * BK0;
                    tma_load_2d_pair(smem_u32(smem_a + (size_t)s * C::A_BYTES), ma, bar, kc, m_tile * 256 + (int)rank * BM);
                    if (B_MN && !ext) {
#pragma unroll
                        for (int c = 0; c < BLOCK_N / 128; ++c)  // 64-column chunks of this CTA's half, 64 reduction rows each
                            tma_load_2d_pair(smem_u32(smem_b + (size_t)s * C::B_BYTES) + c * 8192, mb, bar,
                                             n_tile * BLOCK_N + (int)rank * (BLOCK_N / 2) + c * 64, kc);
                    } else {
                        tma_load_2d_pair(smem_u32(smem_b + (size_t)s * C::B_BYTES), mb, bar, kc,
                                         n_tile * BLOCK_N + (int)rank * (BLOCK_N / 2));
                    }
                    if (++s == STAGES) { s = 0; phase ^= 1u; }
                }
            }
            if (!ok)
                for (int i = 0; i < 64; ++i) __nanosleep(1000);
        }
    } else if (warp == 1) {
        if (lane == 0 && leader) {
            // ---------------- MMA issuer (leader CTA only) ----------------
            constexpr uint32_t idesc = make_idesc(1, 1, false, false, 256, BLOCK_N);
            constexpr uint32_t idesc_mn = make_idesc(1, 1, false, true, 256, BLOCK_N);
            constexpr uint32_t idesc8 = make_idesc(0, 0, false, false, 256, BLOCK_N);
            const uint32_t d_hi = desc_hi(1024);
            const uint32_t a_lo0 = desc_lo(smem_u32(smem_a), 16);
            const uint32_t b_lo0 = desc_lo(smem_u32(smem_b), 16);
            const uint32_t b_lo0_mn = desc_lo(smem_u32(smem_b), 8192);
            int s = 0, acc = 0;
            uint32_t phase = 0, acc_phase = 0;
            bool ok = true;
            for (int item = cid; ok && item < num_items; item += ncl) {
                if (!mbar_wait(smem_u32(&tempty[acc]), acc_phase ^ 1u, abort_flag, p.status, 52)) { ok = false; break; }
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + (uint32_t)(acc * BLOCK_N);
                int tile, kb_begin, kb_end, slot;
                pair_item(p, item, kb_total, tile, kb_begin, kb_end, slot);
                for (int kb = kb_begin; kb < kb_end; ++kb) {
                    if (!mbar_wait(smem_u32(&full[s]), phase, abort_flag, p.status, 53)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_lo = a_lo0 + (uint32_t)s * (C::A_BYTES >> 4);
                    const uint32_t b_lo = b_lo0 + (uint32_t)s * (C::B_BYTES >> 4);
                    if (F8 && kb < p.kb0) {
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            mma2_f8(tmem_d, desc_join(a_lo + k * 2u, d_hi), desc_join(b_lo + k * 2u, d_hi), idesc8,
                                    (kb > kb_begin || k > 0) ? 1u : 0u);
                    } else if (B_MN && kb < p.kb0) {
                        const uint32_t bm_lo = b_lo0_mn + (uint32_t)s * (C::B_BYTES >> 4);
#pragma unroll
                        for (int k = 0; k < BK / 16; ++k)  // 16 reduction rows of 128 bytes per step
                            mma2_f16(tmem_d, desc_join(a_lo + k * 2u, d_hi), desc_join(bm_lo + k * 128u, d_hi), idesc_mn,
                                     (kb > kb_begin || k > 0) ? 1u : 0u);
                    } else {
#pragma unroll
                        for (int k = 0; k < BK / 16; ++k)
                            mma2_f16(tmem_d, desc_join(a_lo + k * 2u, d_hi), desc_join(b_lo + k * 2u, d_hi), idesc,
                                     (kb > kb_begin || k > 0) ? 1u : 0u);
                    }
                    mma2_commit_mc(smem_u32(&empty[s]), 3);  // frees the stage in both CTAs
                    if (++s == STAGES) { s = 0; phase ^= 1u; }
                }
                if (!ok) break;
                mma2_commit_mc(smem_u32(&tfull[acc]), 3);  // accumulator complete -> both epilogues
                if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
            }
        }
    } else {
        // ---------------- epilogue (warps 2..9 of both CTAs, each its own 128 rows) ----------------
        const int quarter = warp & 3;
        const int chalf = (warp - 2) >> 2;
        int acc = 0;
        uint32_t acc_phase = 0;
        bool ok = true;
        for (int item = cid; ok && item < num_items; item += ncl) {
            int m_tile, n_tile, z, tile, kb_begin, kb_end, slot;
            pair_item(p, item, kb_total, tile, kb_begin, kb_end, slot);
            item_coords(p, tile, m_tile, n_tile, z);
            if (!mbar_wait(smem_u32(&tfull[acc]), acc_phase, abort_flag, p.status, 54)) { ok = false; break; }
            tc_fence_after();
            if (slot >= 0) {
                // a k-range of a cut tile: the raw f32 accumulator goes to its partial slot (scales, bias
                // and the bf16 rounding are applied once, by the launch that sums the slots)
                float* dst = p.tail_part + ((size_t)slot * 256 + (size_t)((int)rank * BM + quarter * 32 + lane)) * BLOCK_N;
#pragma unroll 1
                for (int c = 0; c < BLOCK_N / 64; ++c) {
                    uint32_t r[32];
                    const int cc = chalf * (BLOCK_N / 2) + c * 32;
                    tmem_ld_x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * BLOCK_N + cc), r);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 32; j += 4)
                        *(uint4*)(dst + cc + j) = make_uint4(r[j], r[j + 1], r[j + 2], r[j + 3]);
                }
                tc_fence_before();
                if (leader) mbar_arrive(smem_u32(&tempty[acc]));
                else mbar_arrive_leader(smem_u32(&tempty[acc]));
                if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
                continue;
            }
            const int row0 = m_tile * 256 + (int)rank * BM + quarter * 32;
            const int row = row0 + lane;
            const float rs = (p.row_scale && row < p.Mg) ? p.row_scale[row] : 1.f;
#pragma unroll 1
            for (int c = 0; c < BLOCK_N / 64; ++c) {
                uint32_t r[32];
                const int cc = chalf * (BLOCK_N / 2) + c * 32;
                tmem_ld_x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * BLOCK_N + cc), r);
                tmem_ld_wait();
                const int col0 = n_tile * BLOCK_N + cc;
                uint32_t wds[16];
#pragma unroll
                for (int j = 0; j < 32; j += 8) {
                    const int col = col0 + j;
                    float v[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) v[e] = __uint_as_float(r[j + e]);
                    if (col < p.Ng) {
                        if (p.col_scale && !p.col_scale_bcast) {
                            const float4 c0 = *(const float4*)(p.col_scale + col);
                            const float4 c1 = *(const float4*)(p.col_scale + col + 4);
                            const float cs[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
#pragma unroll
                            for (int e = 0; e < 8; ++e) v[e] *= rs * cs[e];
                        } else if (p.row_scale || p.col_scale) {
                            const float sc = p.col_scale ? rs * p.col_scale[0] : rs;
#pragma unroll
                            for (int e = 0; e < 8; ++e) v[e] *= sc;
                        }
                        if (p.bias) {
                            const float4 b0 = *(const float4*)(p.bias + col);
                            const float4 b1 = *(const float4*)(p.bias + col + 4);
                            const float bs[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
                            for (int e = 0; e < 8; ++e) v[e] += bs[e];
                        }
                    }
#pragma unroll
                    for (int e = 0; e < 8; e += 2) {
                        __nv_bfloat162 h2 = __floats2bfloat162_rn(v[e], v[e + 1]);
                        wds[(j + e) >> 1] = *(uint32_t*)&h2;
                    }
                }
                uint8_t* my_stage = stage_out + (warp - 2) * 2048;
                if (lane == 0) bulk_wait_read0();
                __syncwarp();
#pragma unroll
                for (int q = 0; q < 4; ++q)
                    *(uint4*)(my_stage + lane * 64 + ((q ^ ((lane >> 1) & 3)) << 4)) =
                        make_uint4(wds[4 * q], wds[4 * q + 1], wds[4 * q + 2], wds[4 * q + 3]);
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    tma_store_2d(&tmC, smem_u32(my_stage), col0, row0);
                    bulk_commit();
                }
            }
            tc_fence_before();
            if (leader) mbar_arrive(smem_u32(&tempty[acc]));
            else mbar_arrive_leader(smem_u32(&tempty[acc]));
            if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
        }
        if (lane == 0) bulk_wait0();
    }

    tc_fence_before();
    cluster_sync_all();  // neither CTA leaves (and frees shared memory / TMEM) while the other may still signal it
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc2(tmem_base, C::TMEM_COLS);
    }
}

// Second launch of a pair GEMM whose last tiles were cut along k: sums the partial slots of each cut
// tile in a fixed order, applies what the epilogue would have (scales, bias) and stores bf16.
template <int BLOCK_N>
__global__ void __launch_bounds__(256) pair_tail_reduce_kernel(GemmParams p) {
    constexpr int CG = BLOCK_N / 4;        // 4-column groups per row
    constexpr int RPB = 256 / CG;          // rows per block (BLOCK_N 256: 4, 192: 5 with idle threads)
    const int t = (int)threadIdx.x;
    if (t >= RPB * CG) return;
    const int blocks_per_tile = (256 + RPB - 1) / RPB;
    const int j = (int)blockIdx.x / blocks_per_tile;
    const int r = ((int)blockIdx.x - j * blocks_per_tile) * RPB + t / CG;
    const int c = (t % CG) * 4;
    if (r >= 256) return;
    int m_tile, n_tile, z;
    item_coords(p, p.tail_first + j, m_tile, n_tile, z);
    const int row = m_tile * 256 + r, col = n_tile * BLOCK_N + c;
    if (row >= p.Mg || col >= p.Ng) return;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int q = 0; q < p.tail_splits; ++q) {
        const float4 a = *(const float4*)(p.tail_part + (((size_t)j * p.tail_splits + q) * 256 + r) * BLOCK_N + c);
        v.x += a.x; v.y += a.y; v.z += a.z; v.w += a.w;
    }
    float e[4] = {v.x, v.y, v.z, v.w};
    const float rs = p.row_scale ? p.row_scale[row] : 1.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        if (col + i >= p.Ng) continue;
        if (p.col_scale) e[i] *= rs * p.col_scale[p.col_scale_bcast ? 0 : col + i];
        else if (p.row_scale) e[i] *= rs;
        if (p.bias) e[i] += p.bias[col + i];
    }
    __nv_bfloat16* out = (__nv_bfloat16*)p.C + (size_t)row * p.ldc + col;
    if (col + 3 < p.Ng) {  // Ng % 8 == 0 on this path: a 4-column group is whole or absent, kept general anyway
        __nv_bfloat162 lo = __floats2bfloat162_rn(e[0], e[1]), hi = __floats2bfloat162_rn(e[2], e[3]);
        *(uint2*)out = make_uint2(*(uint32_t*)&lo, *(uint32_t*)&hi);
    } else {
        for (int i = 0; i < 4 && col + i < p.Ng; ++i) out[i] = __float2bfloat16(e[i]);
    }
}

// ---- small elementwise helpers ----------------------------------------------------------

// out[i * ldo + j] = bf16(alpha * in[i * si + j * sj] / div_i) for j < J, 0 for J <= j < Jpad, where
// div_i = row_div[i] (or row_div[0] with row_div_bcast), 1 when row_div is NULL.
__global__ void __launch_bounds__(256) cast_pad_kernel(const float* __restrict__ in, long long si, long long sj,
                                                       __nv_bfloat16* __restrict__ out, long long ldo, long long I,
                                                       int J, int Jpad, float alpha,
                                                       const float* __restrict__ row_div, int row_div_bcast) {
    long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= I * Jpad) return;
    long long i = idx / Jpad;
    int j = (int)(idx - i * Jpad);
    float v = j < J ? alpha * in[i * si + j * sj] : 0.f;
    if (row_div) v = __fdiv_rn(v, row_div[row_div_bcast ? 0 : i]);
    out[i * ldo + j] = __float2bfloat16(v);
}

// Second stage of a split contraction: sums `splits` f32 partial tiles in a fixed order.
//   val = alpha * sum_z part[z][i][j]
//   f32 out (optional): transposed ? out[j * ldo + i] : out[i * ldo + j]   (+= when accumulate)
//   bf16 ext (optional): ext[i * ld_ext + j] = bf16(ext_scale * val), zero for J <= j < Jpad
__global__ void __launch_bounds__(256) reduce_partials_kernel(const float* __restrict__ part, long long split_stride,
                                                              int splits, long long ldp, long long I, int J, int Jpad,
                                                              float alpha, float* __restrict__ out, long long ldo,
                                                              int transposed, int accumulate,
                                                              __nv_bfloat16* __restrict__ ext, long long ld_ext,
                                                              float ext_scale,
                                                              const float* __restrict__ ext_row_div = nullptr) {
    long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= I * Jpad) return;
    long long i = idx / Jpad;
    int j = (int)(idx - i * Jpad);
    float v = 0.f;
    if (j < J) {
        for (int z = 0; z < splits; ++z) v += part[z * split_stride + i * ldp + j];
        v *= alpha;
        if (out) {
            long long o = transposed ? (long long)j * ldo + i : i * ldo + j;
            out[o] = accumulate ? out[o] + v : v;
        }
    }
    if (ext) {
        float e = j < J ? ext_scale * v : 0.f;
        if (ext_row_div) e = __fdiv_rn(e, ext_row_div[i]);  // pre-divide by the row scale the epilogue multiplies back
        ext[i * ld_ext + j] = __float2bfloat16(e);
    }
}

// ---- host side -------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)f;
    });
    if (!fn) throw LqError(LQ_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    return fn;
}

// 2-D bf16 tensor [rows, inner] with `ld` elements between rows; box = 64 x box_rows, 128-byte swizzle.
// `u8`: one-byte elements (e4m3 bytes), box 128 x box_rows; otherwise bf16, box 64 x box_rows — 128 bytes per box
// row either way.
CUtensorMap make_map(const void* base, int64_t inner, int64_t rows, int64_t ld, int box_rows, bool u8 = false) {
    const int esz = u8 ? 1 : 2;
    if (((uintptr_t)base & 15) != 0) throw LqError(LQ_ERR_INVALID, "tensor-core path: pointers must be 16-byte aligned");
    if ((ld * esz) % 16 != 0) throw LqError(LQ_ERR_INVALID, "tensor-core path: row stride must be a multiple of 16 bytes");
    CUtensorMap m;
    cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * esz};
    cuuint32_t box[2] = {u8 ? 128u : 64u, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1u, 1u};
    CUresult r = encode_fn()(&m, u8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                             const_cast<void*>(base), dims, strides, box, estr,
                             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        throw LqError(LQ_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult " + std::to_string((int)r));
    return m;
}

// bf16 output [rows, cols] (ld elements between rows): box 32 x 32, 64-byte swizzle, for TMA stores.
CUtensorMap make_store_map(const void* base, int64_t cols, int64_t rows, int64_t ld) {
    if (((uintptr_t)base & 15) != 0) throw LqError(LQ_ERR_INVALID, "tensor-core path: output must be 16-byte aligned");
    if ((ld * 2) % 16 != 0) throw LqError(LQ_ERR_INVALID, "tensor-core path: output row stride must be a multiple of 16 bytes");
    CUtensorMap m;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {32u, 32u};
    cuuint32_t estr[2] = {1u, 1u};
    CUresult r = encode_fn()(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        throw LqError(LQ_ERR_CUDA, "cuTensorMapEncodeTiled (output) failed with CUresult " + std::to_string((int)r));
    return m;
}

// Fork-join helper objects of one caller stream: the steps of a forward or backward that do not
// depend on each other (weight dequantisation and operand casts on one side, the LoRA down
// projection on the other; dA and dB) are enqueued on a second stream between an event fork and
// an event join, so that their launch latencies overlap instead of adding up.  Both the eager
// path and a stream capture of the call see an ordinary fork-join (the side stream joins the
// capture through the fork event and is joined back before the call returns).
struct Fork {
    cudaStream_t side = nullptr;
    cudaEvent_t ev_fork = nullptr;
    cudaEvent_t ev_join[2] = {nullptr, nullptr};
};

struct DevCtx {
    int sm_count = 0;
    int* status = nullptr;
    std::mutex fork_mu;
    std::map<cudaStream_t, Fork> forks;
};

constexpr int kMaxDevices = 64;

DevCtx& dev_ctx(int dev) {
    static std::mutex mu;
    static DevCtx ctx[kMaxDevices];  // fixed storage: references stay valid
    if (dev < 0 || dev >= kMaxDevices) throw LqError(LQ_ERR_INVALID, "device index out of range");
    std::lock_guard<std::mutex> lk(mu);
    DevCtx& c = ctx[dev];
    if (!c.status) {
        LQ_CUDA(cudaDeviceGetAttribute(&c.sm_count, cudaDevAttrMultiProcessorCount, dev));
        LQ_CUDA(cudaMalloc((void**)&c.status, sizeof(int)));
        LQ_CUDA(cudaMemset(c.status, 0, sizeof(int)));
    }
    return c;
}

bool fork_enabled() {
    static const bool on = [] {
        const char* e = getenv("LQ_SERIAL_LAUNCH");
        return !(e && e[0] == '1');
    }();
    return on;
}

// One Fork per (device, caller stream), created on first use.  Creation happens with the thread's
// capture mode relaxed, so a first call made under a global-mode stream capture still works.
Fork& fork_for(DevCtx& c, cudaStream_t st) {
    std::lock_guard<std::mutex> lk(c.fork_mu);
    auto it = c.forks.find(st);
    if (it != c.forks.end()) return it->second;
    cudaStreamCaptureMode mode = cudaStreamCaptureModeRelaxed;
    LQ_CUDA(cudaThreadExchangeStreamCaptureMode(&mode));
    Fork f;
    cudaError_t e = cudaStreamCreateWithFlags(&f.side, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&f.ev_fork, cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&f.ev_join[0], cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&f.ev_join[1], cudaEventDisableTiming);
    cudaThreadExchangeStreamCaptureMode(&mode);
    if (e != cudaSuccess) throw LqError(LQ_ERR_CUDA, std::string("fork-join objects: ") + cudaGetErrorString(e));
    return c.forks.emplace(st, f).first->second;
}

// `side()` is the second stream after `fork()`, or the caller's stream itself when forking is off.
struct ForkJoin {
    Fork* f = nullptr;
    cudaStream_t main_st;
    ForkJoin(DevCtx& c, cudaStream_t st, bool want) : main_st(st) {
        if (want && fork_enabled()) f = &fork_for(c, st);
    }
    cudaStream_t side() const { return f ? f->side : main_st; }
    void fork() {
        if (!f) return;
        LQ_CUDA(cudaEventRecord(f->ev_fork, main_st));
        LQ_CUDA(cudaStreamWaitEvent(f->side, f->ev_fork, 0));
    }
    // record(i): marks the point the side stream has reached; wait(i): the caller's stream waits for it
    void record(int i) {
        if (f) LQ_CUDA(cudaEventRecord(f->ev_join[i], f->side));
    }
    void wait(int i) {
        if (f) LQ_CUDA(cudaStreamWaitEvent(main_st, f->ev_join[i], 0));
    }
    void join(int i) {
        record(i);
        wait(i);
    }
};

struct Operand {
    const void* ptr;  // bf16
    bool mn_major;    // false: [rows, Kg] (Kg contiguous); true: [Kg, rows] (rows contiguous)
    int64_t ld;       // elements between consecutive rows of the stored matrix
};

struct EpiScales {
    const float* row = nullptr;  // [Mg]
    const float* col = nullptr;  // [Ng], or one value when col_bcast
    int col_bcast = 0;
};

// "reserve_sms" (LQ_RESERVE_SMS): SMs the persistent grids leave free.  A persistent grid sized to the
// whole machine with a static item walk has a cliff when another kernel (an NCCL collective of the
// data-parallel trainer) holds a few SMs for its whole life: the CTAs that do not fit start only when
// resident ones exit, i.e. after their entire walk.  Leaving as many SMs free as the collective takes
// (NCCL_MAX_CTAS) costs reserve / 148 of peak throughput and removes the cliff.
std::atomic<int> g_reserve_sms{[] {
    const char* e = getenv("LQ_RESERVE_SMS");
    return e ? atoi(e) : 0;
}()};
inline int usable_sms(int sm_count) { return std::max(2, sm_count - std::max(0, g_reserve_sms.load())); }

template <int BLOCK_N, bool A_MN, bool B_MN, typename OutT, bool F8 = false>
void launch_gemm(const Operand& a0, const Operand& b0, int64_t K0, const Operand* a1, const Operand* b1, int64_t K1,
                 OutT* Cout, int64_t ldc, int64_t split_stride, int64_t Mg, int64_t Ng, int splits, const float* bias,
                 cudaStream_t st, int64_t b_rows = -1, int prof_kind = LQ_K_GEMM_MAIN, EpiScales sc = EpiScales()) {
    // b_rows: rows the B operand really has when fewer than Ng (TMA zero-fills the rest).
    using C = Cfg<BLOCK_N>;
    if (b_rows < 0) b_rows = Ng;
    int dev;
    LQ_CUDA(cudaGetDevice(&dev));
    DevCtx& ctx = dev_ctx(dev);
    auto mapA = [&](const Operand& o, int64_t Kg) {
        return A_MN ? make_map(o.ptr, Mg, Kg, o.ld, 64) : make_map(o.ptr, Kg, Mg, o.ld, BM);
    };
    auto mapB = [&](const Operand& o, int64_t Kg) {
        return B_MN ? make_map(o.ptr, b_rows, Kg, o.ld, 64) : make_map(o.ptr, Kg, b_rows, o.ld, BLOCK_N);
    };
    CUtensorMap tA0 = F8 ? make_map(a0.ptr, K0, Mg, a0.ld, BM, true) : mapA(a0, K0);
    CUtensorMap tB0 = F8 ? make_map(b0.ptr, K0, b_rows, b0.ld, BLOCK_N, true) : mapB(b0, K0);
    CUtensorMap tA1 = a1 ? mapA(*a1, K1) : tA0, tB1 = b1 ? mapB(*b1, K1) : tB0;
    constexpr int BK0 = F8 ? 128 : BK;
    GemmParams p;
    p.Mg = (int)Mg;
    p.Ng = (int)Ng;
    p.kb0 = (int)((K0 + BK0 - 1) / BK0);
    p.kb1 = a1 ? (int)((K1 + BK - 1) / BK) : 0;
    p.m_tiles = (int)((Mg + BM - 1) / BM);
    p.n_tiles = (int)((Ng + BLOCK_N - 1) / BLOCK_N);
    p.splits = splits;
    p.C = Cout;
    p.ldc = ldc;
    p.split_stride = split_stride;
    p.bias = bias;
    p.status = ctx.status;
    p.row_scale = sc.row;
    p.col_scale = sc.col;
    p.col_scale_bcast = sc.col_bcast;
    // bf16 output (never split): 32 x 32 boxes, 64-byte swizzle, stored by TMA
    p.tma_store = (sizeof(OutT) == 2 && splits == 1) ? 1 : 0;
    p.group_m = 0;
    CUtensorMap tC = tA0;
    if (p.tma_store) tC = make_store_map(Cout, Ng, Mg, ldc);
    long long items = (long long)p.m_tiles * p.n_tiles * splits;
    int grid = (int)std::min<long long>(items, usable_sms(ctx.sm_count));
    auto kern = umma_gemm_kernel<BLOCK_N, A_MN, B_MN, OutT, F8>;
    LQ_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::SMEM));
    LqProf prof(prof_kind, st);
    kern<<<grid, kThreads, C::SMEM, st>>>(tA0, tB0, tA1, tB1, tC, p);
    LQ_CUDA(cudaGetLastError());
}

// "bwd_mn" (LQ_BWD_MN=1): the backward's dX GEMM reads a NON-transposed bf16 scratch as an MN-major
// operand instead of a transposed scratch as a K-major one.  Off by default: the MN-major GEMM
// measured 2-4 % slower and the row-major dequantisation pass no faster than the transposing one.
std::atomic<int> g_bwd_mn{[] {
    const char* e = getenv("LQ_BWD_MN");
    return e ? atoi(e) : 0;
}()};

// "tail_split" (LQ_TAIL_SPLIT=0 to switch off): cut the tiles of a thin last round along k
std::atomic<int> g_tail_split{[] {
    const char* e = getenv("LQ_TAIL_SPLIT");
    return e ? atoi(e) : 1;
}()};
constexpr int kMaxTailSplits = 8;
constexpr int kMinTailKBlocks = 96;
// f32 partial tiles of the cut round: (tiles of the round) x splits <= kTailSlots slots of 256 x 256
constexpr int kTailSlots = 80;
constexpr size_t kTailWsBytes = (size_t)kTailSlots * 256 * 256 * 4;

bool pair_enabled() {
    static const bool on = [] {
        const char* e = getenv("LQ_GEMM_1CTA");
        return !(e && e[0] == '1');
    }();
    return on;
}

// The frozen GEMM on CTA pairs: 256 x BLOCK_N tiles, K-major operands, bf16 output through TMA stores.
template <int BLOCK_N, bool F8, bool B_MN = false>
void launch_gemm_pair(const Operand& a0, const Operand& b0, int64_t K0, const Operand* a1, const Operand* b1, int64_t K1,
                      __nv_bfloat16* Cout, int64_t ldc, int64_t Mg, int64_t Ng, const float* bias, cudaStream_t st,
                      EpiScales sc = EpiScales(), float* tail_ws = nullptr) {
    using C = Cfg2<BLOCK_N>;
    int dev;
    LQ_CUDA(cudaGetDevice(&dev));
    DevCtx& ctx = dev_ctx(dev);
    CUtensorMap tA0 = make_map(a0.ptr, K0, Mg, a0.ld, BM, F8);
    // MN-major B: [K0 rows of the reduction, Ng columns] in memory, boxes of 64 columns x 64 rows
    CUtensorMap tB0 = B_MN ? make_map(b0.ptr, Ng, K0, b0.ld, 64) : make_map(b0.ptr, K0, Ng, b0.ld, BLOCK_N / 2, F8);
    CUtensorMap tA1 = a1 ? make_map(a1->ptr, K1, Mg, a1->ld, BM) : tA0;
    CUtensorMap tB1 = b1 ? make_map(b1->ptr, K1, Ng, b1->ld, BLOCK_N / 2) : tB0;
    constexpr int BK0 = F8 ? 128 : BK;
    GemmParams p;
    p.Mg = (int)Mg;
    p.Ng = (int)Ng;
    p.kb0 = (int)((K0 + BK0 - 1) / BK0);
    p.kb1 = a1 ? (int)((K1 + BK - 1) / BK) : 0;
    p.m_tiles = (int)((Mg + 255) / 256);  // pair tiles
    p.n_tiles = (int)((Ng + BLOCK_N - 1) / BLOCK_N);
    p.splits = 1;
    p.C = Cout;
    p.ldc = ldc;
    p.split_stride = 0;
    p.bias = bias;
    p.status = ctx.status;
    p.row_scale = sc.row;
    p.col_scale = sc.col;
    p.col_scale_bcast = sc.col_bcast;
    p.tma_store = 1;
    CUtensorMap tC = make_store_map(Cout, Ng, Mg, ldc);
    const long long items = (long long)p.m_tiles * p.n_tiles;
    p.group_m = lq_tc_pair_group_m(ctx.sm_count, BLOCK_N, Ng, K0, F8 ? 1 : 2, p.n_tiles);
    auto kern = umma_gemm2_kernel<BLOCK_N, F8, B_MN>;
    LQ_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::SMEM));
    // persistent grid = the number of CTA pairs that can be resident at once (asked once per device)
    static std::mutex mu;
    static int pairs_by_dev[kMaxDevices] = {};
    int pairs;
    {
        std::lock_guard<std::mutex> lk(mu);
        if (pairs_by_dev[dev] == 0) {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(ctx.sm_count & ~1);
            cfg.blockDim = dim3(kThreads);
            cfg.dynamicSmemBytes = C::SMEM;
            int n = 0;
            LQ_CUDA(cudaOccupancyMaxActiveClusters(&n, kern, &cfg));
            pairs_by_dev[dev] = std::max(1, std::min(n, ctx.sm_count / 2));
        }
        pairs = std::min(pairs_by_dev[dev], usable_sms(ctx.sm_count) / 2);
    }
    // A thin last round (at most half the pairs busy) is cut along k so that it fills the machine:
    // config 2's backward is 384 tiles on 74 pairs = 5.19 rounds, which ran as 6.
    // ... and so is a GEMM whose ONLY round is at most half full (a 512-token site with a long
    // reduction: 24 tiles for 74 pairs), all of whose tiles are then cut
    const int rem = items > pairs ? (int)(items % pairs) : (int)items;
    const int kb_total = p.kb0 + p.kb1;
    // Worth it only for long reductions: the cut saves (1 - 1/splits) of a round (0.28 us per k-block)
    // and costs the summing launch plus the overlap the idle pairs used to give the dA contraction
    // (measured: config 2's dX GEMM 0.41 -> 0.36 ms, whole step -1..2 %; a 49-k-block GEMM loses 7 us)
    if (tail_ws && g_tail_split.load() != 0 && rem > 0 && 2 * rem <= pairs && kb_total >= kMinTailKBlocks) {
        const int splits = std::min(std::min(pairs / rem, kTailSlots / rem), std::min(kMaxTailSplits, kb_total / 8));
        if (splits >= 2) {
            p.tail_first = (int)(items - rem);
            p.tail_splits = splits;
            p.tail_part = tail_ws;
        }
    }
    const long long work = p.tail_splits > 1 ? (long long)p.tail_first + (long long)rem * p.tail_splits : items;
    const int grid = 2 * (int)std::min<long long>(work, pairs);
    {
        LqProf prof(LQ_K_GEMM_MAIN, st);
        kern<<<grid, kThreads, C::SMEM, st>>>(tA0, tB0, tA1, tB1, tC, p);
        LQ_CUDA(cudaGetLastError());
    }
    if (p.tail_splits > 1) {
        LqProf prof(LQ_K_REDUCE, st);
        constexpr int RPB = 256 / (BLOCK_N / 4);
        const int blocks = rem * ((256 + RPB - 1) / RPB);
        pair_tail_reduce_kernel<BLOCK_N><<<blocks, 256, 0, st>>>(p);
        LQ_CUDA(cudaGetLastError());
    }
}

// Tile width for the pair kernel.  Measured on config 2's backward (512 tiles of 192 columns in 7
// rounds of 74 pairs against 384 tiles of 256 columns in 6): a 192-column tile takes about as long
// as a 256-column one (the MMA does not get cheaper in proportion), so what counts is the number of
// rounds; 192 is taken only when it saves rounds or padding columns outright.
inline int forced_pair_bn() {
    static const int v = [] { const char* e = getenv("LQ_PAIR_BN"); return e ? atoi(e) : 0; }();
    return v;
}
inline int pair_block_n(int64_t Mg, int64_t Ng, int sm_count, int kb_total = 0) {
    if (forced_pair_bn() == 192 || forced_pair_bn() == 256) return forced_pair_bn();
    const int64_t pairs = std::max(1, sm_count / 2);
    auto cost = [&](int bn) {
        const int64_t tiles = ((Mg + 255) / 256) * ((Ng + bn - 1) / bn);
        const int64_t rem = tiles > pairs ? tiles % pairs : tiles;
        double rounds = (double)((tiles + pairs - 1) / pairs);
        // a last round that is at most half full is cut along k (launch_gemm_pair): it costs its share
        // of a round plus the launch that sums the partial tiles
        if (g_tail_split.load() != 0 && rem > 0 && 2 * rem <= pairs && kb_total >= kMinTailKBlocks)
            rounds += -1.0 + 1.0 / (double)std::min<int64_t>(pairs / rem, kMaxTailSplits) + 0.3;
        return rounds * (bn == 256 ? 1.0 : 0.95);
    };
    return cost(192) < cost(256) ? 192 : 256;
}

// Splits of a 64-wide contraction: the persistent grid walks `tiles * s` items in rounds of one CTA
// per SM, so what counts is (rounds) x (k-blocks per item + a fixed cost per item), plus the partial
// tiles the summing launch has to read.  (The former rule, about two items per SM, put config 2's
// dH = dY . B^T at 5 splits = 320 items = 2.16 rounds run as 3; 4 splits run as 2.)
int choose_splits(int64_t out_tiles, int64_t k_blocks, int sm_count) {
    int best = 1;
    double best_cost = 0.0;
    for (int s = 1; s <= 16 && s <= k_blocks; ++s) {
        const int64_t rounds = (out_tiles * s + sm_count - 1) / sm_count;
        const double cost = (double)rounds * ((double)((k_blocks + s - 1) / s) + 4.0) + 0.75 * s;
        if (s == 1 || cost < best_cost) {
            best = s;
            best_cost = cost;
        }
    }
    return best;
}

inline size_t al256(size_t x) { return (x + 255) & ~size_t(255); }
inline int ext_width(int r) { return 64 * ((r + 63) / 64); }

struct TcWs {
    __nv_bfloat16* wscr;  // dequantized weight: [M, K] (fwd) or [K, M] (bwd)
    float* Hf;            // [N, r]
    float* dHf;           // [N, r]
    __nv_bfloat16* ext_a; // [N, EXT]  fwd: s*H      bwd: dH
    __nv_bfloat16* ext_b; // [N, EXT]                bwd: s*H
    __nv_bfloat16* pdown; // fwd: A^T [r, K]         bwd: B [r, M]
    __nv_bfloat16* pext;  // fwd: B^T [M, EXT]       bwd: A [K, EXT]
    float* part;          // split partials
    float* part2;         // split partials of the contractions that run on the side stream (dB, recomputed H)
    __nv_bfloat16* pdown2; // bwd, H recomputed: A^T [r, K]
    float* tail;          // f32 partial tiles of a frozen GEMM whose last round is cut along k
    size_t bytes;
};

TcWs carve_tc(const lq_weight* w, int64_t N, int r, void* base, int sm_count) {
    const size_t M = (size_t)w->M, K = (size_t)w->K;
    const size_t EXT = (size_t)ext_width(r > 0 ? r : 1);
    size_t off = 0;
    auto take = [&](size_t bytes) {
        size_t o = al256(off);
        off = o + bytes;
        return base ? (void*)((char*)base + o) : nullptr;
    };
    TcWs t{};
    t.wscr = (__nv_bfloat16*)take(M * K * 2);
    t.tail = N >= 256 ? (float*)take(kTailWsBytes) : nullptr;
    if (r > 0) {
        t.Hf = (float*)take((size_t)N * r * 4);
        t.dHf = (float*)take((size_t)N * r * 4);
        t.ext_a = (__nv_bfloat16*)take((size_t)N * EXT * 2);
        t.ext_b = (__nv_bfloat16*)take((size_t)N * EXT * 2);
        t.pdown = (__nv_bfloat16*)take((size_t)r * std::max(M, K) * 2);
        t.pext = (__nv_bfloat16*)take(std::max(M, K) * EXT * 2);
        size_t rows = std::max((size_t)N, std::max(M, K));
        (void)sm_count;
        t.part = (float*)take((size_t)16 * rows * EXT * 4);
        t.part2 = (float*)take((size_t)16 * rows * EXT * 4);
        t.pdown2 = (__nv_bfloat16*)take((size_t)r * K * 2);
    }
    t.bytes = al256(off);
    return t;
}

// Out[I, r] = alpha * Z[I, C] . P[r, C]^T  via split-K tcgen05 GEMM + fixed-order reduce.
void skinny_down(const void* Z, int64_t I, int64_t Cdim, int64_t ldz, const __nv_bfloat16* P, int64_t ldp_in, int r,
                 float alpha, float* out_f32, __nv_bfloat16* ext, float ext_scale, float* part, int sm_count,
                 cudaStream_t st, const float* ext_row_div = nullptr, ForkJoin* wait_before_reduce = nullptr) {
    const int EXT = ext_width(r);
    const int64_t kb = (Cdim + BK - 1) / BK;
    const int64_t m_tiles = (I + BM - 1) / BM, n_tiles = EXT / 64;
    const int splits = choose_splits(m_tiles * n_tiles, kb, sm_count);
    Operand a{Z, false, ldz}, b{P, false, ldp_in};
    launch_gemm<64, false, false, float>(a, b, Cdim, nullptr, nullptr, 0, part, EXT, I * (int64_t)EXT, I, EXT, splits,
                                         nullptr, st, r, LQ_K_GEMM_DOWN);
    long long total = (long long)I * EXT;
    if (wait_before_reduce) wait_before_reduce->wait(0);  // `ext_row_div` is produced on the side stream
    LqProf prof(LQ_K_REDUCE, st);
    reduce_partials_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(part, I * (long long)EXT, splits, EXT, I, r,
                                                                          EXT, alpha, out_f32, r, 0, 0, ext, EXT,
                                                                          ext_scale, ext_row_div);
    LQ_CUDA(cudaGetLastError());
}

// Out = alpha * Z[Nred, C]^T . T[Nred, EXT]  (reduction over rows), Out is [C, r] or transposed [r, C].
void skinny_grad(const void* Z, int64_t Nred, int64_t Cdim, int64_t ldz, const __nv_bfloat16* T, int r, float alpha,
                 float* out, int transposed, int accumulate, float* part, int sm_count, cudaStream_t st) {
    const int EXT = ext_width(r);
    const int64_t kb = (Nred + BK - 1) / BK;
    const int64_t m_tiles = (Cdim + BM - 1) / BM, n_tiles = EXT / 64;
    const int splits = choose_splits(m_tiles * n_tiles, kb, sm_count);
    Operand a{Z, true, ldz}, b{T, true, (int64_t)EXT};
    launch_gemm<64, true, true, float>(a, b, Nred, nullptr, nullptr, 0, part, EXT, Cdim * (int64_t)EXT, Cdim, EXT, splits,
                                       nullptr, st, -1, LQ_K_GEMM_GRAD);
    long long total = (long long)Cdim * EXT;
    LqProf prof(LQ_K_REDUCE, st);
    reduce_partials_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(
        part, Cdim * (long long)EXT, splits, EXT, Cdim, r, EXT, alpha, out, transposed ? Cdim : r, transposed,
        accumulate, nullptr, 0, 0.f);
    LQ_CUDA(cudaGetLastError());
}

void cast_pad(const float* in, long long si, long long sj, __nv_bfloat16* out, long long ldo, long long I, int J,
              int Jpad, float alpha, cudaStream_t st, const float* row_div = nullptr, int row_div_bcast = 0) {
    long long total = I * Jpad;
    if (total <= 0) return;
    LqProf prof(LQ_K_PREP, st);
    cast_pad_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(in, si, sj, out, ldo, I, J, Jpad, alpha, row_div,
                                                                     row_div_bcast);
    LQ_CUDA(cudaGetLastError());
}

// ---- bf16 mirror of one site's LoRA factors ----------------------------------------------------
// The tensor-core path consumes A and B as four bf16 operand arrays.  Casting them inside every call
// costs five short launches per forward + backward; the factors change once per optimizer step, so
// a caller may keep this mirror beside the f32 parameters and refresh it after each update.
//   At [r, K]    A transposed (B operand of H = X . A, and of the recomputed H)
//   Bt [M, EXT]  B transposed, zero padded to EXT columns (K extension of the forward GEMM)
//   Bb [r, M]    B (B operand of dH = s . dY . B^T)
//   Ap [K, EXT]  A, zero padded (K extension of the dX GEMM)
struct LoraMirror {
    __nv_bfloat16 *At, *Bt, *Bb, *Ap;
    size_t bytes;
};
LoraMirror carve_mirror(int64_t K, int64_t M, int r, void* base) {
    const size_t EXT = (size_t)ext_width(r);
    size_t off = 0;
    auto take = [&](size_t bytes) {
        size_t o = al256(off);
        off = o + bytes;
        return base ? (__nv_bfloat16*)((char*)base + o) : nullptr;
    };
    LoraMirror m;
    m.At = take((size_t)r * K * 2);
    m.Bt = take((size_t)M * EXT * 2);
    m.Bb = take((size_t)r * M * 2);
    m.Ap = take((size_t)K * EXT * 2);
    m.bytes = al256(off);
    return m;
}

__global__ void __launch_bounds__(256) lora_mirror_kernel(const float* __restrict__ A, const float* __restrict__ B,
                                                          long long K, long long M, int r, int EXT, LoraMirror m) {
    const long long n0 = (long long)r * K, n1 = M * EXT, n2 = (long long)r * M, n3 = K * EXT;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n0 + n1 + n2 + n3;
         i += (long long)gridDim.x * blockDim.x) {
        if (i < n0) {  // At[j, k] = A[k, j]
            const long long j = i / K, k = i - j * K;
            m.At[i] = __float2bfloat16(A[k * r + j]);
        } else if (i < n0 + n1) {  // Bt[mm, j] = B[j, mm]
            const long long t = i - n0, mm = t / EXT;
            const int j = (int)(t - mm * EXT);
            m.Bt[t] = __float2bfloat16(j < r ? B[(long long)j * M + mm] : 0.f);
        } else if (i < n0 + n1 + n2) {
            const long long t = i - n0 - n1;
            m.Bb[t] = __float2bfloat16(B[t]);
        } else {  // Ap[k, j] = A[k, j]
            const long long t = i - n0 - n1 - n2, k = t / EXT;
            const int j = (int)(t - k * EXT);
            m.Ap[t] = __float2bfloat16(j < r ? A[k * r + j] : 0.f);
        }
    }
}

template <typename OutT>
void main_gemm(const Operand& a0, const Operand& b0, int64_t K0, const Operand* a1, const Operand* b1, int64_t K1,
               OutT* Cout, int64_t ldc, int64_t Mg, int64_t Ng, const float* bias, int sm_count, cudaStream_t st,
               float* tail_ws = nullptr) {
    // Tile width: 128 x 256 is the efficient shape (96 B/clk of operand traffic per SM); 128 x 128
    // needs 128 B/clk and measured 1.5x slower per FLOP.  128 x 192 sits close to 256 and is taken
    // when it fills the last wave of the persistent grid markedly better.
    if constexpr (sizeof(OutT) == 2) {
        if (pair_enabled() && Mg >= 256 && Ng > 192 && sm_count >= 2) {  // the frozen GEMMs proper: CTA pairs
            if (pair_block_n(Mg, Ng, sm_count, tail_ws ? (int)((K0 + BK - 1) / BK + (a1 ? (K1 + BK - 1) / BK : 0)) : 0) == 256)
                launch_gemm_pair<256, false>(a0, b0, K0, a1, b1, K1, (__nv_bfloat16*)Cout, ldc, Mg, Ng, bias, st,
                                             EpiScales(), tail_ws);
            else
                launch_gemm_pair<192, false>(a0, b0, K0, a1, b1, K1, (__nv_bfloat16*)Cout, ldc, Mg, Ng, bias, st,
                                             EpiScales(), tail_ws);
            return;
        }
    }
    const int64_t m_tiles = (Mg + BM - 1) / BM;
    auto waves_eff = [&](int bn) {
        const int64_t tiles = m_tiles * ((Ng + bn - 1) / bn);
        const int64_t rounds = (tiles + sm_count - 1) / sm_count;
        const double pad = (double)Ng / (double)(((Ng + bn - 1) / bn) * bn);
        return pad * (double)tiles / (double)(rounds * sm_count);
    };
    if (Ng <= 128) {
        launch_gemm<128, false, false, OutT>(a0, b0, K0, a1, b1, K1, Cout, ldc, 0, Mg, Ng, 1, bias, st);
    } else if (Ng > 192 && waves_eff(256) >= 0.95 * waves_eff(192)) {
        launch_gemm<256, false, false, OutT>(a0, b0, K0, a1, b1, K1, Cout, ldc, 0, Mg, Ng, 1, bias, st);
    } else {
        launch_gemm<192, false, false, OutT>(a0, b0, K0, a1, b1, K1, Cout, ldc, 0, Mg, Ng, 1, bias, st);
    }
}


// =========================================================================================
// Native fp8 compute (w8a8): e4m3 weights straight from HBM x e4m3 activations
// =========================================================================================
//
// For scaled-fp8 weights the frozen GEMM can run on tcgen05's kind::f8f6f4 at twice the bf16 rate
// with NO dequantisation pass: TMA loads the stored e4m3 bytes as the MMA operand.  The activations
// are quantised to e4m3 on the fly with one f32 scale per token (absmax / 448); the scales are
// applied in the epilogue, v = acc * s_row[n] * s_w[m].  In the backward the weight scale lies on
// the reduction axis (dX = (dY . diag(s_w)) . W8), so it is folded into dY before dY is quantised.
// The LoRA K extension stays bf16 (its operands are pre-divided by the scales the epilogue applies),
// so the trained low-rank path never passes through 8 bits.

// One block per row: q[n, :] = e4m3(x[n, :] * colmul[:] / s_n), s_n = max(absmax / 448, 1e-12).
__global__ void __launch_bounds__(256) quant_rows_e4m3_kernel(const __nv_bfloat16* __restrict__ x, long long C,
                                                              const float* __restrict__ colmul,
                                                              uint8_t* __restrict__ q, float* __restrict__ scale) {
    __shared__ float red[8];
    __shared__ float s_inv;
    const long long n = blockIdx.x;
    const __nv_bfloat16* xr = x + n * C;
    float amax = 0.f;
    for (long long c = (long long)threadIdx.x * 8; c < C; c += 256 * 8) {  // C % 8 == 0
        const uint4 v = *(const uint4*)(xr + c);
        const __nv_bfloat162* h = (const __nv_bfloat162*)&v;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            float2 f = __bfloat1622float2(h[e]);
            if (colmul) { f.x *= colmul[c + 2 * e]; f.y *= colmul[c + 2 * e + 1]; }
            amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
        }
    }
    for (int off = 16; off >= 1; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
    __syncthreads();
    if (threadIdx.x == 0) {
        float a = red[0];
        for (int i = 1; i < 8; ++i) a = fmaxf(a, red[i]);
        const float s = fmaxf(__fdiv_rn(a, 448.f), 1e-12f);
        scale[n] = s;
        s_inv = __fdiv_rn(1.f, s);
    }
    __syncthreads();
    const float inv = s_inv;
    uint8_t* qr = q + n * C;
    for (long long c = (long long)threadIdx.x * 8; c < C; c += 256 * 8) {
        const uint4 v = *(const uint4*)(xr + c);  // second read of the row: L1/L2 hit
        const __nv_bfloat162* h = (const __nv_bfloat162*)&v;
        uint32_t out[2] = {0u, 0u};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            float2 f = __bfloat1622float2(h[e]);
            if (colmul) { f.x *= colmul[c + 2 * e]; f.y *= colmul[c + 2 * e + 1]; }
            f.x *= inv;
            f.y *= inv;
            const uint32_t pr = (uint32_t)__nv_cvt_float2_to_fp8x2(f, __NV_SATFINITE, __NV_E4M3);  // RNE, saturating
            out[e >> 1] |= pr << (16 * (e & 1));
        }
        *(uint2*)(qr + c) = make_uint2(out[0], out[1]);
    }
}

// Same result, single pass over HBM: a persistent block walks rows; every thread owns a fixed set of
// 8-column vectors (VPT of them), keeps their column multipliers in registers for the whole launch
// and the row's values in registers between the absmax reduction and the conversion.
template <int VPT>
__global__ void __launch_bounds__(256) quant_rows_e4m3_reg_kernel(const __nv_bfloat16* __restrict__ x, long long N,
                                                                  long long C, const float* __restrict__ colmul,
                                                                  uint8_t* __restrict__ q, float* __restrict__ scale) {
    __shared__ float red[2][8];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float cm[VPT][8];
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const long long c = ((long long)i * 256 + threadIdx.x) * 8;
#pragma unroll
        for (int e = 0; e < 8; ++e) cm[i][e] = (colmul && c < C) ? colmul[c + e] : 1.f;
    }
    int buf = 0;
    for (long long n = blockIdx.x; n < N; n += gridDim.x, buf ^= 1) {
        const __nv_bfloat16* xr = x + n * C;
        float f[VPT][8];
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const long long c = ((long long)i * 256 + threadIdx.x) * 8;
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (c < C) v = *(const uint4*)(xr + c);
            const __nv_bfloat162* h = (const __nv_bfloat162*)&v;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 t = __bfloat1622float2(h[e]);
                f[i][2 * e] = t.x * cm[i][2 * e];
                f[i][2 * e + 1] = t.y * cm[i][2 * e + 1];
                amax = fmaxf(amax, fmaxf(fabsf(f[i][2 * e]), fabsf(f[i][2 * e + 1])));
            }
        }
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
        if (lane == 0) red[buf][warp] = amax;
        __syncthreads();  // double-buffered: the next row's writes go to the other half
        float a = red[buf][0];
#pragma unroll
        for (int i = 1; i < 8; ++i) a = fmaxf(a, red[buf][i]);
        const float s = fmaxf(__fdiv_rn(a, 448.f), 1e-12f);
        const float inv = __fdiv_rn(1.f, s);
        if (threadIdx.x == 0) scale[n] = s;
        uint8_t* qr = q + n * C;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const long long c = ((long long)i * 256 + threadIdx.x) * 8;
            if (c < C) {
                uint32_t out[2] = {0u, 0u};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 t = make_float2(f[i][2 * e] * inv, f[i][2 * e + 1] * inv);
                    const uint32_t pr = (uint32_t)__nv_cvt_float2_to_fp8x2(t, __NV_SATFINITE, __NV_E4M3);
                    out[e >> 1] |= pr << (16 * (e & 1));
                }
                *(uint2*)(qr + c) = make_uint2(out[0], out[1]);
            }
        }
    }
}

// out[k, m] = in[m, k] for e4m3 bytes (load-time: the backward wants the weight K-major in d_out).
__global__ void __launch_bounds__(256) transpose_u8_kernel(const uint8_t* __restrict__ in, long long M, long long K,
                                                           uint8_t* __restrict__ out) {
    __shared__ uint8_t t[64][65];
    const long long m0 = (long long)blockIdx.y * 64, k0 = (long long)blockIdx.x * 64;
    const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;
    for (int i = ty; i < 64; i += 4)
        t[i][tx] = (m0 + i < M && k0 + tx < K) ? in[(m0 + i) * K + k0 + tx] : 0;
    __syncthreads();
    for (int i = ty; i < 64; i += 4)
        if (k0 + i < K && m0 + tx < M) out[(k0 + i) * M + m0 + tx] = t[tx][i];
}

struct W8Ws {
    uint8_t* q8;          // quantised activations: [N, K] (fwd) or [N, M] (bwd)
    float* srow;          // [N] per-token scale
    float* Hf;            // [N, r]
    float* dHf;           // [N, r]
    __nv_bfloat16* ext_a; // [N, EXT]  extension operand (pre-divided by the row scale)
    __nv_bfloat16* ext_b; // [N, EXT]  s*H   (dB operand)
    __nv_bfloat16* ext_c; // [N, EXT]  dH    (dA operand)
    __nv_bfloat16* pdown; // A^T [r, K] / B [r, M]
    __nv_bfloat16* pext;  // B^T [M, EXT] / A [K, EXT]
    float* part;
    float* part2;          // partials of the contractions on the side stream (dB, recomputed H)
    __nv_bfloat16* pdown2; // bwd, H recomputed: A^T [r, K]
    float* tail;           // f32 partial tiles of a frozen GEMM whose last round is cut along k
    size_t bytes;
};

W8Ws carve_w8(const lq_weight* w, int64_t N, int r, void* base) {
    const size_t M = (size_t)w->M, K = (size_t)w->K;
    const size_t EXT = (size_t)ext_width(r > 0 ? r : 1);
    size_t off = 0;
    auto take = [&](size_t bytes) {
        size_t o = al256(off);
        off = o + bytes;
        return base ? (void*)((char*)base + o) : nullptr;
    };
    W8Ws t{};
    t.q8 = (uint8_t*)take((size_t)N * std::max(M, K));
    t.srow = (float*)take((size_t)N * 4);
    t.tail = N >= 256 ? (float*)take(kTailWsBytes) : nullptr;
    if (r > 0) {
        t.Hf = (float*)take((size_t)N * r * 4);
        t.dHf = (float*)take((size_t)N * r * 4);
        t.ext_a = (__nv_bfloat16*)take((size_t)N * EXT * 2);
        t.ext_b = (__nv_bfloat16*)take((size_t)N * EXT * 2);
        t.ext_c = (__nv_bfloat16*)take((size_t)N * EXT * 2);
        t.pdown = (__nv_bfloat16*)take((size_t)r * std::max(M, K) * 2);
        t.pext = (__nv_bfloat16*)take(std::max(M, K) * EXT * 2);
        t.part = (float*)take((size_t)16 * std::max((size_t)N, std::max(M, K)) * EXT * 4);
        t.part2 = (float*)take((size_t)16 * std::max((size_t)N, std::max(M, K)) * EXT * 4);
        t.pdown2 = (__nv_bfloat16*)take((size_t)r * K * 2);
    }
    t.bytes = al256(off);
    return t;
}

void quant_rows(const void* x, int64_t N, int64_t C, const float* colmul, uint8_t* q, float* scale, cudaStream_t st) {
    LqProf prof(LQ_K_DEQUANT, st);
    const __nv_bfloat16* xb = (const __nv_bfloat16*)x;
    const unsigned grid = (unsigned)std::min<int64_t>(N, 148 * 4);
    const int64_t vec = (C + 2047) / 2048;  // 8-column vectors per thread
    if (vec <= 2) quant_rows_e4m3_reg_kernel<2><<<grid, 256, 0, st>>>(xb, N, C, colmul, q, scale);
    else if (vec <= 4) quant_rows_e4m3_reg_kernel<4><<<grid, 256, 0, st>>>(xb, N, C, colmul, q, scale);
    else if (vec <= 6) quant_rows_e4m3_reg_kernel<6><<<grid, 256, 0, st>>>(xb, N, C, colmul, q, scale);
    else if (vec <= 8) quant_rows_e4m3_reg_kernel<8><<<grid, 256, 0, st>>>(xb, N, C, colmul, q, scale);
    else quant_rows_e4m3_kernel<<<(unsigned)N, 256, 0, st>>>(xb, C, colmul, q, scale);
    LQ_CUDA(cudaGetLastError());
}

void main_gemm_f8(const Operand& a0, const Operand& b0, int64_t K0, const Operand* a1, const Operand* b1, int64_t K1,
                  __nv_bfloat16* Cout, int64_t ldc, int64_t Mg, int64_t Ng, const float* bias, const EpiScales& sc,
                  int sm_count, cudaStream_t st, float* tail_ws = nullptr) {
    const int64_t m_tiles = (Mg + BM - 1) / BM;
    auto waves_eff = [&](int bn) {
        const int64_t tiles = m_tiles * ((Ng + bn - 1) / bn);
        const int64_t rounds = (tiles + sm_count - 1) / sm_count;
        const double pad = (double)Ng / (double)(((Ng + bn - 1) / bn) * bn);
        return pad * (double)tiles / (double)(rounds * sm_count);
    };
    using T = __nv_bfloat16;
    if (pair_enabled() && Mg >= 256 && Ng > 192 && sm_count >= 2) {
        if (pair_block_n(Mg, Ng, sm_count, tail_ws ? (int)((K0 + 127) / 128 + (a1 ? (K1 + BK - 1) / BK : 0)) : 0) == 256)
            launch_gemm_pair<256, true>(a0, b0, K0, a1, b1, K1, Cout, ldc, Mg, Ng, bias, st, sc, tail_ws);
        else
            launch_gemm_pair<192, true>(a0, b0, K0, a1, b1, K1, Cout, ldc, Mg, Ng, bias, st, sc, tail_ws);
        return;
    }
    if (Ng <= 128)
        launch_gemm<128, false, false, T, true>(a0, b0, K0, a1, b1, K1, Cout, ldc, 0, Mg, Ng, 1, bias, st, -1, LQ_K_GEMM_MAIN, sc);
    else if (Ng > 192 && waves_eff(256) >= 0.95 * waves_eff(192))
        launch_gemm<256, false, false, T, true>(a0, b0, K0, a1, b1, K1, Cout, ldc, 0, Mg, Ng, 1, bias, st, -1, LQ_K_GEMM_MAIN, sc);
    else
        launch_gemm<192, false, false, T, true>(a0, b0, K0, a1, b1, K1, Cout, ldc, 0, Mg, Ng, 1, bias, st, -1, LQ_K_GEMM_MAIN, sc);
}

std::mutex g_wt_mu;

// The e4m3 weight transposed to [d_in, d_out], built once per handle (first w8a8 backward, or
// explicitly at load time) so that the dX contraction is K-major in d_out like every other operand.
const uint8_t* ensure_transposed(const lq_weight* w, cudaStream_t st) {
    std::lock_guard<std::mutex> lk(g_wt_mu);
    lq_weight* mw = const_cast<lq_weight*>(w);
    if (!mw->packed_t) {
        void* buf = nullptr;
        LQ_CUDA(cudaMalloc(&buf, (size_t)w->M * (size_t)w->K));
        dim3 grid((unsigned)((w->K + 63) / 64), (unsigned)((w->M + 63) / 64));
        LqProf prof(LQ_K_QUANT, st);
        transpose_u8_kernel<<<grid, 256, 0, st>>>((const uint8_t*)w->packed, w->M, w->K, (uint8_t*)buf);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) {
            cudaFree(buf);
            throw LqError(LQ_ERR_CUDA, std::string("transpose_u8_kernel: ") + cudaGetErrorString(e));
        }
        mw->packed_t = buf;
    }
    return (const uint8_t*)mw->packed_t;
}

}  // namespace

// Raster of the CTA-pair GEMMs: the CTAs of a wave run through K in step, so a wave reads each of its
// distinct A and B row bands from DRAM once.  With 16-pair-tile groups a wave is 16 bands of A and
// ncl/16 of B; when that exceeds what L2 keeps comfortably (long K) and the whole B operand is small
// enough to stay resident, waves instead span ALL column tiles of a few A bands: B is then read from
// DRAM once for the whole launch and A streams through.
int lq_tc_pair_group_m(int sm_count, int block_n, int64_t Ng, int64_t K0, int b_elem_bytes, int n_tiles) {
    const int ncl_est = std::max(1, sm_count / 2);
    const double esz = (double)b_elem_bytes;
    const double wave16 = (16.0 * 256 + (double)ncl_est / 16 * block_n) * (double)K0 * esz;
    const double whole_b = (double)Ng * (double)K0 * esz;
    int group_m = 16;
    if (wave16 > 48e6 && whole_b <= 90e6) group_m = std::max(1, (ncl_est + n_tiles - 1) / n_tiles);
    static const int forced = [] { const char* e = getenv("LQ_GROUP_M"); return e ? atoi(e) : 0; }();
    if (forced > 0) group_m = forced;
    return group_m;
}
CUtensorMap lq_tc_make_store_map(const void* base, int64_t cols, int64_t rows, int64_t ld) {
    return make_store_map(base, cols, rows, ld);
}
CUtensorMap lq_tc_make_map(const void* base, int64_t inner, int64_t rows, int64_t ld, int box_rows) {
    return make_map(base, inner, rows, ld, box_rows);
}
cudaStream_t lq_tc_fork(int device, cudaStream_t st) {
    ForkJoin fj(dev_ctx(device), st, true);
    fj.fork();
    return fj.side();
}
void lq_tc_join(int device, cudaStream_t st) {
    ForkJoin fj(dev_ctx(device), st, true);
    fj.join(1);
}

CUtensorMap lq_tc_make_map_u8(const void* base, int64_t inner, int64_t rows, int64_t ld, int box_rows) {
    return make_map(base, inner, rows, ld, box_rows, true);
}
int* lq_tc_status_word(int device) { return dev_ctx(device).status; }
int lq_tc_sm_count(int device) { return dev_ctx(device).sm_count; }

bool lq_tc_supported(const lq_weight* w, int64_t n_tokens, int rank) {
    (void)n_tokens;
    (void)rank;
    return w->K % 8 == 0 && w->M % 8 == 0 && w->K >= 8 && w->M >= 8;
}

size_t lq_tc_workspace_bytes(const lq_weight* w, int64_t n_tokens, int rank) {
    return carve_tc(w, n_tokens, rank, nullptr, 148).bytes;
}

int lq_static_read_sticky(int device);  // the allocation-free split contraction's own error word (below)

int lq_tc_read_status(int device, cudaStream_t st) {
    DevCtx& c = dev_ctx(device);
    int v = 0;
    LQ_CUDA(cudaStreamSynchronize(st));
    LQ_CUDA(cudaMemcpy(&v, c.status, sizeof(int), cudaMemcpyDeviceToHost));
    if (v != 0) LQ_CUDA(cudaMemset(c.status, 0, sizeof(int)));
    const int v2 = lq_static_read_sticky(device);
    return v != 0 ? v : v2;
}

size_t lq_tc_mirror_bytes(int64_t K, int64_t M, int r) { return r > 0 ? carve_mirror(K, M, r, nullptr).bytes : 0; }

bool lq_tc_option_set(const char* name, int value) {
    if (std::strcmp(name, "bwd_mn") == 0) { g_bwd_mn = value; return true; }
    if (std::strcmp(name, "tail_split") == 0) { g_tail_split = value; return true; }
    if (std::strcmp(name, "reserve_sms") == 0) { g_reserve_sms = value; return true; }
    return false;
}

// The mirrors of many sites in one launch (a trainer refreshes all of them after an optimizer step):
// blockIdx.y is the site, the launch parameter carries up to kMirrorBatch sites.
constexpr int kMirrorBatch = 24;
struct MirrorJob {
    const float *A, *B;
    long long K, M;
    int r, EXT;
    LoraMirror m;
};
struct MirrorBatch {
    MirrorJob job[kMirrorBatch];
};
__global__ void __launch_bounds__(256) lora_mirror_batch_kernel(const __grid_constant__ MirrorBatch mb) {
    const MirrorJob& j = mb.job[blockIdx.y];
    const float* __restrict__ A = j.A;
    const float* __restrict__ B = j.B;
    const long long K = j.K, M = j.M;
    const int r = j.r, EXT = j.EXT;
    const long long n0 = (long long)r * K, n1 = M * EXT, n2 = (long long)r * M, n3 = K * EXT;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n0 + n1 + n2 + n3;
         i += (long long)gridDim.x * blockDim.x) {
        if (i < n0) {
            const long long jj = i / K, k = i - jj * K;
            j.m.At[i] = __float2bfloat16(A[k * r + jj]);
        } else if (i < n0 + n1) {
            const long long t = i - n0, mm = t / EXT;
            const int c = (int)(t - mm * EXT);
            j.m.Bt[t] = __float2bfloat16(c < r ? B[(long long)c * M + mm] : 0.f);
        } else if (i < n0 + n1 + n2) {
            const long long t = i - n0 - n1;
            j.m.Bb[t] = __float2bfloat16(B[t]);
        } else {
            const long long t = i - n0 - n1 - n2, k = t / EXT;
            const int c = (int)(t - k * EXT);
            j.m.Ap[t] = __float2bfloat16(c < r ? A[k * r + c] : 0.f);
        }
    }
}

void lq_tc_mirror_build_batch(const lq_mirror_job* jobs, int n, cudaStream_t st) {
    for (int base = 0; base < n; base += kMirrorBatch) {
        const int cnt = std::min(kMirrorBatch, n - base);
        MirrorBatch mb;
        long long most = 0;
        for (int i = 0; i < cnt; ++i) {
            const lq_mirror_job& q = jobs[base + i];
            MirrorJob& j = mb.job[i];
            j.A = q.A;
            j.B = q.B;
            j.K = q.d_in;
            j.M = q.d_out;
            j.r = q.rank;
            j.EXT = ext_width(q.rank);
            j.m = carve_mirror(q.d_in, q.d_out, q.rank, q.mirror);
            most = std::max(most, (long long)j.r * j.K + j.M * j.EXT + (long long)j.r * j.M + j.K * j.EXT);
        }
        for (int i = cnt; i < kMirrorBatch; ++i) mb.job[i] = mb.job[0];
        LqProf prof(LQ_K_PREP, st);
        dim3 grid((unsigned)std::min<long long>((most + 255) / 256, 64), (unsigned)cnt);
        lora_mirror_batch_kernel<<<grid, 256, 0, st>>>(mb);
        LQ_CUDA(cudaGetLastError());
    }
}

void lq_tc_mirror_build(const float* A, const float* B, int64_t K, int64_t M, int r, void* mirror, cudaStream_t st) {
    LoraMirror m = carve_mirror(K, M, r, mirror);
    const int EXT = ext_width(r);
    const long long total = (long long)r * K + M * EXT + (long long)r * M + K * EXT;
    LqProf prof(LQ_K_PREP, st);
    lora_mirror_kernel<<<(unsigned)std::min<long long>((total + 255) / 256, 148 * 8), 256, 0, st>>>(A, B, K, M, r, EXT, m);
    LQ_CUDA(cudaGetLastError());
}

void lq_tc_fwd(const lq_weight* w, const void* X, int64_t N, const float* A, const float* B, int r, float s, void* Y,
               float* H_out, void* ws, size_t ws_bytes, cudaStream_t st, const void* mirror) {
    const int64_t M = w->M, K = w->K;
    DevCtx& ctx = dev_ctx(w->device);
    LQ_CHECK_ARG(ws != nullptr, "workspace is NULL");
    LQ_CHECK_ARG(((uintptr_t)ws & 255) == 0, "workspace must be 256-byte aligned");
    TcWs t = carve_tc(w, N, r, ws, ctx.sm_count);
    if (t.bytes > ws_bytes)
        throw LqError(LQ_ERR_WORKSPACE, "workspace too small: need " + std::to_string(t.bytes) + " bytes, got " +
                                            std::to_string(ws_bytes));
    Operand a0{X, false, K}, b0{t.wscr, false, K};
    // int4 weights at tile-filling sizes: the weight is converted inside the GEMM's mainloop and no
    // bf16 copy of it is written; otherwise it is dequantised once per call into the scratch
    const bool w4 = !w->bf16_copy && lq_w4_supported(w, N, 0);
    const bool cached = w->bf16_copy != nullptr;  // a resident bf16 copy stands in for the per-call scratch
    if (cached) b0.ptr = w->bf16_copy;
    if (r == 0) {
        if (w4) {
            lq_w4_gemm(w, 0, X, K, nullptr, 0, nullptr, 0, 0, Y, M, N, w->bias, st);
            return;
        }
        if (!cached) lq_launch_dequant(w, t.wscr, LQ_BF16, K, 0, st);
        main_gemm<__nv_bfloat16>(a0, b0, K, nullptr, nullptr, 0, (__nv_bfloat16*)Y, M, N, M, w->bias, ctx.sm_count, st, t.tail);
        return;
    }
    const int EXT = ext_width(r);
    if (mirror) {  // the caller keeps the factors' bf16 operands: nothing to cast
        const LoraMirror m = carve_mirror(K, M, r, const_cast<void*>(mirror));
        t.pdown = m.At;
        t.pext = m.Bt;
    }
    ForkJoin fj(ctx, st, !((w4 || cached) && mirror));  // nothing is left for a second stream in that case
    fj.fork();
    // main: H = X . A  (f32 [N, r] for the backward; bf16 s*H, zero padded, as the K extension).
    // Enqueued BEFORE the side stream's dequantisation pass: that pass is thousands of small blocks
    // which, launched first, hold every SM until they drain, so the two ran one after the other
    // (config 2: 33 + 20 us); launched second they fill in beside the persistent 64-wide GEMM.
    if (!mirror) cast_pad(A, 1, r, t.pdown, K, r, (int)K, (int)K, 1.f, st);  // A^T [r, K]
    float* Hf = H_out ? H_out : t.Hf;
    skinny_down(X, N, K, K, t.pdown, K, r, 1.f, Hf, t.ext_a, s, t.part, ctx.sm_count, st);
    // side: frozen weight -> bf16 scratch [M, K] (rounds q*scale, resp. LUT*scale, once to bf16),
    //       and B^T [M, EXT] for the K extension
    if (!w4 && !cached) lq_launch_dequant(w, t.wscr, LQ_BF16, K, 0, fj.side());
    if (!mirror) cast_pad(B, 1, M, t.pext, EXT, M, r, EXT, 1.f, fj.side());
    fj.join(0);
    // Y = [X | s*H] . [W | B^T]^T + bias
    if (w4) {
        lq_w4_gemm(w, 0, X, K, t.ext_a, EXT, t.pext, EXT, EXT, Y, M, N, w->bias, st);
        return;
    }
    Operand a1{t.ext_a, false, EXT}, b1{t.pext, false, EXT};
    main_gemm<__nv_bfloat16>(a0, b0, K, &a1, &b1, EXT, (__nv_bfloat16*)Y, M, N, M, w->bias, ctx.sm_count, st, t.tail);
}

void lq_tc_bwd(const lq_weight* w, const void* dY, const void* X, const float* H, int64_t N, const float* A,
               const float* B, int r, float s, void* dX, float* dA, float* dB, int accumulate, void* ws,
               size_t ws_bytes, cudaStream_t st, const void* mirror) {
    const int64_t M = w->M, K = w->K;
    DevCtx& ctx = dev_ctx(w->device);
    LQ_CHECK_ARG(ws != nullptr, "workspace is NULL");
    LQ_CHECK_ARG(((uintptr_t)ws & 255) == 0, "workspace must be 256-byte aligned");
    TcWs t = carve_tc(w, N, r, ws, ctx.sm_count);
    if (t.bytes > ws_bytes)
        throw LqError(LQ_ERR_WORKSPACE, "workspace too small: need " + std::to_string(t.bytes) + " bytes, got " +
                                            std::to_string(ws_bytes));
    const int EXT = ext_width(r > 0 ? r : 1);
    Operand a0{dY, false, M}, b0{t.wscr, false, M};
    const bool w4 = dX && !w->bf16_copy && lq_w4_supported(w, N, 1);
    // a resident bf16 copy [M, K] is read as an MN-major B operand (reduction over its rows) by the
    // CTA-pair kernel: no transposed scratch is written
    const bool mn_ok = dX && pair_enabled() && N >= 256 && K > 192 && ctx.sm_count >= 2;
    const bool cached = mn_ok && w->bf16_copy;
    // without a resident copy the same operand form serves the per-call scratch: the weight is
    // dequantised in its own [M, K] orientation (the cheaper pass: full output lines per warp, no
    // staging) and the dX GEMM reads the scratch MN-major
    const bool mn_scratch = mn_ok && !cached && !w4 && g_bwd_mn.load() != 0 && K % 8 == 0;
    Operand bmn{cached ? (const void*)w->bf16_copy : (const void*)t.wscr, true, K};
    if (r == 0) {
        if (dX && w4) {
            lq_w4_gemm(w, 1, dY, M, nullptr, 0, nullptr, 0, 0, dX, K, N, nullptr, st);
        } else if (dX && (cached || mn_scratch)) {
            if (mn_scratch) lq_launch_dequant(w, t.wscr, LQ_BF16, K, 0, st);
            launch_gemm_pair<256, false, true>(a0, bmn, M, nullptr, nullptr, 0, (__nv_bfloat16*)dX, K, N, K, nullptr, st,
                                               EpiScales(), t.tail);
        } else if (dX) {
            lq_launch_dequant(w, t.wscr, LQ_BF16, M, 1, st);  // W^T [K, M]
            main_gemm<__nv_bfloat16>(a0, b0, M, nullptr, nullptr, 0, (__nv_bfloat16*)dX, K, N, K, nullptr, ctx.sm_count, st, t.tail);
        }
        return;
    }
    if (mirror) {
        const LoraMirror m = carve_mirror(K, M, r, const_cast<void*>(mirror));
        t.pdown = m.Bb;
        t.pext = m.Ap;
        t.pdown2 = m.At;
    }
    ForkJoin fj(ctx, st, true);
    fj.fork();
    // main, first in issue order (see lq_tc_fwd): dH = s * dY . B^T   (f32 [N, r]; bf16 copy as the K
    // extension of the dX GEMM and as dA's operand)
    if (!mirror) cast_pad(B, M, 1, t.pdown, M, r, (int)M, (int)M, 1.f, st);  // B as bf16 [r, M]
    skinny_down(dY, N, M, M, t.pdown, M, r, s, t.dHf, t.ext_a, 1.f, t.part, ctx.sm_count, st);
    // side: what the dX GEMM needs besides dH: W^T [K, M] and A [K, EXT] in bf16
    if (dX) {
        if (mn_scratch) lq_launch_dequant(w, t.wscr, LQ_BF16, K, 0, fj.side());       // W [M, K]
        else if (!w4 && !cached) lq_launch_dequant(w, t.wscr, LQ_BF16, M, 1, fj.side());  // W^T [K, M]
        if (!mirror) cast_pad(A, r, 1, t.pext, EXT, K, r, EXT, 1.f, fj.side());
    }
    fj.record(0);  // the caller's stream waits for this point just before the dX GEMM
    // side, continued (independent of everything on the caller's stream): dB[r, M] = (s*H)^T . dY
    if (dB) {
        const float* Hsrc = H;
        if (!Hsrc) {  // H not kept by the caller: recompute it (own cast buffer: pdown holds B meanwhile)
            if (!mirror) cast_pad(A, 1, r, t.pdown2, K, r, (int)K, (int)K, 1.f, fj.side());
            skinny_down(X, N, K, K, t.pdown2, K, r, 1.f, t.Hf, t.ext_b, s, t.part2, ctx.sm_count, fj.side());
        } else {
            cast_pad(Hsrc, r, 1, t.ext_b, EXT, N, r, EXT, s, fj.side());
        }
        skinny_grad(dY, N, M, M, t.ext_b, r, 1.f, dB, 1, accumulate, t.part2, ctx.sm_count, fj.side());
    }
    // dA[K, r] = X^T . dH stays on the caller's stream, after the dX GEMM: the dB chain on the side
    // stream and dA then run beside each other at the end of the call (both on the side stream, one
    // after the other, measured 2.5 % slower per config-2 step)
    if (dX) {  // dX = [dY | dH] . [W^T | A]^T
        fj.wait(0);
        if (w4) {
            lq_w4_gemm(w, 1, dY, M, t.ext_a, EXT, t.pext, EXT, EXT, dX, K, N, nullptr, st);
        } else if (cached || mn_scratch) {
            Operand a1{t.ext_a, false, EXT}, b1{t.pext, false, EXT};
            launch_gemm_pair<256, false, true>(a0, bmn, M, &a1, &b1, EXT, (__nv_bfloat16*)dX, K, N, K, nullptr, st,
                                               EpiScales(), t.tail);
        } else {
            Operand a1{t.ext_a, false, EXT}, b1{t.pext, false, EXT};
            main_gemm<__nv_bfloat16>(a0, b0, M, &a1, &b1, EXT, (__nv_bfloat16*)dX, K, N, K, nullptr, ctx.sm_count, st, t.tail);
        }
    }
    if (dA)  // dA[K, r] = X^T . dH
        skinny_grad(X, N, K, K, t.ext_a, r, 1.f, dA, 0, accumulate, t.part, ctx.sm_count, st);
    fj.join(1);
}

// ---- native fp8 (w8a8) entry points ------------------------------------------------------

bool lq_w8a8_supported(const lq_weight* w, int64_t n_tokens, int rank) {
    (void)n_tokens;
    (void)rank;
    return w->scheme == LQ_FP8_E4M3 && w->K % 16 == 0 && w->M % 16 == 0;
}

size_t lq_w8a8_workspace_bytes(const lq_weight* w, int64_t n_tokens, int rank) {
    return carve_w8(w, n_tokens, rank, nullptr).bytes;
}

void lq_w8a8_prepare_backward(const lq_weight* w, cudaStream_t st) { ensure_transposed(w, st); }

void lq_w8a8_fwd(const lq_weight* w, const void* X, int64_t N, const float* A, const float* B, int r, float s, void* Y,
                 float* H_out, void* ws, size_t ws_bytes, cudaStream_t st) {
    const int64_t M = w->M, K = w->K;
    DevCtx& ctx = dev_ctx(w->device);
    LQ_CHECK_ARG(ws != nullptr && ((uintptr_t)ws & 255) == 0, "workspace must be non-NULL and 256-byte aligned");
    W8Ws t = carve_w8(w, N, r, ws);
    if (t.bytes > ws_bytes)
        throw LqError(LQ_ERR_WORKSPACE, "workspace too small: need " + std::to_string(t.bytes) + " bytes, got " +
                                            std::to_string(ws_bytes));
    const bool per_channel = w->scale_kind == LQ_SCALE_PER_CHANNEL;
    EpiScales sc;
    sc.row = t.srow;
    sc.col = w->scales;
    sc.col_bcast = per_channel ? 0 : 1;
    Operand a0{t.q8, false, K}, b0{w->packed, false, K};
    if (r == 0) {
        quant_rows(X, N, K, nullptr, t.q8, t.srow, st);  // X -> e4m3 with one scale per token
        main_gemm_f8(a0, b0, K, nullptr, nullptr, 0, (__nv_bfloat16*)Y, M, N, M, w->bias, sc, ctx.sm_count, st, t.tail);
        return;
    }
    const int EXT = ext_width(r);
    ForkJoin fj(ctx, st, true);
    fj.fork();
    // side: X -> e4m3 with one scale per token; B^T / s_w[m] for the K extension
    quant_rows(X, N, K, nullptr, t.q8, t.srow, fj.side());
    cast_pad(B, 1, M, t.pext, EXT, M, r, EXT, 1.f, fj.side(), w->scales, per_channel ? 0 : 1);
    fj.record(0);
    // main: H = X . A (bf16 operands, f32 out); extension operand s*H / s_x[n] (the reduce waits for s_x)
    cast_pad(A, 1, r, t.pdown, K, r, (int)K, (int)K, 1.f, st);
    float* Hf = H_out ? H_out : t.Hf;
    skinny_down(X, N, K, K, t.pdown, K, r, 1.f, Hf, t.ext_a, s, t.part, ctx.sm_count, st, t.srow, &fj);
    fj.wait(0);
    // Y = (X8 . W8^T + ext) * s_x[n] * s_w[m] + bias
    Operand a1{t.ext_a, false, EXT}, b1{t.pext, false, EXT};
    main_gemm_f8(a0, b0, K, &a1, &b1, EXT, (__nv_bfloat16*)Y, M, N, M, w->bias, sc, ctx.sm_count, st, t.tail);
}

void lq_w8a8_bwd(const lq_weight* w, const void* dY, const void* X, const float* H, int64_t N, const float* A,
                 const float* B, int r, float s, void* dX, float* dA, float* dB, int accumulate, void* ws,
                 size_t ws_bytes, cudaStream_t st) {
    const int64_t M = w->M, K = w->K;
    DevCtx& ctx = dev_ctx(w->device);
    LQ_CHECK_ARG(ws != nullptr && ((uintptr_t)ws & 255) == 0, "workspace must be non-NULL and 256-byte aligned");
    W8Ws t = carve_w8(w, N, r, ws);
    if (t.bytes > ws_bytes)
        throw LqError(LQ_ERR_WORKSPACE, "workspace too small: need " + std::to_string(t.bytes) + " bytes, got " +
                                            std::to_string(ws_bytes));
    const bool per_channel = w->scale_kind == LQ_SCALE_PER_CHANNEL;
    const int EXT = ext_width(r > 0 ? r : 1);
    EpiScales sc;
    if (dX) {
        sc.row = t.srow;
        if (!per_channel) { sc.col = w->scales; sc.col_bcast = 1; }
    }
    if (r == 0) {
        if (dX) {
            const uint8_t* wt = ensure_transposed(w, st);
            quant_rows(dY, N, M, per_channel ? w->scales : nullptr, t.q8, t.srow, st);
            Operand a0{t.q8, false, M}, b0{wt, false, M};
            main_gemm_f8(a0, b0, M, nullptr, nullptr, 0, (__nv_bfloat16*)dX, K, N, K, nullptr, sc, ctx.sm_count, st, t.tail);
        }
        return;
    }
    ForkJoin fj(ctx, st, true);
    fj.fork();
    const uint8_t* wt = nullptr;
    if (dX) {
        // side: dY' = dY * s_w[m] (per-channel scale folded in: it lies on the reduction axis), then e4m3
        // per token; A [K, EXT] (/ s_w when that is a scalar) for the K extension
        wt = ensure_transposed(w, fj.side());
        quant_rows(dY, N, M, per_channel ? w->scales : nullptr, t.q8, t.srow, fj.side());
        cast_pad(A, r, 1, t.pext, EXT, K, r, EXT, 1.f, fj.side(), per_channel ? nullptr : w->scales, 1);
    }
    fj.record(0);
    if (dB) {  // side, continued: dB = (s*H)^T . dY, independent of everything on the caller's stream
        if (!H) {
            cast_pad(A, 1, r, t.pdown2, K, r, (int)K, (int)K, 1.f, fj.side());
            skinny_down(X, N, K, K, t.pdown2, K, r, 1.f, t.Hf, t.ext_b, s, t.part2, ctx.sm_count, fj.side());
        } else {
            cast_pad(H, r, 1, t.ext_b, EXT, N, r, EXT, s, fj.side());
        }
        skinny_grad(dY, N, M, M, t.ext_b, r, 1.f, dB, 1, accumulate, t.part2, ctx.sm_count, fj.side());
    }
    // main: dH = s * dY . B^T from the bf16 dY; extension operand dH / s_dy[n] (the reduce waits for s_dy)
    cast_pad(B, M, 1, t.pdown, M, r, (int)M, (int)M, 1.f, st);
    skinny_down(dY, N, M, M, t.pdown, M, r, s, t.dHf, t.ext_a, 1.f, t.part, ctx.sm_count, st, dX ? t.srow : nullptr,
                dX ? &fj : nullptr);
    if (dX) {
        fj.wait(0);
        Operand a0{t.q8, false, M}, b0{wt, false, M};
        Operand a1{t.ext_a, false, EXT}, b1{t.pext, false, EXT};
        main_gemm_f8(a0, b0, M, &a1, &b1, EXT, (__nv_bfloat16*)dX, K, N, K, nullptr, sc, ctx.sm_count, st, t.tail);
    }
    if (dA) {  // dA = X^T . dH with the plain bf16 dH
        const __nv_bfloat16* dh_plain = t.ext_a;
        if (dX) {
            cast_pad(t.dHf, r, 1, t.ext_c, EXT, N, r, EXT, 1.f, st);
            dh_plain = t.ext_c;
        }
        skinny_grad(X, N, K, K, dh_plain, r, 1.f, dA, 0, accumulate, t.part, ctx.sm_count, st);
    }
    fj.join(1);
}

// ---- self-test of the bounded wait ----------------------------------------------------------
// One warp waits on an mbarrier that nothing ever arrives on, with the same wait routine the GEMM
// kernels use but a caller-chosen limit.  The wait gives up after the limit, records `code` in the
// per-device error word and the kernel returns normally: the context stays usable and the host
// sees LQ_ERR_TIMEOUT from lq_check_device_status.  Nothing here faults, traps or spins unbounded.
namespace {
__global__ void selftest_wait_kernel(int* status, unsigned long long limit_ns, int code) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        abort_flag = 0;
        fence_barrier_init();
    }
    __syncthreads();
    mbar_wait_ns(smem_u32(&bar), 0, &abort_flag, status, code, limit_ns);
}
}  // namespace

void lq_tc_selftest_wait(int device, unsigned limit_ms, cudaStream_t st) {
    DevCtx& ctx = dev_ctx(device);
    selftest_wait_kernel<<<1, 32, 0, st>>>(ctx.status, (unsigned long long)limit_ms * 1000000ull, 90);
    LQ_CUDA(cudaGetLastError());
}

void lq_tc_gemm_bf16(const void* A, int a_mn, int64_t lda, const void* B, int b_mn, int64_t ldb, void* Cout,
                     int c_dtype, int64_t ldc, int64_t Mg, int64_t Ng, int64_t Kg, int block_n, int splits,
                     float* partial_ws, const float* bias, cudaStream_t st) {
    Operand a{A, a_mn != 0, lda}, b{B, b_mn != 0, ldb};
    LQ_CHECK_ARG(Ng % 8 == 0 && ldc % 8 == 0, "gemm: Ng and ldc must be multiples of 8");
    LQ_CHECK_ARG(((uintptr_t)bias & 15) == 0, "gemm: bias must be 16-byte aligned");
    if (splits > 1) {
        LQ_CHECK_ARG(c_dtype == LQ_F32 && partial_ws != nullptr && block_n == 64, "split gemm: f32 out, block_n 64");
        // an empty k-range would publish an accumulator no MMA ever wrote
        LQ_CHECK_ARG(splits <= (Kg + BK - 1) / BK, "split gemm: splits must not exceed ceil(Kg / 64)");
        int64_t ldp = ((Ng + 63) / 64) * 64;
        if (a_mn && b_mn)
            launch_gemm<64, true, true, float>(a, b, Kg, nullptr, nullptr, 0, partial_ws, ldp, Mg * ldp, Mg, Ng, splits, nullptr, st);
        else if (!a_mn && !b_mn)
            launch_gemm<64, false, false, float>(a, b, Kg, nullptr, nullptr, 0, partial_ws, ldp, Mg * ldp, Mg, Ng, splits, nullptr, st);
        else
            throw LqError(LQ_ERR_UNSUPPORTED, "split gemm: mixed operand majors are not built");
        long long total = (long long)Mg * ldp;
        LqProf prof(LQ_K_REDUCE, st);
        reduce_partials_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(partial_ws, Mg * ldp, splits, ldp, Mg, (int)Ng,
                                                                              (int)ldp, 1.f, (float*)Cout, ldc, 0, 0, nullptr, 0, 0.f);
        LQ_CUDA(cudaGetLastError());
        return;
    }
#define LQ_GEMM_CASE(BN, AMN, BMN)                                                                                  \
    if (block_n == BN && (a_mn != 0) == AMN && (b_mn != 0) == BMN) {                                                \
        if (c_dtype == LQ_F32)                                                                                      \
            launch_gemm<BN, AMN, BMN, float>(a, b, Kg, nullptr, nullptr, 0, (float*)Cout, ldc, 0, Mg, Ng, 1, bias, st); \
        else                                                                                                        \
            launch_gemm<BN, AMN, BMN, __nv_bfloat16>(a, b, Kg, nullptr, nullptr, 0, (__nv_bfloat16*)Cout, ldc, 0, Mg, Ng, 1, bias, st); \
        return;                                                                                                     \
    }
    LQ_GEMM_CASE(256, false, false)
    LQ_GEMM_CASE(192, false, false)
    LQ_GEMM_CASE(128, false, false)
    LQ_GEMM_CASE(64, false, false)
    LQ_GEMM_CASE(64, true, true)
    LQ_GEMM_CASE(128, false, true)
    LQ_GEMM_CASE(128, true, false)
#undef LQ_GEMM_CASE
    throw LqError(LQ_ERR_UNSUPPORTED, "gemm: this (block_n, operand major) combination is not built");
}

// =========================================================================================
// Split contraction for callers that must not allocate device memory
// =========================================================================================
//
// Some hosts of this library cannot call cudaMalloc at the point where they need a split-K
// contraction: code running while a CUDA graph is being captured on the stream, code inside
// a framework allocator's callback, or a real-time loop whose memory was fixed at start-up.
// For them the partial tiles of the split live in a fixed array inside the library image
// instead of in a caller workspace.  The array exists once per GPU that loads the library,
// for the life of the process, and is shared by every call: two calls that can overlap on the
// GPU (different streams) would overwrite each other's partials.
namespace {

constexpr size_t kStaticPartialFloats = size_t(4) << 20;  // 16 MiB of f32 partials per GPU
static __device__ __align__(256) float g_static_partials[kStaticPartialFloats];
static __device__ int g_static_status;  // wait-gave-up code of the current call, 0 = fine
static __device__ int g_static_sticky;  // first such code since the host last looked (lq_check_device_status)

// Second stage for the static array: device code names the array directly.  Sums the splits
// in a fixed order; if the first stage recorded a timed-out wait, the output is NaN instead.
__global__ void __launch_bounds__(256) reduce_static_kernel(long long split_stride, int splits, long long ldp,
                                                            long long I, int J, float* __restrict__ out,
                                                            long long ldo) {
    long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= I * J) return;
    long long i = idx / J;
    int j = (int)(idx - i * J);
    float v = 0.f;
    for (int z = 0; z < splits; ++z) v += g_static_partials[z * split_stride + i * ldp + j];
    if (g_static_status != 0) {
        v = __int_as_float(0x7FC00000);
        if (idx == 0) atomicCAS(&g_static_sticky, 0, g_static_status);  // survives the next call's reset
    }
    out[i * ldo + j] = v;
}

struct StaticCtx {
    float* partials = nullptr;  // device address of g_static_partials on this device
    int* status = nullptr;      // device address of g_static_status on this device
    int* sticky = nullptr;      // device address of g_static_sticky on this device
    int sm_count = 0;
    bool ready = false;
};

// One-time set-up per device, with that device current.  In host code the array's name is
// only a handle; cudaGetSymbolAddress turns it into the pointer a kernel can be given.
std::mutex g_static_mu;
StaticCtx g_static_ctx[kMaxDevices];  // fixed storage: a reference handed out stays valid

// Device address of the sticky error word if the static path was set up on `dev`, else NULL.
int* static_ctx_peek(int dev) {
    std::lock_guard<std::mutex> lk(g_static_mu);
    return g_static_ctx[dev].ready ? g_static_ctx[dev].sticky : nullptr;
}

StaticCtx& static_ctx(int dev) {
    if (dev < 0 || dev >= kMaxDevices) throw LqError(LQ_ERR_INVALID, "device index out of range");
    std::lock_guard<std::mutex> lk(g_static_mu);
    StaticCtx& c = g_static_ctx[dev];
    if (!c.ready) {
        int major = 0;
        LQ_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
        if (major != 10)
            throw LqError(LQ_ERR_UNSUPPORTED, "lq_gemm_bf16_splitk_static needs an sm_100 device (no fallback)");
        LQ_CUDA(cudaGetSymbolAddress((void**)&c.partials, g_static_partials));
        LQ_CUDA(cudaGetSymbolAddress((void**)&c.status, g_static_status));
        LQ_CUDA(cudaGetSymbolAddress((void**)&c.sticky, g_static_sticky));
        LQ_CUDA(cudaDeviceGetAttribute(&c.sm_count, cudaDevAttrMultiProcessorCount, dev));
        c.ready = true;
    }
    return c;
}

template <bool MN>
void launch_static_split(const void* A, int64_t lda, const void* B, int64_t ldb, int64_t Mg, int64_t Ng, int64_t Kg,
                         int splits, int64_t ldp, const StaticCtx& ctx, cudaStream_t st) {
    using C = Cfg<64>;
    CUtensorMap tA = MN ? make_map(A, Mg, Kg, lda, 64) : make_map(A, Kg, Mg, lda, BM);
    CUtensorMap tB = MN ? make_map(B, Ng, Kg, ldb, 64) : make_map(B, Kg, Ng, ldb, 64);
    GemmParams p;
    p.Mg = (int)Mg;
    p.Ng = (int)Ng;
    p.kb0 = (int)((Kg + BK - 1) / BK);
    p.kb1 = 0;
    p.m_tiles = (int)((Mg + BM - 1) / BM);
    p.n_tiles = (int)((Ng + 63) / 64);
    p.splits = splits;
    p.C = ctx.partials;
    p.ldc = ldp;
    p.split_stride = Mg * ldp;
    p.bias = nullptr;
    p.status = ctx.status;
    p.row_scale = nullptr;
    p.col_scale = nullptr;
    p.col_scale_bcast = 0;
    p.tma_store = 0;
    long long items = (long long)p.m_tiles * p.n_tiles * splits;
    int grid = (int)std::min<long long>(items, ctx.sm_count);
    auto kern = umma_gemm_kernel<64, MN, MN, float>;
    LQ_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::SMEM));
    LqProf prof(LQ_K_GEMM_DOWN, st);
    kern<<<grid, kThreads, C::SMEM, st>>>(tA, tB, tA, tB, tA, p);
    LQ_CUDA(cudaGetLastError());
}

}  // namespace

// Reads and clears the sticky error word of the static path on `device` (0 when that path was never
// set up there).  The caller has synchronised the stream.
int lq_static_read_sticky(int device) {
    if (device < 0 || device >= kMaxDevices) return 0;
    int* addr = nullptr;
    {
        int cur = -1;
        if (cudaGetDevice(&cur) != cudaSuccess || cur != device) return 0;  // set-up happens with the device current
        addr = static_ctx_peek(device);
    }
    if (!addr) return 0;
    int v = 0;
    LQ_CUDA(cudaMemcpy(&v, addr, sizeof(int), cudaMemcpyDeviceToHost));
    if (v != 0) LQ_CUDA(cudaMemset(addr, 0, sizeof(int)));
    return v;
}

extern "C" int lq_gemm_bf16_splitk_static(const void* A, const void* B, int operands_mn, int64_t lda, int64_t ldb,
                                          float* Cout, int64_t ldc, int64_t Mg, int64_t Ng, int64_t Kg, int splits,
                                          void* stream) {
    try {
        LQ_CHECK_ARG(A && B && Cout, "NULL operand");
        LQ_CHECK_ARG(Mg > 0 && Ng > 0 && Kg > 0, "gemm dims must be positive");
        LQ_CHECK_ARG(Ng % 8 == 0 && ldc >= Ng, "Ng must be a multiple of 8 and ldc >= Ng");
        if (operands_mn)
            LQ_CHECK_ARG(lda >= Mg && ldb >= Ng, "MN-major operands: lda >= Mg and ldb >= Ng (row strides of [Kg, rows])");
        else
            LQ_CHECK_ARG(lda >= Kg && ldb >= Kg, "K-major operands: lda >= Kg and ldb >= Kg (row strides of [rows, Kg])");
        const int64_t kb = (Kg + BK - 1) / BK;
        LQ_CHECK_ARG(splits >= 1 && splits <= 64 && splits <= kb, "splits must be in [1, min(64, ceil(Kg / 64))]");
        const int64_t ldp = ((Ng + 63) / 64) * 64;
        const unsigned long long need = (unsigned long long)splits * (unsigned long long)Mg * (unsigned long long)ldp;
        if (need > kStaticPartialFloats)
            throw LqError(LQ_ERR_WORKSPACE,
                          "lq_gemm_bf16_splitk_static: splits * Mg * roundup(Ng, 64) = " + std::to_string(need) +
                              " floats exceeds the built-in scratch of " + std::to_string(kStaticPartialFloats) +
                              " floats (16 MiB); use lq_gemm_bf16 with a caller workspace");
        int dev = 0;
        LQ_CUDA(cudaGetDevice(&dev));
        StaticCtx& ctx = static_ctx(dev);
        cudaStream_t st = (cudaStream_t)stream;
        // the error word must start at zero for this call; the partials need no clearing (every
        // element the second stage reads is written by the first)
        LQ_CUDA(cudaMemsetAsync(ctx.status, 0, sizeof(int), st));
        if (operands_mn)
            launch_static_split<true>(A, lda, B, ldb, Mg, Ng, Kg, splits, ldp, ctx, st);
        else
            launch_static_split<false>(A, lda, B, ldb, Mg, Ng, Kg, splits, ldp, ctx, st);
        const long long total = (long long)Mg * Ng;
        {
            LqProf prof(LQ_K_REDUCE, st);
            reduce_static_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(Mg * ldp, splits, ldp, Mg, (int)Ng,
                                                                                Cout, ldc);
            LQ_CUDA(cudaGetLastError());
        }
        lq_set_last_error("");
        return LQ_OK;
    } catch (const LqError& e) {
        lq_set_last_error(e.what());
        return e.status;
    } catch (const std::exception& e) {
        lq_set_last_error(std::string("internal error: ") + e.what());
        return LQ_ERR_INVALID;
    }
}
