// The frozen GEMM with the int4 weight dequantised INSIDE the mainloop, on CTA pairs.
//
//   forward   C[Mg, d_out] = A0[Mg, d_in]  . dequant(W)^T (+ bias)     (Y = X . W^T)
//   backward  C[Mg, d_in]  = A0[Mg, d_out] . dequant(W)                (dX = dY . W)
//
// Nothing bf16-sized is ever written to HBM for the weight: the packed 4-bit tiles (0.5 byte per
// element plus the group scales) are the only weight traffic, where the reference writes and
// re-reads a full f32 copy per call (crates/loractl-core/src/quant.rs:232-233,250-251).
//
// Two CTAs of a cluster (an SM pair) share one 256 x 256 output tile exactly as in the bf16 pair
// kernel: each CTA holds 128 rows of the A operand and HALF of the B operand tile, one thread of the
// even CTA issues tcgen05.mma.cta_group::2 with M = 256, and each CTA's TMEM receives its own 128
// accumulator rows.  What differs is where the B half comes from:
//
//   warp 0       producer: TMA tile of A (cp.async.bulk.tensor, no multicast), and the plain bf16
//                B tiles of the LoRA extension blocks
//   warps 10-17  dequant, as four groups of two warps; group g owns k-blocks g, g+4, ...: it loads
//                this CTA's packed words and group scales for its next block from global memory
//                straight into registers (one block ahead of the stage it is waiting for), then
//                writes bf16 in the 128-byte-swizzled operand layout the MMA descriptor expects
//                (generic-proxy stores, fence.proxy.async, one arrival per warp on the leader CTA's
//                barrier)
//   warp 1       MMA issuer (leader CTA): waits for both CTAs' A bytes and both CTAs' dequantised
//                halves, issues four 256 x 256 x 16 MMAs, commits the stage back to both CTAs
//   warps 2-9    epilogue: TMEM -> registers -> bias -> bf16 -> swizzled staging -> TMA stores
//
// One packed tile is [128 weight rows][64 d_in] (row-major, 8 words of 8 nibbles per row).  Dequantised
// it is a row-major [128][64] bf16 image with 128-byte rows.  For the forward that image is a K-major
// B operand (rows = output columns).  For the backward the SAME image layout serves as an MN-major B
// operand: a k-block of 64 reduction rows (d_out) against this CTA's 128 output columns (d_in) is the
// upper or lower 64 rows of two adjacent packed tiles, each becoming one 64-column MN-major chunk
// [64 reduction rows][64 columns].  The conversion code is therefore the same for both directions;
// only the loads' source addresses and the MMA descriptors differ.
//
// Conversion: `(word >> 4j) & 0x000F000F | 0x43004300` is the bf16 pair (128 + u, 128 + u') of two
// adjacent elements (u = q + 8, nibble order chosen at pack time).  MODE 1 reproduces
// bf16(q * scale) with the f32 product of the scratch-copy path bit for bit; MODE 0 uses two packed
// bf16 instructions per pair, w = bf16(q * bf16(scale)) (q exact, the scale rounded once, relative
// 2^-9 — the same rule as the 17..64-token kernel); MODE 2 splits the scale into bf16 hi + lo and
// computes fma(q, s_hi, q * s_lo), which rounds q * scale once except next to a rounding boundary.
//
// The LoRA product rides along as extra k-blocks ("K extension") whose operands are plain bf16
// tiles loaded by TMA into the same stage buffers; the dequant warps pass those blocks through.
// Every wait is bounded; a wait that gives up records a code in the per-device error word.
#include <algorithm>
#include <atomic>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "lq_gemm.cuh"
#include "lq_prof.cuh"
#include "lq_tc.cuh"
#include "lq_umma.cuh"

namespace {

using namespace umma;
using namespace lqgemm;

constexpr int kGroupWarps = 2;   // warps per dequant group (four per group measured slower: 0.29 vs 0.26 ms)
constexpr int kGroupThreads = 32 * kGroupWarps;
constexpr int kChunks = 256 / kGroupThreads;  // 16-byte packed chunks per thread and k-block
// producer warp, MMA warp, 8 epilogue warps, 4 dequant groups
constexpr int kW4Threads = 64 + 256 + 4 * kGroupThreads;
constexpr int BN = 256;          // columns of the pair tile; each CTA converts 128 of them
constexpr int kGroups = 4;       // dequant groups (2 warps each) working on consecutive k-blocks

// One ring: an operand stage holds this CTA's A tile and its dequantised B half.  The packed weight
// bytes never pass through shared memory: the dequant threads load them from global memory straight
// into registers, one block ahead (the operand reads of the tensor core, the A tiles' arrival and the
// stores of the converted half already take most of the shared-memory bandwidth of a k-block time;
// staging the packed bytes there too measured 0.27 ms against 0.22 ms for the same GEMM over a bf16
// weight copy).  Four groups of two warps convert four consecutive k-blocks at once.
struct W4Cfg {
    static constexpr uint32_t A_BYTES = BM * BK * 2;        // 16 KB: this CTA's 128 rows of A
    static constexpr uint32_t B_BYTES = (BN / 2) * BK * 2;  // 16 KB: this CTA's dequantised half of B
    static constexpr int STAGES = 6;
    static constexpr uint32_t TMEM_COLS = 512;  // two 256-column accumulator stages
    static constexpr uint32_t STAGE_OUT = 8 * 2048;
    static constexpr size_t SMEM = (size_t)STAGES * (A_BYTES + B_BYTES) + STAGE_OUT + 1024 + 512;
};
static_assert(W4Cfg::SMEM <= 232448, "shared memory budget of one CTA");

struct W4Params {
    GemmParams g;
    const uint8_t* packed;  // [m_tiles][k_tiles][4096]
    const float* scales;    // [m_tiles][n_groups][128]
    int w_m_tiles, w_k_tiles, n_groups, gpt;  // gpt: scale groups per 64 d_in (1 or 2)
};

// Address of the same shared-memory object in the cluster's CTA `rank`.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t saddr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
    return r;
}
// Arrival (release at CTA scope, the default) on a barrier anywhere in the cluster; `cluster_addr` is an
// address in the shared::cluster window.  The data the arrival publishes was written to this CTA's own
// shared memory and handed to the async proxy by fence.proxy.async before the arrival; a cluster-scope
// release here measured 0.60 ms against 0.37 ms per launch at 4608 x 3072 x 12288.
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// Bounded wait for roles that sit idle for most of a tile (the epilogue during the mainloop): sleeps
// between polls so that the polling does not take issue slots from the conversion warps.
template <int SLEEP_NS = 200>
__device__ __forceinline__ bool mbar_wait_idle(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status,
                                               int code) {
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = globaltimer_ns();
    for (uint32_t i = 1;; ++i) {
        __nanosleep(SLEEP_NS);
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 63u) == 0u) {
            if (*abort_flag) return false;
            if (globaltimer_ns() - t0 > LQ_WAIT_LIMIT_NS) {
                *abort_flag = 1;
                atomicCAS(status, 0, code);
                return false;
            }
        }
    }
}

// 16-byte read-only load that does not allocate in L1 (every packed byte is read once per output tile).
__device__ __forceinline__ uint4 ld_nc_v4(const uint4* ptr) {
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "l"(ptr));
    return r;
}

// Eight packed elements (one word) -> eight bf16 (one 16-byte chunk of an operand row).
//   MODE 1 (exact): bf16(q * scale) with the f32 product — bit-identical to the scratch-copy path;
//                   nine instructions per pair of weights.
//   MODE 2 (split): q is made an exact bf16 integer ((128 + u) - 136), the scale is split into two
//                   bf16 terms s = s_hi + s_lo, and w = fma(q, s_hi, bf16(q * s_lo)) rounds the sum
//                   once: the result differs from bf16(q * scale) only when q * scale lies within
//                   2^-18 (relative) of a rounding boundary; five instructions per pair.
//   MODE 0 (fast):  w = bf16(q * bf16(scale)), four instructions per pair (scale rounded once, 2^-9).
struct ScalePair {
    float f;
    __nv_bfloat162 hi, lo;
};
__device__ __forceinline__ ScalePair make_scale(float sc) {
    ScalePair s;
    s.f = sc;
    const __nv_bfloat16 h = __float2bfloat16_rn(sc);
    const __nv_bfloat16 l = __float2bfloat16_rn(sc - __bfloat162float(h));
    s.hi = __halves2bfloat162(h, h);
    s.lo = __halves2bfloat162(l, l);
    return s;
}
template <int MODE>
__device__ __forceinline__ uint4 convert_word(uint32_t w, const ScalePair& sp) {
    uint32_t o[4];
    if (MODE == 1) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            // 0x4B000000 | u is the f32 2^23 + u; minus (2^23 + 8) leaves q exactly; one f32 product,
            // one round-to-nearest-even conversion of the pair: bf16(q * scale)
            const float lo = __uint_as_float(((w >> (4 * j)) & 0xFu) | 0x4B000000u) - 8388616.f;
            const float hi = __uint_as_float(((w >> (4 * j + 16)) & 0xFu) | 0x4B000000u) - 8388616.f;
            const __nv_bfloat162 v = __floats2bfloat162_rn(lo * sp.f, hi * sp.f);
            o[j] = *(const uint32_t*)&v;
        }
    } else {
        const __nv_bfloat162 off = __float2bfloat162_rn(136.f);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            uint32_t t = ((w >> (4 * j)) & 0x000F000Fu) | 0x43004300u;  // (128 + u_lo, 128 + u_hi)
            const __nv_bfloat162 q = __hsub2(*(__nv_bfloat162*)&t, off);  // exact integers -8..7
            const __nv_bfloat162 v = MODE == 2 ? __hfma2(q, sp.hi, __hmul2(q, sp.lo)) : __hmul2(q, sp.hi);
            o[j] = *(const uint32_t*)&v;
        }
    }
    return make_uint4(o[0], o[1], o[2], o[3]);
}

// TRANS = false: forward (B tile rows are weight rows, K-major); true: backward (MN-major chunks).
template <bool TRANS, int MODE>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kW4Threads, 1)
w4_gemm2_kernel(const __grid_constant__ CUtensorMap tmA0, const __grid_constant__ CUtensorMap tmA1,
                const __grid_constant__ CUtensorMap tmB1, const __grid_constant__ CUtensorMap tmC, W4Params wp) {
    using C = W4Cfg;
    constexpr int STAGES = C::STAGES;
    const GemmParams& p = wp.g;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* smem_a = smem;
    uint8_t* smem_b = smem_a + (size_t)STAGES * C::A_BYTES;
    uint8_t* stage_out = smem_b + (size_t)STAGES * C::B_BYTES;  // 1024-aligned
    uint64_t* bars = (uint64_t*)(stage_out + C::STAGE_OUT);
    uint64_t* full = bars;                 // leader: A bytes (and extension B bytes) of both CTAs
    uint64_t* bfull = bars + STAGES;       // leader: 4 arrivals, the two warps of one dequant group in both CTAs
    uint64_t* empty = bars + 2 * STAGES;   // both: the leader's multicast commit
    uint64_t* tfull = bars + 3 * STAGES;
    uint64_t* tempty = tfull + 2;
    uint32_t* tmem_slot = (uint32_t*)(tempty + 2);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&full[s]), 1);
            mbar_init(smem_u32(&bfull[s]), 2 * kGroupWarps);
            mbar_init(smem_u32(&empty[s]), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(smem_u32(&tfull[a]), 1);
            mbar_init(smem_u32(&tempty[a]), 512);
        }
        *abort_flag = 0;
        fence_barrier_init();
        prefetch_tmap(&tmA0);
        prefetch_tmap(&tmA1);
        prefetch_tmap(&tmB1);
        prefetch_tmap(&tmC);
    }
    if (warp == 1) {
        tmem_alloc2(smem_u32(tmem_slot), C::TMEM_COLS);
        tmem_relinquish2();
    }
    tc_fence_before();
    cluster_sync_all();  // both CTAs' barriers are initialised before either signals the other's
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int kb_total = p.kb0 + p.kb1;
    const int num_items = p.m_tiles * p.n_tiles;  // 256-row pair tiles x 256-column tiles
    const int cid = (int)(blockIdx.x >> 1), ncl = (int)(gridDim.x >> 1);

    if (warp == 0) {
        if (lane == 0) {
            // ---------------- producer (both CTAs): the A tiles, and the K extension's B tiles ----------------
            // (the packed weight bytes are fetched by the dequant groups themselves: one thread issuing
            // every copy of a k-block could not keep up with the MMA, above all in the backward, where a
            // k-block takes up to seven copies)
            int s = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int item = cid; ok && item < num_items; item += ncl) {
                int m_tile, n_tile, z;
                item_coords(p, item, m_tile, n_tile, z);
                const int arow = m_tile * 256 + (int)rank * BM;
                for (int kb = 0; kb < kb_total; ++kb) {
                    if (!mbar_wait(smem_u32(&empty[s]), phase ^ 1u, abort_flag, p.status, 61)) { ok = false; break; }
                    const uint32_t bar = smem_u32(&full[s]);
                    const uint32_t sa = smem_u32(smem_a + (size_t)s * C::A_BYTES);
                    if (kb >= p.kb0) {
                        // K extension: both operands are bf16 tiles; nothing to convert
                        if (leader) mbar_expect_tx(bar, 2 * (C::A_BYTES + C::B_BYTES));
                        const int kc = (kb - p.kb0) * BK;
                        tma_load_2d_pair(sa, &tmA1, bar, kc, arow);
                        tma_load_2d_pair(smem_u32(smem_b + (size_t)s * C::B_BYTES), &tmB1, bar, kc,
                                         n_tile * BN + (int)rank * (BN / 2));
                    } else {
                        if (leader) mbar_expect_tx(bar, 2 * C::A_BYTES);
                        tma_load_2d_pair(sa, &tmA0, bar, kb * BK, arow);
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
            constexpr uint32_t idesc_main = make_idesc(1, 1, false, TRANS, 256, BN);
            constexpr uint32_t idesc_ext = make_idesc(1, 1, false, false, 256, BN);
            const uint32_t d_hi = desc_hi(1024);
            const uint32_t a_lo0 = desc_lo(smem_u32(smem_a), 16);
            const uint32_t b_lo0_main = desc_lo(smem_u32(smem_b), TRANS ? 8192 : 16);
            const uint32_t b_lo0_ext = desc_lo(smem_u32(smem_b), 16);
            int s = 0, acc = 0;
            uint32_t phase = 0, acc_phase = 0;
            bool ok = true;
            for (int item = cid; ok && item < num_items; item += ncl) {
                if (!mbar_wait(smem_u32(&tempty[acc]), acc_phase ^ 1u, abort_flag, p.status, 62)) { ok = false; break; }
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + (uint32_t)(acc * BN);
                for (int kb = 0; kb < kb_total; ++kb) {
                    if (!mbar_wait(smem_u32(&full[s]), phase, abort_flag, p.status, 63)) { ok = false; break; }
                    if (!mbar_wait(smem_u32(&bfull[s]), phase, abort_flag, p.status, 64)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_lo = a_lo0 + (uint32_t)s * (C::A_BYTES >> 4);
                    const bool ext = kb >= p.kb0;
                    if (ext || !TRANS) {
                        const uint32_t b_lo = b_lo0_ext + (uint32_t)s * (C::B_BYTES >> 4);
#pragma unroll
                        for (int k = 0; k < BK / 16; ++k)
                            mma2_f16(tmem_d, desc_join(a_lo + k * 2u, d_hi), desc_join(b_lo + k * 2u, d_hi),
                                     ext ? idesc_ext : idesc_main, (kb > 0 || k > 0) ? 1u : 0u);
                    } else {
                        const uint32_t b_lo = b_lo0_main + (uint32_t)s * (C::B_BYTES >> 4);
#pragma unroll
                        for (int k = 0; k < BK / 16; ++k)  // MN-major B: 16 reduction rows of 128 bytes per step
                            mma2_f16(tmem_d, desc_join(a_lo + k * 2u, d_hi), desc_join(b_lo + k * 128u, d_hi), idesc_main,
                                     (kb > 0 || k > 0) ? 1u : 0u);
                    }
                    mma2_commit_mc(smem_u32(&empty[s]), 3);  // frees the stage in both CTAs
                    if (++s == STAGES) { s = 0; phase ^= 1u; }
                }
                if (!ok) break;
                mma2_commit_mc(smem_u32(&tfull[acc]), 3);
                if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
            }
        }
    } else if (warp >= 10) {
        // ---------------- dequant (warps 10..17 of both CTAs): four groups of two warps ----------------
        // Group g converts the k-blocks whose running index is g modulo 4, so four consecutive k-blocks
        // are in conversion at once and a group's fixed costs (the barrier wait, the proxy fence, the
        // arrival) are paid once per 8192 weights.  A thread owns four 16-byte chunks of the block's
        // packed bytes (chunk c = gt + 64 i: operand row c >> 1, 32-element half c & 1) and their row
        // scales; it loads the NEXT block's chunks from global memory before converting the current one.
        const int grp = (warp - 10) / kGroupWarps;
        const int gt = (threadIdx.x - 320) % kGroupThreads;  // thread within the group
        const int half = gt & 1;
        const uint32_t bfull_leader = map_to_cta(smem_u32(&bfull[0]), 0);  // the leader's barriers (own, if leader)

        // Loads the chunks behind k-block `kb` of output-column tile `n_tile`; false when that block has
        // no packed bytes (K extension, or columns past the weight's extent: those are clipped by the store).
        auto fetch = [&](int n_tile, int kb, uint4 (&v)[kChunks], float (&sc)[kChunks]) -> bool {
            if (kb >= p.kb0) return false;
            if (!TRANS) {
                const int mt = n_tile * 2 + (int)rank;  // this CTA's 128 output columns = packed tile row block mt
                if (mt >= wp.w_m_tiles) return false;
                const uint4* tile = (const uint4*)(wp.packed + ((size_t)mt * wp.w_k_tiles + kb) * 4096);
                const float* scl = wp.scales + ((size_t)mt * wp.n_groups + (size_t)kb * wp.gpt + (wp.gpt == 2 ? half : 0)) * 128;
#pragma unroll
                for (int i = 0; i < kChunks; ++i) {
                    v[i] = ld_nc_v4(tile + gt + kGroupThreads * i);
                    sc[i] = __ldg(scl + (gt >> 1) + (kGroupThreads / 2) * i);
                }
                return true;
            }
            // backward: 64 reduction rows = the upper or lower half of packed m-tile kb / 2; this CTA's 128
            // output columns = the two k-tiles kt0, kt0 + 1 (chunks 0..127 and 128..255)
            const int mt = kb >> 1, hrow = (kb & 1) * 64;
            const int kt0 = n_tile * 4 + (int)rank * 2;
            if (kt0 >= wp.w_k_tiles) return false;
#pragma unroll
            for (int i = 0; i < kChunks; ++i) {
                const int ch = gt + kGroupThreads * i;  // chunk of the 256: k-tile ch >> 7, chunk ch & 127 of its half tile
                const int kt = min(kt0 + (ch >> 7), wp.w_k_tiles - 1);  // a missing second k-tile: its columns are clipped
                const uint4* tile = (const uint4*)(wp.packed + ((size_t)mt * wp.w_k_tiles + kt) * 4096 + hrow * 32);
                v[i] = ld_nc_v4(tile + (ch & 127));
                sc[i] = __ldg(wp.scales + ((size_t)mt * wp.n_groups + (size_t)kt * wp.gpt + (wp.gpt == 2 ? half : 0)) * 128 +
                              hrow + ((ch & 127) >> 1));
            }
            return true;
        };
        // position of the group's current block in this CTA's sequence of (item, k-block)
        auto advance = [&](int& item, int& kb, int by) {
            kb += by;
            while (item < num_items && kb >= kb_total) { kb -= kb_total; item += ncl; }
        };
        auto tile_of = [&](int item) {
            int m_tile, n_tile, z;
            item_coords(p, item, m_tile, n_tile, z);
            return n_tile;
        };
        int item = cid, kb = 0;
        advance(item, kb, grp);
        uint4 v[kChunks], vn[kChunks];
        float sc[kChunks], scn[kChunks];
        bool have = item < num_items && fetch(tile_of(item), kb, v, sc);
        uint32_t kbi = (uint32_t)grp;
        bool ok = true;
        while (ok && item < num_items) {
            const int s = (int)(kbi % STAGES);
            const uint32_t phase = (kbi / STAGES) & 1u;
            int item1 = item, kb1 = kb;
            advance(item1, kb1, kGroups);
            const bool have1 = item1 < num_items && fetch(tile_of(item1), kb1, vn, scn);  // in flight during the conversion
            if (!mbar_wait(smem_u32(&empty[s]), phase ^ 1u, abort_flag, p.status, 66)) { ok = false; break; }
            if (have) {
                uint8_t* bst = smem_b + (size_t)s * C::B_BYTES;
#pragma unroll
                for (int i = 0; i < kChunks; ++i) {
                    const int row = (gt >> 1) + (kGroupThreads / 2) * i;
                    const ScalePair sp = make_scale(sc[i]);
                    const uint32_t words[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
                    uint8_t* brow = bst + row * 128;
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const int chunk = (half * 4 + q) ^ (row & 7);  // 128-byte swizzle of the operand layout
                        *(uint4*)(brow + chunk * 16) = convert_word<MODE>(words[q], sp);
                    }
                }
                fence_proxy_async_smem();  // this lane's stores are visible to the tensor core's reads
            }
            __syncwarp();
            if (lane == 0) mbar_arrive_remote(bfull_leader + (uint32_t)s * 8u);
            item = item1;
            kb = kb1;
            have = have1;
#pragma unroll
            for (int i = 0; i < kChunks; ++i) {
                v[i] = vn[i];
                sc[i] = scn[i];
            }
            kbi += kGroups;
        }
    } else {
        // ---------------- epilogue (warps 2..9 of both CTAs, each its own 128 rows) ----------------
        const int quarter = warp & 3;
        const int chalf = (warp - 2) >> 2;
        int acc = 0;
        uint32_t acc_phase = 0;
        bool ok = true;
        for (int item = cid; ok && item < num_items; item += ncl) {
            int m_tile, n_tile, z;
            item_coords(p, item, m_tile, n_tile, z);
            if (!mbar_wait_idle(smem_u32(&tfull[acc]), acc_phase, abort_flag, p.status, 67)) { ok = false; break; }
            tc_fence_after();
            const int row0 = m_tile * 256 + (int)rank * BM + quarter * 32;
#pragma unroll 1
            for (int c = 0; c < BN / 64; ++c) {
                uint32_t r[32];
                const int cc = chalf * (BN / 2) + c * 32;
                tmem_ld_x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * BN + cc), r);
                tmem_ld_wait();
                const int col0 = n_tile * BN + cc;
                uint32_t wds[16];
#pragma unroll
                for (int j = 0; j < 32; j += 8) {
                    const int col = col0 + j;
                    float v[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) v[e] = __uint_as_float(r[j + e]);
                    if (p.bias && col < p.Ng) {
                        const float4 b0 = *(const float4*)(p.bias + col);
                        const float4 b1 = *(const float4*)(p.bias + col + 4);
                        const float bs[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
                        for (int e = 0; e < 8; ++e) v[e] += bs[e];
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
    cluster_sync_all();  // neither CTA leaves while the other may still signal it or read its operand half
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc2(tmem_base, C::TMEM_COLS);
    }
}

int env_int(const char* name, int dflt) {
    const char* e = getenv(name);
    return e ? atoi(e) : dflt;
}

// Run-time switches (initial values from the environment, changed through lq_option_set).
std::atomic<int> g_w4_on{env_int("LQ_W4", 0)};
std::atomic<int> g_w4_exact{env_int("LQ_W4_EXACT", 1)};

template <bool TRANS, int MODE>
void launch_w4(const lq_weight* w, const void* A0, int64_t lda, const void* a1, int64_t lda1, const void* b1,
               int64_t ldb1, int64_t K1, void* Cout, int64_t ldc, int64_t Mg, const float* bias, cudaStream_t st) {
    using C = W4Cfg;
    const int64_t Ng = TRANS ? w->K : w->M;   // output columns
    const int64_t Kr = TRANS ? w->M : w->K;   // reduction length
    const int sm_count = lq_tc_sm_count(w->device);
    CUtensorMap tA0 = lq_tc_make_map(A0, Kr, Mg, lda, BM);
    CUtensorMap tA1 = a1 ? lq_tc_make_map(a1, K1, Mg, lda1, BM) : tA0;
    CUtensorMap tB1 = b1 ? lq_tc_make_map(b1, K1, Ng, ldb1, BN / 2) : tA0;
    CUtensorMap tC = lq_tc_make_store_map(Cout, Ng, Mg, ldc);
    W4Params wp;
    GemmParams& p = wp.g;
    p.Mg = (int)Mg;
    p.Ng = (int)Ng;
    p.kb0 = (int)((Kr + BK - 1) / BK);
    p.kb1 = a1 ? (int)((K1 + BK - 1) / BK) : 0;
    p.m_tiles = (int)((Mg + 255) / 256);
    p.n_tiles = (int)((Ng + BN - 1) / BN);
    p.splits = 1;
    p.C = Cout;
    p.ldc = ldc;
    p.bias = bias;
    p.status = lq_tc_status_word(w->device);
    p.tma_store = 1;
    // the packed weight is a quarter of a bf16 B operand: it stays in L2 while bands of A stream through
    p.group_m = lq_tc_pair_group_m(sm_count, BN, Ng, Kr, 1, p.n_tiles);
    wp.packed = (const uint8_t*)w->packed;
    wp.scales = w->scales;
    wp.w_m_tiles = (int)w->m_tiles;
    wp.w_k_tiles = (int)w->k_tiles;
    wp.n_groups = (int)w->n_groups;
    wp.gpt = 64 / w->group;
    auto kern = w4_gemm2_kernel<TRANS, MODE>;
    LQ_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::SMEM));
    static std::mutex mu;
    static int pairs_by_dev[64] = {};
    int pairs;
    {
        std::lock_guard<std::mutex> lk(mu);
        if (pairs_by_dev[w->device] == 0) {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(sm_count & ~1);
            cfg.blockDim = dim3(kW4Threads);
            cfg.dynamicSmemBytes = C::SMEM;
            int n = 0;
            LQ_CUDA(cudaOccupancyMaxActiveClusters(&n, kern, &cfg));
            pairs_by_dev[w->device] = std::max(1, std::min(n, sm_count / 2));
        }
        pairs = pairs_by_dev[w->device];
    }
    const long long items = (long long)p.m_tiles * p.n_tiles;
    const int grid = 2 * (int)std::min<long long>(items, pairs);
    LqProf prof(LQ_K_GEMM_MAIN, st);
    kern<<<grid, kW4Threads, C::SMEM, st>>>(tA0, tA1, tB1, tC, wp);
    LQ_CUDA(cudaGetLastError());
}

}  // namespace

// "w4" = 0 (or LQ_W4=0 in the environment) switches the in-mainloop path off: the bf16 scratch copy
// is used instead.  "w4_exact" = 0 (LQ_W4_EXACT=0) selects the two-instruction conversion
// w = bf16(q * bf16(scale)).
bool lq_w4_option_set(const char* name, int value) {
    if (std::strcmp(name, "w4") == 0) { g_w4_on = value; return true; }
    if (std::strcmp(name, "w4_exact") == 0) { g_w4_exact = value; return true; }
    return false;
}

bool lq_w4_supported(const lq_weight* w, int64_t Mg, int transposed) {
    if (!g_w4_on.load()) return false;
    if (w->scheme != LQ_INT4) return false;
    if (w->K % 64 != 0 || w->M % 8 != 0) return false;   // whole packed k-tiles; 16-byte output rows
    if (w->device < 0 || w->device >= 64) return false;
    const int64_t Ng = transposed ? w->K : w->M;
    return Mg >= 128 && Ng > 192 && lq_tc_sm_count(w->device) >= 2;
}

void lq_w4_gemm(const lq_weight* w, int transposed, const void* A0, int64_t lda, const void* a1, int64_t lda1,
                const void* b1, int64_t ldb1, int64_t K1, void* Cout, int64_t ldc, int64_t Mg, const float* bias,
                cudaStream_t st) {
    const int mode = g_w4_exact.load();
#define LQ_W4_CASE(T, MD)                                                                     \
    if ((transposed != 0) == T && mode == MD) {                                               \
        launch_w4<T, MD>(w, A0, lda, a1, lda1, b1, ldb1, K1, Cout, ldc, Mg, bias, st);        \
        return;                                                                               \
    }
    LQ_W4_CASE(false, 0) LQ_W4_CASE(false, 1) LQ_W4_CASE(false, 2)
    LQ_W4_CASE(true, 0) LQ_W4_CASE(true, 1) LQ_W4_CASE(true, 2)
#undef LQ_W4_CASE
    throw LqError(LQ_ERR_INVALID, "w4_exact must be 0 (fast), 1 (exact) or 2 (split scale)");
}
