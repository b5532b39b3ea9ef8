// Pieces shared by the tcgen05 GEMM translation units: tile constants, the kernel parameter block
// and the raster that maps a work item to its output tile.
#pragma once

#include <stdint.h>

namespace lqgemm {

constexpr int BM = 128;
constexpr int BK = 64;

struct GemmParams {
    int Mg = 0, Ng = 0;
    int kb0 = 0, kb1 = 0;
    int m_tiles = 0, n_tiles = 0, splits = 1;
    void* C = nullptr;
    long long ldc = 0, split_stride = 0;
    const float* bias = nullptr;
    int* status = nullptr;
    // optional epilogue scales: v = acc * row_scale[row] * col_scale[col] (NULL = 1); with
    // col_scale_bcast the single value col_scale[0] applies to every column
    const float* row_scale = nullptr;
    const float* col_scale = nullptr;
    int col_scale_bcast = 0;
    int tma_store = 0;  // bf16 output leaves through shared memory and TMA tensor stores (full 64-byte row pieces)
    int group_m = 0;    // m-tiles per raster group (0 = 16)
    // CTA-pair kernel: the tiles from `tail_first` on (a thin last round of the persistent grid) are cut
    // into `tail_splits` ranges of k-blocks, one work item each, so that the round fills the machine;
    // those items write f32 partial tiles to `tail_part` ([tile - tail_first][split][256][BLOCK_N]) and a
    // second launch sums them in a fixed order.  tail_splits <= 1: no tile is cut.
    int tail_first = 0, tail_splits = 1;
    float* tail_part = nullptr;
};

// Work item -> (tile, k-block range) with the last tiles cut along k.  `slot` >= 0 is the partial-tile
// slot a cut item writes, -1 for a whole tile.
__device__ __forceinline__ void pair_item(const GemmParams& p, int item, int kb_total, int& tile, int& kb_begin,
                                          int& kb_end, int& slot) {
    const int tiles = p.m_tiles * p.n_tiles;
    const int tail_first = p.tail_splits > 1 ? p.tail_first : tiles;
    if (item < tail_first) {
        tile = item;
        kb_begin = 0;
        kb_end = kb_total;
        slot = -1;
    } else {
        const int q = item - tail_first, z = q % p.tail_splits;
        tile = tail_first + q / p.tail_splits;
        kb_begin = (int)(((long long)kb_total * z) / p.tail_splits);
        kb_end = (int)(((long long)kb_total * (z + 1)) / p.tail_splits);
        slot = q;
    }
}
__device__ __forceinline__ int pair_num_items(const GemmParams& p) {
    const int tiles = p.m_tiles * p.n_tiles;
    return p.tail_splits > 1 ? p.tail_first + (tiles - p.tail_first) * p.tail_splits : tiles;
}

template <int BLOCK_N>
struct Cfg {
    static constexpr uint32_t A_BYTES = BM * BK * 2;
    static constexpr uint32_t B_BYTES = BLOCK_N * BK * 2;
    // 64-wide tiles belong to the memory-bound LoRA contractions that run BESIDE the dequantisation
    // pass: six stages (144 KB, ample for the HBM latency) leave room for four of that pass's blocks
    // per SM where eight stages left room for one
    static constexpr int STAGES = BLOCK_N == 64 ? 6 : (208 * 1024) / (A_BYTES + B_BYTES);
    // 2 accumulator stages; the allocation must be a power of two >= 32 columns
    static constexpr uint32_t TMEM_COLS = BLOCK_N * 2 <= 128 ? 128 : (BLOCK_N * 2 <= 256 ? 256 : 512);
    static constexpr uint32_t STAGE_OUT = 8 * 2048;  // per epilogue warp: 32 rows x 64 bytes of bf16 output
    static constexpr size_t SMEM = (size_t)STAGES * (A_BYTES + B_BYTES) + STAGE_OUT + 1024 /*align*/ + 256 /*barriers*/;
};

__device__ __forceinline__ void item_coords(const GemmParams& p, int item, int& m_tile, int& n_tile, int& z) {
    const int tiles = p.m_tiles * p.n_tiles;
    z = item / tiles;
    int t = item - z * tiles;
    const int GROUP = p.group_m > 0 ? p.group_m : 16;  // m-tiles per raster group: a band of A kept hot in L2
    int per_group = GROUP * p.n_tiles;
    int g = t / per_group;
    int first_m = g * GROUP;
    int gsize = min(GROUP, p.m_tiles - first_m);
    int r = t - g * per_group;
    m_tile = first_m + r % gsize;
    n_tile = r / gsize;
}


}  // namespace lqgemm
