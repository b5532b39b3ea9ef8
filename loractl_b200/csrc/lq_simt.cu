// f32 SIMT GEMM with pluggable operand loaders: the full-precision (LQ_F32) path.
//
// The reference's quant path is f32 end to end (crates/loractl-core/src/
// diffusion_trainer.rs:395-401); this kernel keeps that arithmetic — f32 operands,
// f32 FMA accumulation, the frozen weight dequantized element-wise as `q * scale` on
// load — so results agree with the f32 oracle to summation-order rounding.  It also
// serves shapes the tensor-core path does not take (tiny or unaligned problems).
//
//   C[i,j] = alpha * sum_k A(i,k) * B(k,j) + (beta ? C[i,j] : 0) + bias[j]
#include "lq_internal.cuh"
#include "lq_prof.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, PAD = 4;

__device__ __forceinline__ float load_a(const LqSimtArgs& p, int64_t i, int64_t k) {
    int64_t off = i * p.sa_i + k * p.sa_k;
    return p.a_dtype == LQ_F32 ? ((const float*)p.A)[off] : __bfloat162float(((const __nv_bfloat16*)p.A)[off]);
}

__device__ __forceinline__ float load_b(const LqSimtArgs& p, int64_t k, int64_t j) {
    if (p.b_mode == 0) {
        int64_t off = k * p.sb_k + j * p.sb_j;
        return p.b_dtype == LQ_F32 ? ((const float*)p.Bp)[off] : __bfloat162float(((const __nv_bfloat16*)p.Bp)[off]);
    }
    if (p.b_mode == 1) return lq_dequant_elem(p.W, j, k);
    return lq_dequant_elem(p.W, k, j);
}

__global__ void __launch_bounds__(256) simt_gemm_kernel(LqSimtArgs p) {
    __shared__ __align__(16) float As[BK][BM + PAD];
    __shared__ __align__(16) float Bs[BK][BN + PAD];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int64_t i0 = (int64_t)blockIdx.y * BM, j0 = (int64_t)blockIdx.x * BN;

    // Pick the thread -> element mapping whose fastest index is the contiguous one.
    const bool a_k_fast = (p.sa_k == 1);
    const bool b_k_fast = (p.b_mode == 1) || (p.b_mode == 0 && p.sb_k == 1 && p.sb_j != 1);

    float acc[4][4] = {};
    for (int64_t k0 = 0; k0 < p.Kred; k0 += BK) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            int ii, kk;
            if (a_k_fast) { kk = tid & 15; ii = (tid >> 4) + 16 * q; }
            else          { ii = tid & 63; kk = (tid >> 6) + 4 * q; }
            int64_t i = i0 + ii, k = k0 + kk;
            As[kk][ii] = (i < p.I && k < p.Kred) ? load_a(p, i, k) : 0.f;
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            int jj, kk;
            if (b_k_fast) { kk = tid & 15; jj = (tid >> 4) + 16 * q; }
            else          { jj = tid & 63; kk = (tid >> 6) + 4 * q; }
            int64_t j = j0 + jj, k = k0 + kk;
            Bs[kk][jj] = (j < p.J && k < p.Kred) ? load_b(p, k, j) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float4 a4 = *(const float4*)&As[kk][ty * 4];
            float4 b4 = *(const float4*)&Bs[kk][tx * 4];
            float a[4] = {a4.x, a4.y, a4.z, a4.w}, b[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
            for (int x = 0; x < 4; ++x)
#pragma unroll
                for (int y = 0; y < 4; ++y) acc[x][y] = fmaf(a[x], b[y], acc[x][y]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int x = 0; x < 4; ++x) {
        int64_t i = i0 + ty * 4 + x;
        if (i >= p.I) continue;
#pragma unroll
        for (int y = 0; y < 4; ++y) {
            int64_t j = j0 + tx * 4 + y;
            if (j >= p.J) continue;
            float v = p.alpha * acc[x][y];
            int64_t off = i * p.ldc + j;
            if (p.beta) v += p.c_dtype == LQ_F32 ? ((float*)p.C)[off] : __bfloat162float(((__nv_bfloat16*)p.C)[off]);
            if (p.bias) v += p.bias[j];
            if (p.c_dtype == LQ_F32) ((float*)p.C)[off] = v;
            else ((__nv_bfloat16*)p.C)[off] = __float2bfloat16(v);
        }
    }
}

}  // namespace

void lq_launch_simt_gemm(const LqSimtArgs& a, cudaStream_t st) {
    if (a.I <= 0 || a.J <= 0) return;
    dim3 grid((unsigned)((a.J + BN - 1) / BN), (unsigned)((a.I + BM - 1) / BM));
    if (grid.y > 65535u) throw LqError(LQ_ERR_UNSUPPORTED, "simt gemm: more than 65535*64 rows");
    LqProf prof(LQ_K_SIMT, st);
    simt_gemm_kernel<<<grid, 256, 0, st>>>(a);
    LQ_CUDA(cudaGetLastError());
}
