// Tensor-core (tcgen05) path of the LoRA linear: host-side entry points.
#pragma once

#include <cuda.h>

#include "lq_internal.cuh"

// True when the bf16 tcgen05 path can run this (weight, N, rank): TMA needs 16-byte row
// strides, i.e. d_in % 8 == 0 and d_out % 8 == 0.
bool lq_tc_supported(const lq_weight* w, int64_t n_tokens, int rank);
size_t lq_tc_workspace_bytes(const lq_weight* w, int64_t n_tokens, int rank);

// `mirror` (may be NULL): the bf16 operand arrays of this site's LoRA factors, built by
// lq_tc_mirror_build; with it the calls cast nothing.
void lq_tc_fwd(const lq_weight* w, const void* X, int64_t N, const float* A, const float* B, int r, float s, void* Y,
               float* H_out, void* ws, size_t ws_bytes, cudaStream_t st, const void* mirror);
void lq_tc_bwd(const lq_weight* w, const void* dY, const void* X, const float* H, int64_t N, const float* A,
               const float* B, int r, float s, void* dX, float* dA, float* dB, int accumulate, void* ws,
               size_t ws_bytes, cudaStream_t st, const void* mirror);
size_t lq_tc_mirror_bytes(int64_t K, int64_t M, int r);
void lq_tc_mirror_build(const float* A, const float* B, int64_t K, int64_t M, int r, void* mirror, cudaStream_t st);
void lq_tc_mirror_build_batch(const lq_mirror_job* jobs, int n, cudaStream_t st);

// Plain bf16 GEMM entry used by tests and probes: C[Mg,Ng] = A . B^T with either operand
// K-major ([rows, Kg], Kg contiguous) or MN-major ([Kg, rows], rows contiguous).
void lq_tc_gemm_bf16(const void* A, int a_mn, int64_t lda, const void* B, int b_mn, int64_t ldb, void* C, int c_dtype,
                     int64_t ldc, int64_t Mg, int64_t Ng, int64_t Kg, int block_n, int splits, float* partial_ws,
                     const float* bias, cudaStream_t st);

// Per-device error word written by kernels whose bounded waits gave up.  Synchronises `st`.
int lq_tc_read_status(int device, cudaStream_t st);

// Launches a one-warp kernel whose bounded wait is certain to run out after `limit_ms` (wait site 90).
void lq_tc_selftest_wait(int device, unsigned limit_ms, cudaStream_t st);

// Shared with the fused small-batch kernel (lq_fused.cu).
// 2-D bf16 tensor map over [rows, inner] (ld elements between rows), box 64 x box_rows, 128-byte swizzle.
CUtensorMap lq_tc_make_map(const void* base, int64_t inner, int64_t rows, int64_t ld, int box_rows);
// Same for a byte matrix: box 128 bytes x box_rows, 128-byte swizzle.
CUtensorMap lq_tc_make_map_u8(const void* base, int64_t inner, int64_t rows, int64_t ld, int box_rows);
// bf16 output [rows, cols]: box 32 x 32, 64-byte swizzle, for the epilogues' TMA tensor stores.
CUtensorMap lq_tc_make_store_map(const void* base, int64_t cols, int64_t rows, int64_t ld);
// m-tiles per raster group of a CTA-pair GEMM (see the definition for the rule).
int lq_tc_pair_group_m(int sm_count, int block_n, int64_t Ng, int64_t K0, int b_elem_bytes, int n_tiles);
int* lq_tc_status_word(int device);
// Event fork / join with the per-(device, caller stream) side stream: `fork` returns the stream to
// enqueue independent work on (the caller's own stream when forking is switched off); `join` makes
// the caller's stream wait for everything enqueued there since.
cudaStream_t lq_tc_fork(int device, cudaStream_t st);
void lq_tc_join(int device, cudaStream_t st);
int lq_tc_sm_count(int device);

// Small-batch forward (int4 weights at N <= 64 tokens, scaled-fp8 weights at N <= 16): the packed
// weight is streamed from HBM exactly once and converted on chip (registers + mma.sync at N <= 16,
// shared memory + tcgen05.mma above).
bool lq_fused_supported(const lq_weight* w, int64_t n_tokens, int rank);
size_t lq_fused_workspace_bytes(const lq_weight* w, int64_t n_tokens, int rank);
void lq_fused_fwd(const lq_weight* w, const void* X, int64_t N, const float* A, const float* B, int r, float s,
                  void* Y, float* H_out, void* ws, size_t ws_bytes, cudaStream_t st);

// Small-batch backward (int4 block-64 weights at N <= 16 tokens): dX over the packed stream with the
// weights converted in registers, dH / dA / dB in the same two launches (lq_bwd_small.cu).
bool lq_small_bwd_supported(const lq_weight* w, int64_t n_tokens, int rank);
size_t lq_small_bwd_workspace_bytes(const lq_weight* w, int64_t n_tokens, int rank);
void lq_small_bwd(const lq_weight* w, const void* dY, const void* X, const float* H, int64_t N, const float* A,
                  const float* B, int r, float s, void* dX, float* dA, float* dB, int accumulate, void* ws,
                  size_t ws_bytes, cudaStream_t st);

// A group of sites that share X, as one launch of the <= 16-token stream kernel plus one finalize.
bool lq_fused_group_supported(const lq_group_site* sites, int n_sites, int64_t n_tokens);
size_t lq_fused_group_workspace_bytes(const lq_group_site* sites, int n_sites, int64_t n_tokens);
void lq_fused_fwd_grouped(const lq_group_site* sites, int n_sites, const void* X, int64_t N, void* ws, size_t ws_bytes,
                          cudaStream_t st);

// Native fp8 compute (scaled-fp8 weights only): e4m3 weights straight from HBM x per-token e4m3
// activations on tcgen05 kind::f8f6f4, scales applied in the epilogue, LoRA extension kept in bf16.
bool lq_w8a8_supported(const lq_weight* w, int64_t n_tokens, int rank);
size_t lq_w8a8_workspace_bytes(const lq_weight* w, int64_t n_tokens, int rank);
void lq_w8a8_prepare_backward(const lq_weight* w, cudaStream_t st);
void lq_w8a8_fwd(const lq_weight* w, const void* X, int64_t N, const float* A, const float* B, int r, float s, void* Y,
                 float* H_out, void* ws, size_t ws_bytes, cudaStream_t st);
void lq_w8a8_bwd(const lq_weight* w, const void* dY, const void* X, const float* H, int64_t N, const float* A,
                 const float* B, int r, float s, void* dX, float* dA, float* dB, int accumulate, void* ws,
                 size_t ws_bytes, cudaStream_t st);

// Frozen GEMM with the int4 weight dequantised inside the mainloop (lq_w4.cu): no bf16 copy of the
// weight exists in HBM.  `transposed` = 0: C[Mg, d_out] = A0[Mg, d_in] . W^T (+ bias); 1: C[Mg, d_in] =
// A0[Mg, d_out] . W.  (a1, b1): optional bf16 K extension [Mg, K1] / [Ng, K1] (the LoRA product).
bool lq_w4_supported(const lq_weight* w, int64_t Mg, int transposed);
bool lq_w4_option_set(const char* name, int value);  // "w4", "w4_exact"; false: unknown name
bool lq_tc_option_set(const char* name, int value);  // "bwd_mn", "tail_split", "reserve_sms"; false: unknown name
void lq_w4_gemm(const lq_weight* w, int transposed, const void* A0, int64_t lda, const void* a1, int64_t lda1,
                const void* b1, int64_t ldb1, int64_t K1, void* Cout, int64_t ldc, int64_t Mg, const float* bias,
                cudaStream_t st);
