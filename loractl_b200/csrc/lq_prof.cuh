// Launch accounting and optional per-kernel-class CUDA-event timing.
//
// Every kernel launch of the library goes through an LqProf scope: it bumps a process-wide
// launch counter and, while profiling is enabled, records a CUDA event pair on the launch
// stream so a benchmark can read the time each kernel class took inside its own timed region.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

enum LqKernelKind {
    LQ_K_QUANT = 0,   // quantize / pack / unpack / fp8 repack
    LQ_K_DEQUANT,     // packed weight -> bf16/f32 scratch
    LQ_K_PREP,        // small casts / paddings of the LoRA factors
    LQ_K_GEMM_MAIN,   // frozen GEMM (+ fused LoRA K extension)
    LQ_K_GEMM_DOWN,   // H = X.A, dH = s.dY.B^T
    LQ_K_GEMM_GRAD,   // dA = X^T.dH, dB = (sH)^T.dY
    LQ_K_REDUCE,      // fixed-order second stage of split contractions
    LQ_K_SIMT,        // f32 SIMT GEMM
    LQ_K_COUNT
};

void lq_prof_begin(int kind, cudaStream_t st);
void lq_prof_end(int kind, cudaStream_t st);

struct LqProf {
    int kind;
    cudaStream_t st;
    LqProf(int k, cudaStream_t s) : kind(k), st(s) { lq_prof_begin(kind, st); }
    ~LqProf() { lq_prof_end(kind, st); }
};
