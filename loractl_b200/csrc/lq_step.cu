// Step glue on the flat LoRA buffers: the non-finite gradient check and a fused multi-tensor
// AdamW, both HBM-bound single passes over one flat f32 buffer.
//
// Reference: crates/loractl-core/src/diffusion_trainer.rs:1703-1743 — per step the trainer sums
// |g| over every adapter gradient (one tiny kernel per tensor plus a host read-back), then either
// runs burn's AdamW per parameter or skips the update.  Here every adapter's A and B live in one
// flat parameter buffer with a parallel flat gradient buffer (the same buffer NCCL all-reduces),
// so the check is one kernel and the optimizer is one kernel; the skip decision is read by the
// optimizer kernel from device memory, so the step itself needs no host synchronisation.
//
// AdamW arithmetic (burn-optim 0.21's `AdamW`, decoupled decay; identical to torch.optim.AdamW):
//   p <- p - lr * wd * p
//   m <- b1 m + (1 - b1) g          v <- b2 v + (1 - b2) g^2
//   p <- p - lr * (m / (1 - b1^t)) / (sqrt(v / (1 - b2^t)) + eps)
#include "lq_internal.cuh"
#include "lq_prof.cuh"

namespace {

__global__ void __launch_bounds__(256) nonfinite_kernel(const float* __restrict__ g, int64_t n, int* __restrict__ flag) {
    int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    int64_t stride = (int64_t)gridDim.x * blockDim.x * 4;
    bool bad = false;
    for (; i + 3 < n; i += stride) {
        float4 v = *(const float4*)(g + i);
        // |x| <= FLT_MAX is false for NaN and Inf
        bad |= !(fabsf(v.x) <= 3.402823466e38f) | !(fabsf(v.y) <= 3.402823466e38f) |
               !(fabsf(v.z) <= 3.402823466e38f) | !(fabsf(v.w) <= 3.402823466e38f);
    }
    for (; i < n; ++i) bad |= !(fabsf(g[i]) <= 3.402823466e38f);  // tail (only one thread reaches it)
    if (__any_sync(0xffffffffu, bad) && (threadIdx.x & 31) == 0) atomicOr(flag, 1);
}

__global__ void __launch_bounds__(256) adamw_kernel(float* __restrict__ p, const float* __restrict__ g,
                                                    float* __restrict__ m, float* __restrict__ v, int64_t n, float lr,
                                                    float b1, float b2, float eps, float wd, float bc1, float bc2,
                                                    float grad_scale, const int* __restrict__ skip_flag) {
    if (skip_flag && *skip_flag != 0) return;  // non-finite gradients somewhere: skip the whole update
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) {
        float gi = g[i] * grad_scale;
        float pi = p[i];
        pi = pi - (lr * wd) * pi;
        float mi = b1 * m[i] + (1.f - b1) * gi;
        float vi = b2 * v[i] + (1.f - b2) * gi * gi;
        m[i] = mi;
        v[i] = vi;
        float update = (mi / bc1) / (sqrtf(vi / bc2) + eps);
        p[i] = pi - lr * update;
    }
}

}  // namespace

extern "C" {

/* crates/loractl-core/src/diffusion_trainer.rs:1708-1725: are all adapter gradients finite?
 * Clears `flag` (device int) and sets it to 1 if any of the n floats is NaN or Inf. */
int lq_grad_nonfinite_flag(const float* grads, int64_t n, int* flag, void* stream) {
    try {
        LQ_CHECK_ARG(flag != nullptr && (n == 0 || grads != nullptr), "NULL argument");
        LQ_CHECK_ARG(((uintptr_t)grads & 15) == 0, "gradient buffer must be 16-byte aligned");
        cudaStream_t st = (cudaStream_t)stream;
        LQ_CUDA(cudaMemsetAsync(flag, 0, sizeof(int), st));
        if (n > 0) {
            int64_t blocks = (n / 4 + 255) / 256;
            if (blocks > 148 * 8) blocks = 148 * 8;
            if (blocks < 1) blocks = 1;
            LqProf prof(LQ_K_PREP, st);
            nonfinite_kernel<<<(unsigned)blocks, 256, 0, st>>>(grads, n, flag);
            LQ_CUDA(cudaGetLastError());
        }
        lq_set_last_error("");
        return LQ_OK;
    } catch (const LqError& e) {
        lq_set_last_error(e.what());
        return e.status;
    }
}

/* crates/loractl-core/src/diffusion_trainer.rs:1564-1566,1727-1728: AdamW over every adapter
 * parameter, as ONE pass over the flat buffers.  `step` is the 1-based update count (bias
 * correction); `grad_scale` multiplies the gradients first (1/world for the data-parallel mean);
 * `skip_flag` (device int, may be NULL) non-zero turns the whole call into a no-op — the skip
 * branch of the dynamic loss scale, decided on the device. */
int lq_adamw_step(float* params, const float* grads, float* exp_avg, float* exp_avg_sq, int64_t n, float lr,
                  float beta1, float beta2, float eps, float weight_decay, int64_t step, float grad_scale,
                  const int* skip_flag, void* stream) {
    try {
        LQ_CHECK_ARG(n >= 0 && (n == 0 || (params && grads && exp_avg && exp_avg_sq)), "NULL argument");
        LQ_CHECK_ARG(step >= 1, "step is the 1-based update count");
        LQ_CHECK_ARG(beta1 >= 0.f && beta1 < 1.f && beta2 >= 0.f && beta2 < 1.f, "betas must be in [0, 1)");
        if (n > 0) {
            cudaStream_t st = (cudaStream_t)stream;
            const float bc1 = 1.f - powf(beta1, (float)step), bc2 = 1.f - powf(beta2, (float)step);
            int64_t blocks = (n + 255) / 256;
            if (blocks > 148 * 8) blocks = 148 * 8;
            LqProf prof(LQ_K_PREP, st);
            adamw_kernel<<<(unsigned)blocks, 256, 0, st>>>(params, grads, exp_avg, exp_avg_sq, n, lr, beta1, beta2,
                                                          eps, weight_decay, bc1, bc2, grad_scale, skip_flag);
            LQ_CUDA(cudaGetLastError());
        }
        lq_set_last_error("");
        return LQ_OK;
    } catch (const LqError& e) {
        lq_set_last_error(e.what());
        return e.status;
    }
}

}  // extern "C"
