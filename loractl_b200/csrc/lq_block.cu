// Element-wise companions of the LoRA'd linears inside a DiT block: the adaLN prologue
// y = norm(x) * (1 + scale) + shift and the gated residual out = x + gate * y, each as one pass
// forward and a two-stage, atomic-free backward.
//
// Reference: crates/loractl-core/src/mmdit.rs:857-869 — the block computes
// `(prescale + 1) * prenorm(x) + preshift`, `x + pregate * attn(..)`, `(postscale + 1) *
// postnorm(x) + postshift`, `x + postgate * mlp(..)` as separate broadcast multiplies and adds
// (and burn's autodiff adds a broadcast-sum per modulation tensor in the backward).  Here the
// modulation vectors are [samples, h] and broadcast over the tokens of a sample inside the kernel;
// the norm is a layer norm without affine parameters (eps inside the square root), statistics in
// f32.  The token-axis sums of the backward (d shift, d scale, d gate) are written as per-chunk
// partial rows and summed in a fixed order, so two runs are bit-identical.
#include <algorithm>

#include <cuda_bf16.h>

#include "lq_internal.cuh"
#include "lq_prof.cuh"

namespace {

constexpr int kChunkTokens = 64;  // tokens per partial row of the column reductions

__device__ __forceinline__ float to_f(float v) { return v; }
__device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}

// One warp per token row.  Three passes over the row (mean, centred variance, output); the row
// (h * sizeof(T) bytes) stays in L1 between them.
template <typename T>
__global__ void __launch_bounds__(256) ln_modulate_fwd_kernel(const T* __restrict__ x, const T* __restrict__ shift,
                                                              const T* __restrict__ scale, int64_t rows, int h,
                                                              int64_t tokens, float eps, T* __restrict__ y,
                                                              float* __restrict__ mean, float* __restrict__ rstd) {
    const int64_t row = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (row >= rows) return;
    const T* xr = x + row * h;
    const int64_t b = row / tokens;
    float s = 0.f;
    for (int j = lane; j < h; j += 32) s += to_f(xr[j]);
    const float mu = warp_sum(s) / (float)h;
    float v = 0.f;
    for (int j = lane; j < h; j += 32) {
        const float d = to_f(xr[j]) - mu;
        v = fmaf(d, d, v);
    }
    const float rs = rsqrtf(warp_sum(v) / (float)h + eps);
    const T* sh = shift + b * h;
    const T* sc = scale + b * h;
    T* yr = y + row * h;
    for (int j = lane; j < h; j += 32) {
        const float xh = (to_f(xr[j]) - mu) * rs;
        yr[j] = from_f<T>(fmaf(xh, 1.f + to_f(sc[j]), to_f(sh[j])));
    }
    if (lane == 0) {
        mean[row] = mu;
        rstd[row] = rs;
    }
}

// dx of the modulated layer norm, one warp per row:
//   g = dy * (1 + scale);  dx = rstd * (g - mean_h(g) - xhat * mean_h(g * xhat))
template <typename T>
__global__ void __launch_bounds__(256) ln_modulate_bwd_dx_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                                                                 const T* __restrict__ scale,
                                                                 const float* __restrict__ mean,
                                                                 const float* __restrict__ rstd, int64_t rows, int h,
                                                                 int64_t tokens, T* __restrict__ dx) {
    const int64_t row = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (row >= rows) return;
    const T* xr = x + row * h;
    const T* dyr = dy + row * h;
    const T* sc = scale + (row / tokens) * h;
    const float mu = mean[row], rs = rstd[row];
    float a = 0.f, c = 0.f;
    for (int j = lane; j < h; j += 32) {
        const float g = to_f(dyr[j]) * (1.f + to_f(sc[j]));
        const float xh = (to_f(xr[j]) - mu) * rs;
        a += g;
        c = fmaf(g, xh, c);
    }
    a = warp_sum(a) / (float)h;
    c = warp_sum(c) / (float)h;
    T* dxr = dx + row * h;
    for (int j = lane; j < h; j += 32) {
        const float g = to_f(dyr[j]) * (1.f + to_f(sc[j]));
        const float xh = (to_f(xr[j]) - mu) * rs;
        dxr[j] = from_f<T>(rs * (g - a - xh * c));
    }
}

// Column sums over the tokens of one chunk.  MODE 0: p0[j] = sum_t a[t,j] * b[t,j]   (d gate)
//                                           MODE 1: p0[j] = sum_t a[t,j] * xhat[t,j] (d scale),
//                                                   p1[j] = sum_t a[t,j]            (d shift)
// grid (ceil(h / 256), chunks per sample, samples); thread = one column.
template <typename T, int MODE>
__global__ void __launch_bounds__(256) col_partial_kernel(const T* __restrict__ a, const T* __restrict__ b,
                                                          const float* __restrict__ mean,
                                                          const float* __restrict__ rstd, int64_t tokens, int h,
                                                          int chunks, float* __restrict__ p0, float* __restrict__ p1) {
    const int j = blockIdx.x * 256 + threadIdx.x;
    if (j >= h) return;
    const int chunk = blockIdx.y;
    const int64_t sample = blockIdx.z;
    const int64_t t0 = (int64_t)chunk * kChunkTokens, t1 = min(tokens, t0 + kChunkTokens);
    float s0 = 0.f, s1 = 0.f;
    for (int64_t t = t0; t < t1; ++t) {
        const int64_t row = sample * tokens + t;
        const float av = to_f(a[row * h + j]);
        if (MODE == 0) {
            s0 = fmaf(av, to_f(b[row * h + j]), s0);
        } else {
            const float xh = (to_f(b[row * h + j]) - mean[row]) * rstd[row];
            s0 = fmaf(av, xh, s0);
            s1 += av;
        }
    }
    const int64_t o = (sample * chunks + chunk) * h + j;
    p0[o] = s0;
    if (MODE == 1) p1[o] = s1;
}

// out[sample, j] = sum over chunks (fixed order) of partial[sample, chunk, j]
__global__ void __launch_bounds__(256) col_final_kernel(const float* __restrict__ p, int chunks, int h, int64_t samples,
                                                        float* __restrict__ out) {
    const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= samples * h) return;
    const int64_t sample = i / h;
    const int j = (int)(i - sample * h);
    float s = 0.f;
    for (int c = 0; c < chunks; ++c) s += p[(sample * chunks + c) * h + j];
    out[i] = s;
}

// out = x + gate * y   (gate [samples, h] broadcast over tokens)
template <typename T>
__global__ void __launch_bounds__(256) gate_residual_kernel(const T* __restrict__ x, const T* __restrict__ gate,
                                                            const T* __restrict__ y, int64_t n, int h, int64_t per_sample,
                                                            T* __restrict__ out) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) {
        const int64_t sample = i / per_sample;
        const int j = (int)(i % h);
        const float xv = x ? to_f(x[i]) : 0.f;
        out[i] = from_f<T>(fmaf(to_f(gate[sample * h + j]), to_f(y[i]), xv));
    }
}

// ---- bf16 fast paths (h a multiple of 8, rows 16-byte aligned): 16-byte loads, the row held in
// registers between the passes of the norm ----------------------------------------------------
__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        f[2 * i] = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
    }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const __nv_bfloat162 p = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
        w[i] = *(const uint32_t*)&p;
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
}

// NV = 16-byte vectors per lane (h <= 256 * NV).
template <int NV>
__global__ void __launch_bounds__(256) ln_modulate_fwd_bf16_kernel(const __nv_bfloat16* __restrict__ x,
                                                                   const __nv_bfloat16* __restrict__ shift,
                                                                   const __nv_bfloat16* __restrict__ scale, int64_t rows,
                                                                   int h, int64_t tokens, float eps,
                                                                   __nv_bfloat16* __restrict__ y, float* __restrict__ mean,
                                                                   float* __restrict__ rstd) {
    const int64_t row = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (row >= rows) return;
    const int nvec = h >> 3;
    const uint4* xr = (const uint4*)(x + row * h);
    float v[NV][8];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = lane + 32 * i;
        if (c < nvec) {
            unpack8(xr[c], v[i]);
#pragma unroll
            for (int e = 0; e < 8; ++e) s += v[i][e];
        }
    }
    const float mu = warp_sum(s) / (float)h;
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i)
        if (lane + 32 * i < nvec) {
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const float d = v[i][e] - mu;
                q = fmaf(d, d, q);
            }
        }
    const float rs = rsqrtf(warp_sum(q) / (float)h + eps);
    const int64_t b = row / tokens;
    const uint4* sh = (const uint4*)(shift + b * h);
    const uint4* sc = (const uint4*)(scale + b * h);
    uint4* yr = (uint4*)(y + row * h);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = lane + 32 * i;
        if (c < nvec) {
            float a[8], g[8], o[8];
            unpack8(sh[c], a);
            unpack8(sc[c], g);
#pragma unroll
            for (int e = 0; e < 8; ++e) o[e] = fmaf((v[i][e] - mu) * rs, 1.f + g[e], a[e]);
            yr[c] = pack8(o);
        }
    }
    if (lane == 0) {
        mean[row] = mu;
        rstd[row] = rs;
    }
}

template <int NV>
__global__ void __launch_bounds__(256) ln_modulate_bwd_dx_bf16_kernel(const __nv_bfloat16* __restrict__ dy,
                                                                      const __nv_bfloat16* __restrict__ x,
                                                                      const __nv_bfloat16* __restrict__ scale,
                                                                      const float* __restrict__ mean,
                                                                      const float* __restrict__ rstd, int64_t rows, int h,
                                                                      int64_t tokens, __nv_bfloat16* __restrict__ dx) {
    const int64_t row = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (row >= rows) return;
    const int nvec = h >> 3;
    const uint4* xr = (const uint4*)(x + row * h);
    const uint4* dyr = (const uint4*)(dy + row * h);
    const uint4* sc = (const uint4*)(scale + (row / tokens) * h);
    const float mu = mean[row], rs = rstd[row];
    float g[NV][8], xh[NV][8];
    float a = 0.f, c2 = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = lane + 32 * i;
        if (c < nvec) {
            float s8[8];
            unpack8(dyr[c], g[i]);
            unpack8(xr[c], xh[i]);
            unpack8(sc[c], s8);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                g[i][e] *= 1.f + s8[e];
                xh[i][e] = (xh[i][e] - mu) * rs;
                a += g[i][e];
                c2 = fmaf(g[i][e], xh[i][e], c2);
            }
        }
    }
    a = warp_sum(a) / (float)h;
    c2 = warp_sum(c2) / (float)h;
    uint4* dxr = (uint4*)(dx + row * h);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = lane + 32 * i;
        if (c < nvec) {
            float o[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) o[e] = rs * (g[i][e] - a - xh[i][e] * c2);
            dxr[c] = pack8(o);
        }
    }
}

// Column sums, 4 columns per thread (8-byte loads); grid (ceil(h / 1024), chunks, samples).
template <int MODE>
__global__ void __launch_bounds__(256) col_partial_bf16_kernel(const __nv_bfloat16* __restrict__ a,
                                                               const __nv_bfloat16* __restrict__ b,
                                                               const float* __restrict__ mean,
                                                               const float* __restrict__ rstd, int64_t tokens, int h,
                                                               int chunks, float* __restrict__ p0, float* __restrict__ p1) {
    const int j = (blockIdx.x * 256 + threadIdx.x) * 4;
    if (j >= h) return;
    const int chunk = blockIdx.y;
    const int64_t sample = blockIdx.z;
    const int64_t t0 = (int64_t)chunk * kChunkTokens, t1 = min(tokens, t0 + kChunkTokens);
    float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
    for (int64_t t = t0; t < t1; ++t) {
        const int64_t row = sample * tokens + t;
        const uint2 ua = *(const uint2*)(a + row * h + j);
        const uint2 ub = *(const uint2*)(b + row * h + j);
        const float av[4] = {__uint_as_float(ua.x << 16), __uint_as_float(ua.x & 0xFFFF0000u),
                             __uint_as_float(ua.y << 16), __uint_as_float(ua.y & 0xFFFF0000u)};
        float bv[4] = {__uint_as_float(ub.x << 16), __uint_as_float(ub.x & 0xFFFF0000u),
                       __uint_as_float(ub.y << 16), __uint_as_float(ub.y & 0xFFFF0000u)};
        if (MODE == 1) {
            const float mu = mean[row], rs = rstd[row];
#pragma unroll
            for (int e = 0; e < 4; ++e) bv[e] = (bv[e] - mu) * rs;
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            s0[e] = fmaf(av[e], bv[e], s0[e]);
            if (MODE == 1) s1[e] += av[e];
        }
    }
    const int64_t o = (sample * chunks + chunk) * h + j;
    *(float4*)(p0 + o) = make_float4(s0[0], s0[1], s0[2], s0[3]);
    if (MODE == 1) *(float4*)(p1 + o) = make_float4(s1[0], s1[1], s1[2], s1[3]);
}

// out = x + gate * y, 8 elements per thread.
__global__ void __launch_bounds__(256) gate_residual_bf16_kernel(const __nv_bfloat16* __restrict__ x,
                                                                 const __nv_bfloat16* __restrict__ gate,
                                                                 const __nv_bfloat16* __restrict__ y, int64_t nvec, int h,
                                                                 int64_t per_sample, __nv_bfloat16* __restrict__ out) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (; i < nvec; i += stride) {
        const int64_t e0 = i * 8;
        const int64_t sample = e0 / per_sample;
        const int j = (int)(e0 % h);
        float gv[8], yv[8], xv[8], o[8];
        unpack8(*(const uint4*)(gate + sample * h + j), gv);
        unpack8(*(const uint4*)(y + e0), yv);
        if (x) unpack8(*(const uint4*)(x + e0), xv);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = fmaf(gv[e], yv[e], x ? xv[e] : 0.f);
        *(uint4*)(out + e0) = pack8(o);
    }
}

inline bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }

inline unsigned grid_for(int64_t n, int per_block, int64_t cap) {
    int64_t b = (n + per_block - 1) / per_block;
    if (b > cap) b = cap;
    if (b < 1) b = 1;
    return (unsigned)b;
}

int chunks_of(int64_t tokens) { return (int)((tokens + kChunkTokens - 1) / kChunkTokens); }

void check_common(const void* p0, const void* p1, int dtype, int64_t samples, int64_t tokens, int64_t h) {
    LQ_CHECK_ARG(p0 != nullptr && p1 != nullptr, "NULL argument");
    LQ_CHECK_ARG(dtype == LQ_F32 || dtype == LQ_BF16, "dtype must be LQ_F32 or LQ_BF16");
    LQ_CHECK_ARG(samples >= 1 && tokens >= 1 && h >= 1 && h <= (1 << 20), "samples, tokens and h must be positive");
}

template <typename F>
int guarded_call(F&& f) {
    try {
        f();
        lq_set_last_error("");
        return LQ_OK;
    } catch (const LqError& e) {
        lq_set_last_error(e.what());
        return e.status;
    }
}

// ---- activations between two linears of the reference's own block ------------------------------
// SwiGLU (crates/loractl-core/src/mmdit.rs:695-708): out = silu(gate) * up, and the attention output's
// sigmoid gate (mmdit.rs:659-664): out = x * sigmoid(g).  Both are plain element-wise maps of two
// tensors; one pass forward, one pass backward producing both input gradients; arithmetic in f32.
// MODE 0: out = silu(a) * b        d a = dout * b * sig(a) (1 + a (1 - sig(a))),  d b = dout * silu(a)
// MODE 1: out = a * sigmoid(b)     d a = dout * sig(b),                           d b = dout * a * sig(b) (1 - sig(b))
__device__ __forceinline__ float sigmoid_f(float v) { return 1.f / (1.f + expf(-v)); }

template <int MODE>
__device__ __forceinline__ float act_fwd(float a, float b) {
    return MODE == 0 ? a * sigmoid_f(a) * b : a * sigmoid_f(b);
}
template <int MODE>
__device__ __forceinline__ void act_bwd(float a, float b, float g, float& da, float& db) {
    if (MODE == 0) {
        const float sg = sigmoid_f(a);
        da = g * b * sg * (1.f + a * (1.f - sg));
        db = g * a * sg;
    } else {
        const float sg = sigmoid_f(b);
        da = g * sg;
        db = g * a * sg * (1.f - sg);
    }
}

// VEC elements per thread and step: 8 bf16 or 4 f32 (16-byte accesses); `n` need not be a multiple.
template <typename T, int MODE, bool BWD>
__global__ void __launch_bounds__(256) pair_act_kernel(const T* __restrict__ a, const T* __restrict__ b,
                                                       const T* __restrict__ dout, int64_t n, T* __restrict__ o0,
                                                       T* __restrict__ o1) {
    constexpr int VEC = 16 / (int)sizeof(T);
    const int64_t nv = n / VEC;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nv; i += (int64_t)gridDim.x * blockDim.x) {
        const uint4 va = ((const uint4*)a)[i], vb = ((const uint4*)b)[i];
        uint4 vg = make_uint4(0u, 0u, 0u, 0u);
        if (BWD) vg = ((const uint4*)dout)[i];
        const T* pa = (const T*)&va;
        const T* pb = (const T*)&vb;
        const T* pg = (const T*)&vg;
        uint4 r0, r1;
        T* q0 = (T*)&r0;
        T* q1 = (T*)&r1;
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
            if (BWD) {
                float da, db;
                act_bwd<MODE>(to_f(pa[e]), to_f(pb[e]), to_f(pg[e]), da, db);
                q0[e] = from_f<T>(da);
                q1[e] = from_f<T>(db);
            } else {
                q0[e] = from_f<T>(act_fwd<MODE>(to_f(pa[e]), to_f(pb[e])));
            }
        }
        ((uint4*)o0)[i] = r0;
        if (BWD) ((uint4*)o1)[i] = r1;
    }
    // ragged end (fewer than VEC elements), by the first threads of the grid
    const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t i = nv * VEC + t;
    if (i < n) {
        if (BWD) {
            float da, db;
            act_bwd<MODE>(to_f(a[i]), to_f(b[i]), to_f(dout[i]), da, db);
            o0[i] = from_f<T>(da);
            o1[i] = from_f<T>(db);
        } else {
            o0[i] = from_f<T>(act_fwd<MODE>(to_f(a[i]), to_f(b[i])));
        }
    }
}

// ---- ZRmsNorm (crates/loractl-core/src/mmdit.rs:282-330) -------------------------------------------
// y = x / sqrt(mean(x^2) + eps) * (scale + 1) over the last axis, zero-initialised frozen `scale`;
// one warp per row, statistics in f32.  Backward for x only (the scale belongs to the frozen base):
//   g = dy * (scale + 1),  dx = r * (g - x * r^2 * mean(g * x)),  r = rstd of the row.
template <typename T>
__global__ void __launch_bounds__(256) zrmsnorm_fwd_kernel(const T* __restrict__ x, const float* __restrict__ scale,
                                                           int64_t rows, int h, float eps, T* __restrict__ y,
                                                           float* __restrict__ rstd) {
    const int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= rows) return;
    const T* xr = x + row * h;
    float ss = 0.f;
    for (int i = lane; i < h; i += 32) {
        const float v = to_f(xr[i]);
        ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    const float r = 1.f / sqrtf(ss / (float)h + eps);
    if (lane == 0 && rstd) rstd[row] = r;
    T* yr = y + row * h;
    for (int i = lane; i < h; i += 32) yr[i] = from_f<T>(to_f(xr[i]) * r * (scale[i] + 1.f));
}

template <typename T>
__global__ void __launch_bounds__(256) zrmsnorm_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                                                           const float* __restrict__ scale,
                                                           const float* __restrict__ rstd, int64_t rows, int h,
                                                           T* __restrict__ dx) {
    const int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= rows) return;
    const T* xr = x + row * h;
    const T* gr = dy + row * h;
    const float r = rstd[row];
    float dot = 0.f;
    for (int i = lane; i < h; i += 32) dot = fmaf(to_f(gr[i]) * (scale[i] + 1.f), to_f(xr[i]), dot);
    dot = warp_sum(dot) / (float)h;
    T* dr = dx + row * h;
    for (int i = lane; i < h; i += 32) {
        const float g = to_f(gr[i]) * (scale[i] + 1.f);
        dr[i] = from_f<T>(r * (g - to_f(xr[i]) * r * r * dot));
    }
}

}  // namespace

extern "C" {

size_t lq_block_ops_workspace_bytes(int64_t samples, int64_t tokens, int64_t h) {
    if (samples < 1 || tokens < 1 || h < 1) return 0;
    return (size_t)2 * (size_t)samples * (size_t)chunks_of(tokens) * (size_t)h * sizeof(float);
}

int lq_ln_modulate_fwd(const void* x, const void* shift, const void* scale, int dtype, int64_t samples, int64_t tokens,
                       int64_t h, float eps, void* y, float* mean, float* rstd, void* stream) {
    return guarded_call([&] {
        check_common(x, y, dtype, samples, tokens, h);
        LQ_CHECK_ARG(shift && scale && mean && rstd, "NULL argument");
        cudaStream_t st = (cudaStream_t)stream;
        const int64_t rows = samples * tokens;
        LqProf prof(LQ_K_PREP, st);
        const unsigned grid = (unsigned)((rows + 7) / 8);
        if (dtype == LQ_F32)
            ln_modulate_fwd_kernel<float><<<grid, 256, 0, st>>>((const float*)x, (const float*)shift, (const float*)scale,
                                                                rows, (int)h, tokens, eps, (float*)y, mean, rstd);
        else if (h % 8 == 0 && h <= 4096 && aligned16(x) && aligned16(y) && aligned16(shift) && aligned16(scale)) {
            const __nv_bfloat16 *xb = (const __nv_bfloat16*)x, *shb = (const __nv_bfloat16*)shift, *scb = (const __nv_bfloat16*)scale;
            __nv_bfloat16* yb = (__nv_bfloat16*)y;
            if (h <= 1024) ln_modulate_fwd_bf16_kernel<4><<<grid, 256, 0, st>>>(xb, shb, scb, rows, (int)h, tokens, eps, yb, mean, rstd);
            else if (h <= 2048) ln_modulate_fwd_bf16_kernel<8><<<grid, 256, 0, st>>>(xb, shb, scb, rows, (int)h, tokens, eps, yb, mean, rstd);
            else if (h <= 3072) ln_modulate_fwd_bf16_kernel<12><<<grid, 256, 0, st>>>(xb, shb, scb, rows, (int)h, tokens, eps, yb, mean, rstd);
            else ln_modulate_fwd_bf16_kernel<16><<<grid, 256, 0, st>>>(xb, shb, scb, rows, (int)h, tokens, eps, yb, mean, rstd);
        } else
            ln_modulate_fwd_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(
                (const __nv_bfloat16*)x, (const __nv_bfloat16*)shift, (const __nv_bfloat16*)scale, rows, (int)h, tokens,
                eps, (__nv_bfloat16*)y, mean, rstd);
        LQ_CUDA(cudaGetLastError());
    });
}

int lq_ln_modulate_bwd(const void* dy, const void* x, const void* scale, const float* mean, const float* rstd, int dtype,
                       int64_t samples, int64_t tokens, int64_t h, void* dx, float* dshift, float* dscale, void* ws,
                       size_t ws_bytes, void* stream) {
    return guarded_call([&] {
        check_common(dy, x, dtype, samples, tokens, h);
        LQ_CHECK_ARG(scale && mean && rstd && dx && dshift && dscale && ws, "NULL argument");
        if (ws_bytes < lq_block_ops_workspace_bytes(samples, tokens, h))
            throw LqError(LQ_ERR_WORKSPACE, "workspace too small for the modulated layer-norm backward");
        cudaStream_t st = (cudaStream_t)stream;
        const int64_t rows = samples * tokens;
        const int chunks = chunks_of(tokens);
        float* p0 = (float*)ws;
        float* p1 = p0 + (size_t)samples * chunks * h;
        LqProf prof(LQ_K_PREP, st);
        const unsigned grid = (unsigned)((rows + 7) / 8);
        const dim3 cg((unsigned)((h + 255) / 256), (unsigned)chunks, (unsigned)samples);
        if (dtype == LQ_F32) {
            ln_modulate_bwd_dx_kernel<float><<<grid, 256, 0, st>>>((const float*)dy, (const float*)x, (const float*)scale,
                                                                   mean, rstd, rows, (int)h, tokens, (float*)dx);
            col_partial_kernel<float, 1><<<cg, 256, 0, st>>>((const float*)dy, (const float*)x, mean, rstd, tokens, (int)h,
                                                             chunks, p0, p1);
        } else if (h % 8 == 0 && h <= 4096 && aligned16(dy) && aligned16(x) && aligned16(scale) && aligned16(dx)) {
            const __nv_bfloat16 *dyb = (const __nv_bfloat16*)dy, *xb = (const __nv_bfloat16*)x, *scb = (const __nv_bfloat16*)scale;
            __nv_bfloat16* dxb = (__nv_bfloat16*)dx;
            if (h <= 1024) ln_modulate_bwd_dx_bf16_kernel<4><<<grid, 256, 0, st>>>(dyb, xb, scb, mean, rstd, rows, (int)h, tokens, dxb);
            else if (h <= 2048) ln_modulate_bwd_dx_bf16_kernel<8><<<grid, 256, 0, st>>>(dyb, xb, scb, mean, rstd, rows, (int)h, tokens, dxb);
            else if (h <= 3072) ln_modulate_bwd_dx_bf16_kernel<12><<<grid, 256, 0, st>>>(dyb, xb, scb, mean, rstd, rows, (int)h, tokens, dxb);
            else ln_modulate_bwd_dx_bf16_kernel<16><<<grid, 256, 0, st>>>(dyb, xb, scb, mean, rstd, rows, (int)h, tokens, dxb);
            const dim3 cg4((unsigned)((h + 1023) / 1024), (unsigned)chunks, (unsigned)samples);
            col_partial_bf16_kernel<1><<<cg4, 256, 0, st>>>(dyb, xb, mean, rstd, tokens, (int)h, chunks, p0, p1);
        } else {
            ln_modulate_bwd_dx_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(
                (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (const __nv_bfloat16*)scale, mean, rstd, rows, (int)h,
                tokens, (__nv_bfloat16*)dx);
            col_partial_kernel<__nv_bfloat16, 1><<<cg, 256, 0, st>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, mean,
                                                                     rstd, tokens, (int)h, chunks, p0, p1);
        }
        const unsigned fg = (unsigned)((samples * h + 255) / 256);
        col_final_kernel<<<fg, 256, 0, st>>>(p0, chunks, (int)h, samples, dscale);
        col_final_kernel<<<fg, 256, 0, st>>>(p1, chunks, (int)h, samples, dshift);
        LQ_CUDA(cudaGetLastError());
    });
}

int lq_gate_residual_fwd(const void* x, const void* gate, const void* y, int dtype, int64_t samples, int64_t tokens,
                         int64_t h, void* out, void* stream) {
    return guarded_call([&] {
        check_common(gate, y, dtype, samples, tokens, h);
        LQ_CHECK_ARG(out != nullptr, "NULL argument");
        cudaStream_t st = (cudaStream_t)stream;
        const int64_t n = samples * tokens * h;
        LqProf prof(LQ_K_PREP, st);
        const unsigned grid = grid_for(n, 256 * 4, 148 * 16);
        if (dtype == LQ_F32)
            gate_residual_kernel<float><<<grid, 256, 0, st>>>((const float*)x, (const float*)gate, (const float*)y, n, (int)h,
                                                              tokens * h, (float*)out);
        else if (h % 8 == 0 && aligned16(x) && aligned16(gate) && aligned16(y) && aligned16(out))
            gate_residual_bf16_kernel<<<grid_for(n / 8, 256, 148 * 16), 256, 0, st>>>(
                (const __nv_bfloat16*)x, (const __nv_bfloat16*)gate, (const __nv_bfloat16*)y, n / 8, (int)h, tokens * h,
                (__nv_bfloat16*)out);
        else
            gate_residual_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)gate,
                                                                      (const __nv_bfloat16*)y, n, (int)h, tokens * h,
                                                                      (__nv_bfloat16*)out);
        LQ_CUDA(cudaGetLastError());
    });
}

int lq_gate_residual_bwd(const void* dout, const void* gate, const void* y, int dtype, int64_t samples, int64_t tokens,
                         int64_t h, void* dy, float* dgate, void* ws, size_t ws_bytes, void* stream) {
    return guarded_call([&] {
        check_common(dout, gate, dtype, samples, tokens, h);
        LQ_CHECK_ARG(y && dy && dgate && ws, "NULL argument");
        if (ws_bytes < lq_block_ops_workspace_bytes(samples, tokens, h))
            throw LqError(LQ_ERR_WORKSPACE, "workspace too small for the gated-residual backward");
        cudaStream_t st = (cudaStream_t)stream;
        const int64_t n = samples * tokens * h;
        const int chunks = chunks_of(tokens);
        float* p0 = (float*)ws;
        LqProf prof(LQ_K_PREP, st);
        const unsigned grid = grid_for(n, 256 * 4, 148 * 16);
        const dim3 cg((unsigned)((h + 255) / 256), (unsigned)chunks, (unsigned)samples);
        if (dtype == LQ_F32) {
            gate_residual_kernel<float><<<grid, 256, 0, st>>>(nullptr, (const float*)gate, (const float*)dout, n, (int)h,
                                                              tokens * h, (float*)dy);  // dy = gate * dout
            col_partial_kernel<float, 0><<<cg, 256, 0, st>>>((const float*)dout, (const float*)y, nullptr, nullptr, tokens,
                                                             (int)h, chunks, p0, nullptr);
        } else if (h % 8 == 0 && aligned16(dout) && aligned16(gate) && aligned16(y) && aligned16(dy)) {
            gate_residual_bf16_kernel<<<grid_for(n / 8, 256, 148 * 16), 256, 0, st>>>(
                nullptr, (const __nv_bfloat16*)gate, (const __nv_bfloat16*)dout, n / 8, (int)h, tokens * h, (__nv_bfloat16*)dy);
            const dim3 cg4((unsigned)((h + 1023) / 1024), (unsigned)chunks, (unsigned)samples);
            col_partial_bf16_kernel<0><<<cg4, 256, 0, st>>>((const __nv_bfloat16*)dout, (const __nv_bfloat16*)y, nullptr, nullptr,
                                                            tokens, (int)h, chunks, p0, nullptr);
        } else {
            gate_residual_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(nullptr, (const __nv_bfloat16*)gate,
                                                                      (const __nv_bfloat16*)dout, n, (int)h, tokens * h,
                                                                      (__nv_bfloat16*)dy);
            col_partial_kernel<__nv_bfloat16, 0><<<cg, 256, 0, st>>>((const __nv_bfloat16*)dout, (const __nv_bfloat16*)y, nullptr,
                                                                     nullptr, tokens, (int)h, chunks, p0, nullptr);
        }
        col_final_kernel<<<(unsigned)((samples * h + 255) / 256), 256, 0, st>>>(p0, chunks, (int)h, samples, dgate);
        LQ_CUDA(cudaGetLastError());
    });
}


// ---- SwiGLU / sigmoid gate ---------------------------------------------------------------------

static void pair_act_launch(int mode, bool bwd, const void* a, const void* b, const void* dout, int dtype, int64_t n,
                            void* o0, void* o1, cudaStream_t st) {
    LQ_CHECK_ARG(dtype == LQ_F32 || dtype == LQ_BF16, "dtype must be LQ_F32 or LQ_BF16");
    LQ_CHECK_ARG(n >= 0, "element count must be >= 0");
    if (n == 0) return;
    LQ_CHECK_ARG(a && b && o0 && (!bwd || (dout && o1)), "NULL argument");
    LQ_CHECK_ARG(aligned16(a) && aligned16(b) && aligned16(o0) && (!bwd || (aligned16(dout) && aligned16(o1))),
                 "tensors must be 16-byte aligned");
    int dev = 0;
    LQ_CUDA(cudaGetDevice(&dev));
    LqProf prof(LQ_K_PREP, st);
    const int vec = dtype == LQ_F32 ? 4 : 8;
    const unsigned grid = grid_for(std::max<int64_t>(n / vec, 1), 256, 148 * 16);
#define LQ_PAIR_ACT(T, M, B)                                                                                      \
    pair_act_kernel<T, M, B><<<grid, 256, 0, st>>>((const T*)a, (const T*)b, (const T*)dout, n, (T*)o0, (T*)o1)
    if (dtype == LQ_F32) {
        if (mode == 0 && !bwd) LQ_PAIR_ACT(float, 0, false);
        else if (mode == 0) LQ_PAIR_ACT(float, 0, true);
        else if (!bwd) LQ_PAIR_ACT(float, 1, false);
        else LQ_PAIR_ACT(float, 1, true);
    } else {
        if (mode == 0 && !bwd) LQ_PAIR_ACT(__nv_bfloat16, 0, false);
        else if (mode == 0) LQ_PAIR_ACT(__nv_bfloat16, 0, true);
        else if (!bwd) LQ_PAIR_ACT(__nv_bfloat16, 1, false);
        else LQ_PAIR_ACT(__nv_bfloat16, 1, true);
    }
#undef LQ_PAIR_ACT
    LQ_CUDA(cudaGetLastError());
}

int lq_swiglu_fwd(const void* gate, const void* up, int dtype, int64_t n, void* out, void* stream) {
    return guarded_call([&] { pair_act_launch(0, false, gate, up, nullptr, dtype, n, out, nullptr, (cudaStream_t)stream); });
}
int lq_swiglu_bwd(const void* dout, const void* gate, const void* up, int dtype, int64_t n, void* dgate, void* dup,
                  void* stream) {
    return guarded_call([&] { pair_act_launch(0, true, gate, up, dout, dtype, n, dgate, dup, (cudaStream_t)stream); });
}
int lq_sigmoid_gate_fwd(const void* x, const void* gate, int dtype, int64_t n, void* out, void* stream) {
    return guarded_call([&] { pair_act_launch(1, false, x, gate, nullptr, dtype, n, out, nullptr, (cudaStream_t)stream); });
}
int lq_sigmoid_gate_bwd(const void* dout, const void* x, const void* gate, int dtype, int64_t n, void* dx, void* dgate,
                        void* stream) {
    return guarded_call([&] { pair_act_launch(1, true, x, gate, dout, dtype, n, dx, dgate, (cudaStream_t)stream); });
}


// ---- ZRmsNorm ------------------------------------------------------------------------------------

int lq_zrmsnorm_fwd(const void* x, const float* scale, int dtype, int64_t rows, int64_t h, float eps, void* y,
                    float* rstd, void* stream) {
    return guarded_call([&] {
        LQ_CHECK_ARG(dtype == LQ_F32 || dtype == LQ_BF16, "dtype must be LQ_F32 or LQ_BF16");
        LQ_CHECK_ARG(rows >= 0 && h >= 1 && h <= (1 << 20), "rows must be >= 0 and h in [1, 2^20]");
        if (rows == 0) return;
        LQ_CHECK_ARG(x && scale && y, "NULL argument");
        cudaStream_t st = (cudaStream_t)stream;
        LqProf prof(LQ_K_PREP, st);
        const unsigned grid = (unsigned)((rows + 7) / 8);
        if (dtype == LQ_F32)
            zrmsnorm_fwd_kernel<float><<<grid, 256, 0, st>>>((const float*)x, scale, rows, (int)h, eps, (float*)y, rstd);
        else
            zrmsnorm_fwd_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, scale, rows, (int)h, eps,
                                                                     (__nv_bfloat16*)y, rstd);
        LQ_CUDA(cudaGetLastError());
    });
}

int lq_zrmsnorm_bwd(const void* dy, const void* x, const float* scale, const float* rstd, int dtype, int64_t rows,
                    int64_t h, void* dx, void* stream) {
    return guarded_call([&] {
        LQ_CHECK_ARG(dtype == LQ_F32 || dtype == LQ_BF16, "dtype must be LQ_F32 or LQ_BF16");
        LQ_CHECK_ARG(rows >= 0 && h >= 1 && h <= (1 << 20), "rows must be >= 0 and h in [1, 2^20]");
        if (rows == 0) return;
        LQ_CHECK_ARG(dy && x && scale && rstd && dx, "NULL argument");
        cudaStream_t st = (cudaStream_t)stream;
        LqProf prof(LQ_K_PREP, st);
        const unsigned grid = (unsigned)((rows + 7) / 8);
        if (dtype == LQ_F32)
            zrmsnorm_bwd_kernel<float><<<grid, 256, 0, st>>>((const float*)dy, (const float*)x, scale, rstd, rows, (int)h,
                                                             (float*)dx);
        else
            zrmsnorm_bwd_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, scale,
                                                                     rstd, rows, (int)h, (__nv_bfloat16*)dx);
        LQ_CUDA(cudaGetLastError());
    });
}

}  // extern "C"
