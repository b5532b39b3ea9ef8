/*
 * loractl_b200 — C ABI of the B200 (sm_100a) quantized frozen-base LoRA linear.
 *
 * This is the boundary a `compute.backend: b200` arm of loractl-core binds to.
 * Every entry point names the loractl-core item it replaces (paths are relative
 * to the loractl repository root).  Conventions:
 *
 *   - all tensor pointers are DEVICE pointers on the device that was current
 *     when the weight handle was created; the library never frees caller memory;
 *   - `stream` is a `cudaStream_t` passed as `void*`; all work is stream-ordered,
 *     nothing synchronises the device unless stated;
 *   - every function returns an `lq_status`; on failure `lq_last_error()` holds
 *     an actionable message for the calling thread.  Nothing aborts or traps, and
 *     there is no CPU fallback: an unsupported request is an error;
 *   - shapes use the reference's names: X is [N, K] (tokens x d_in), the frozen
 *     weight is [M, K] in FILE layout (d_out x d_in, K contiguous, never
 *     transposed — crates/loractl-core/src/mmdit.rs:404-412), LoRA A is [K, r],
 *     LoRA B is [r, M] (burn Linear layout, crates/loractl-core/src/lora.rs:129-136),
 *     s = alpha / rank.
 */
#ifndef LORACTL_B200_H
#define LORACTL_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* The library is built with hidden default visibility; only what this header declares is exported. */
#if defined(__GNUC__)
#pragma GCC visibility push(default)
#endif

#define LQ_ABI_VERSION 2

typedef enum lq_status {
    LQ_OK = 0,
    LQ_ERR_INVALID = 1,     /* bad argument (the reference panics / bails here) */
    LQ_ERR_CUDA = 2,        /* a CUDA runtime/driver call failed */
    LQ_ERR_UNSUPPORTED = 3, /* valid request this build cannot run (never falls back) */
    LQ_ERR_TIMEOUT = 4,     /* a bounded device-side wait gave up; context stays usable */
    LQ_ERR_WORKSPACE = 5    /* caller workspace too small */
} lq_status;

/* Activation / output element type of one call.  LQ_F32 runs f32 arithmetic
 * end to end (the reference's own precision on the quant path,
 * crates/loractl-core/src/diffusion_trainer.rs:395-401); LQ_BF16 runs bf16
 * operands with f32 accumulation on the tcgen05 tensor cores. */
typedef enum lq_dtype {
    LQ_F32 = 0,
    LQ_BF16 = 1,
    /* bf16 activations in and out, but the frozen GEMM runs natively in fp8: the stored e4m3
     * weight bytes are the MMA operand (no dequantisation pass), activations are quantised to e4m3
     * with one f32 scale per token, scales are applied in the epilogue (tcgen05 kind::f8f6f4, f32
     * accumulation).  Scaled-fp8 weights only.  The reference has no fp8 compute at all
     * (crates/loractl-core/src/fp8.rs decodes at load time); tolerance is correspondingly looser. */
    LQ_BF16_W8A8 = 2
} lq_dtype;

/* Storage scheme of a frozen weight.  INT8/INT4 are crates/loractl-core/src/
 * config.rs:637-649 `Quant::{Int8,Int4}` (symmetric, per-block f32 scale);
 * FP8_E4M3 is the scaled-fp8 repack of crates/loractl-core/src/fp8.rs. */
typedef enum lq_scheme { LQ_INT4 = 4, LQ_INT8 = 8, LQ_FP8_E4M3 = 108 } lq_scheme;

/* How an fp8 `weight_scale` broadcasts (crates/loractl-core/src/fp8.rs:59-68). */
typedef enum lq_scale_kind { LQ_SCALE_SCALAR = 0, LQ_SCALE_PER_CHANNEL = 1 } lq_scale_kind;

/* Opaque frozen quantized weight: replaces the `QFloat` tensor(s) + bias held by
 * `QuantLinear` (crates/loractl-core/src/mmdit.rs:413-428).  Immutable after
 * creation except for lq_weight_set_bias; shareable across threads. */
typedef struct lq_weight lq_weight_t;

typedef struct lq_weight_info {
    int64_t d_out;        /* M */
    int64_t d_in;         /* K */
    int32_t scheme;       /* lq_scheme */
    int32_t group;        /* elements per scale block along K (0 for fp8) */
    int32_t scale_kind;   /* lq_scale_kind (fp8 only) */
    int32_t has_bias;
    int32_t device;
    int32_t reserved;
    uint64_t packed_bytes; /* resident code bytes (padded, tile-contiguous) */
    uint64_t scale_bytes;  /* resident scale bytes */
} lq_weight_info;

/* Message for the last failure on the calling thread ("" if none). */
const char* lq_last_error(void);
int lq_abi_version(void);

/* ---- quantize / pack -------------------------------------------------------- */

/* crates/loractl-core/src/quant.rs:102-117 `dequant_chunk_rows` — pure host
 * function.  Writes at most `cap` row counts to `rows` and the chunk count to
 * `n_chunks` (call with cap = 0 to size the array). */
int lq_dequant_chunk_rows(uint64_t d_out, uint64_t d_in, uint64_t chunk_bytes,
                          uint64_t* rows, size_t cap, size_t* n_chunks);

/* crates/loractl-core/src/quant.rs:74-82 `quantize_linear_weight`: quantizes a
 * device-resident [M, K] weight (w_dtype LQ_F32 or LQ_BF16, K contiguous) with the
 * `quant_scheme` of quant.rs:61-67 — symmetric, one f32 scale per `group` elements
 * along K, bits 4 (Q4S, clamp +-7) or 8 (Q8S, clamp +-127), rounding half away from
 * zero.  `group` must be 32 (QUANT_BLOCK, quant.rs:52) or 64; K % group != 0 is
 * LQ_ERR_INVALID (the reference asserts, quant.rs:76-80).  Allocates the handle's
 * device storage (load-time path; not for the step loop). */
int lq_quantize(const void* w, int w_dtype, int64_t d_out, int64_t d_in, int group, int bits,
                void* stream, lq_weight_t** out);

/* The streaming requantisation of crates/loractl-core/src/diffusion_trainer.rs:1130-1175 for a
 * scaled-fp8 checkpoint tensor, in one pass on the device: element = LUT[byte] * weight_scale
 * (crates/loractl-core/src/fp8.rs:305-317; `scale` scalar or per-out-channel, device pointer),
 * then quantized like lq_quantize (crates/loractl-core/src/quant.rs:74-82).  Bit-identical to
 * dequantizing to f32 first; the f32 tensor is never materialised.  `bytes`: device, row-major
 * [d_out, d_in] e4m3fn. */
int lq_quantize_from_fp8(const uint8_t* bytes, const float* scale, int scale_kind, int64_t d_out,
                         int64_t d_in, int group, int bits, void* stream, lq_weight_t** out);

/* Builds a handle from already-quantized logical data: `codes` int8 [M, K] and
 * `scales` f32 [M, K/group] on the device (the logical content of a burn QFloat
 * tensor; used to join row chunks — crates/loractl-core/src/quant.rs:130-150 — and
 * to load pre-quantized weights). */
int lq_weight_from_codes(const int8_t* codes, const float* scales, int64_t d_out, int64_t d_in,
                         int group, int bits, void* stream, lq_weight_t** out);

/* crates/loractl-core/src/fp8.rs:279-329: wraps scaled-fp8 storage — `bytes` u8
 * [M, K] e4m3fn (device), `scale` f32 scalar or [M] (device) — WITHOUT decoding it:
 * the bytes stay fp8 in HBM and are decoded inside the kernels.  Copies both. */
int lq_weight_from_fp8(const uint8_t* bytes, const float* scale, int scale_kind, int64_t d_out,
                       int64_t d_in, void* stream, lq_weight_t** out);

/* reference/fp8_reference.py:84-94 `quantize`: scale = amax/448 (>= 1e-12), scalar
 * or per output row; q = e4m3fn(w / scale), round to nearest even.  `w` f32 [M, K]
 * on the device. */
int lq_fp8_quantize(const float* w, int64_t d_out, int64_t d_in, int per_channel, void* stream,
                    lq_weight_t** out);

/* `QuantLinear.bias` (crates/loractl-core/src/mmdit.rs:426-427): optional f32 [M],
 * copied; NULL clears it. */
int lq_weight_set_bias(lq_weight_t* w, const float* bias, void* stream);

int lq_weight_info_get(const lq_weight_t* w, lq_weight_info* info);
int lq_weight_destroy(lq_weight_t* w);

/* Logical view of the packed storage, for bit-exactness checks independent of the
 * tile layout: int4/int8 -> `codes` int8 [M, K], `scales` f32 [M, K/group];
 * fp8 -> `codes` receives the raw e4m3 bytes, `scales` f32 [1] or [M]. */
int lq_unpack(const lq_weight_t* w, int8_t* codes, float* scales, void* stream);

/* `QuantLinear::dequantized_weight` (crates/loractl-core/src/mmdit.rs:435-444) /
 * burn `dequantize`: the full [M, K] weight, `q * scale` (or `LUT[b] * scale`,
 * crates/loractl-core/src/fp8.rs:305-317) computed in f32, stored as out_dtype. */
int lq_dequantize(const lq_weight_t* w, void* out, int out_dtype, void* stream);

/* A resident bf16 copy of the dequantised weight, [d_out, d_in] row-major, in a caller-owned buffer
 * of lq_weight_bf16_copy_bytes() bytes (16-byte aligned, d_in % 8 == 0).  The reference dequantises
 * the whole weight to f32 inside every forward and every backward (crates/loractl-core/src/
 * quant.rs:232,250); the LQ_BF16 tensor-regime calls normally do the same into the caller's
 * workspace, in bf16.  A GPU with 180 GB can afford to keep that copy: while one is attached the
 * calls read it directly — the forward as a K-major operand, the backward (reduction over d_out) as
 * an MN-major operand of the same buffer — and run no dequantisation pass at all.  The values are
 * the same bf16(q * scale), so results do not change.  `lq_weight_attach_bf16_copy` fills the
 * buffer (one pass, stream-ordered) and attaches it; buffer = NULL detaches.  A trainer may attach
 * for the whole run (2 bytes per element resident) or around one block's replay under block
 * checkpointing (one pass instead of two per site).  Load-time call: do not attach or detach while
 * another thread runs calls on the same handle. */
size_t lq_weight_bf16_copy_bytes(const lq_weight_t* w);
int lq_weight_attach_bf16_copy(lq_weight_t* w, void* buffer, void* stream);

/* ---- the hot path ----------------------------------------------------------- */

/* Scratch the two calls below need for this (weight, N, rank, dtype); the caller
 * owns the buffer (no hidden allocation in the step loop).  256-byte aligned. */
size_t lq_linear_workspace_bytes(const lq_weight_t* w, int64_t n_tokens, int rank, int dtype);

/* One LoRA'd quantized site, forward — `site()` at crates/loractl-core/src/
 * mmdit.rs:526-536: BaseLinear::forward (mmdit.rs:483-519: x . dequant(wq)^T + bias)
 * followed by LoraAdapters::apply (crates/loractl-core/src/adapters.rs:75-85) with
 * LoraDelta::forward (crates/loractl-core/src/lora.rs:199-203):
 *
 *     Y[N,M] = X[N,K] . dequant(W)[M,K]^T + bias[M] + s * (X . A[K,r]) . B[r,M]
 *
 * X, Y have element type `dtype`; A, B are f32 (trainable parameters stay f32).
 * rank == 0 (A, B NULL) is exactly `QuantBackend::quant_matmul_t`
 * (crates/loractl-core/src/quant.rs:172-178) plus bias.  `H_out` (f32 [N, r],
 * may be NULL) receives H = X . A for the backward.  Dropout on the adapter input
 * is not supported (p must be 0; the reference forbids it under recompute,
 * crates/loractl-core/src/diffusion_trainer.rs:342-348).  `lora_mirror` (may be NULL): the bf16
 * operand arrays of A and B kept by the caller, see lq_lora_mirror_update; A and B must still be
 * passed (paths that compute in f32 read them). */
int lq_linear_fwd(const lq_weight_t* w, const void* X, int64_t n_tokens, int dtype,
                  const float* A, const float* B, int rank, float scaling,
                  void* Y, float* H_out, void* workspace, size_t workspace_bytes, void* stream,
                  const void* lora_mirror);

/* Backward of lq_linear_fwd — `QuantMatmulT::backward` (crates/loractl-core/src/
 * quant.rs:221-235: dX = dY . dequant(wq), no gradient to the weight) plus the stock
 * autodiff of the LoRA delta (restated in reference/lora_reference.py:103-123):
 *
 *     dH = s * dY . B^T      dX[N,K] = dY . dequant(W) + dH . A^T
 *     dA[K,r] = X^T . dH     dB[r,M] = s * H^T . dY
 *
 * dY, X, dX have element type `dtype`; H is the f32 [N, r] saved by the forward
 * (NULL: recomputed as X . A); dA, dB are f32 and are OVERWRITTEN unless
 * `accumulate` is non-zero (then added to, for a flat gradient bucket).
 * dX may be NULL (input needs no gradient); dA/dB may be NULL when rank == 0.
 * Routes (bf16): int4 weights at <= 16 tokens read the packed weight once and
 * convert it in registers (no bf16 image of W^T is written; dH, dA, dB are formed by the same two
 * launches); everything else dequantises into the workspace, or reads an attached bf16 copy. */
int lq_linear_bwd(const lq_weight_t* w, const void* dY, const void* X, const float* H,
                  int64_t n_tokens, int dtype, const float* A, const float* B, int rank,
                  float scaling, void* dX, float* dA, float* dB, int accumulate,
                  void* workspace, size_t workspace_bytes, void* stream, const void* lora_mirror);

/* bf16 mirror of one site's LoRA factors.  The reference keeps A and B as f32 `Linear` weights and
 * lets every forward and backward read them as they are (crates/loractl-core/src/lora.rs:155-166,
 * 199-203); the tensor-core path wants them as bf16 GEMM operands (A, A^T, B, B^T, zero padded to a
 * multiple of 64 columns).  Casting them inside each call costs five short launches per site and
 * pass; the factors only change once per optimizer step, so a trainer may keep this mirror beside
 * the parameters (lq_lora_mirror_bytes bytes, 256-byte aligned, caller-owned), refresh it with one
 * launch after each update, and hand it to lq_linear_fwd / lq_linear_bwd.  A stale mirror gives
 * stale results: refresh it whenever A or B changed. */
size_t lq_lora_mirror_bytes(int64_t d_in, int64_t d_out, int rank);
int lq_lora_mirror_update(const float* A, const float* B, int64_t d_in, int64_t d_out, int rank,
                          void* mirror, void* stream);
/* The same for many sites at once (all adapters of a model after `optim.step`,
 * crates/loractl-core/src/diffusion_trainer.rs:1728): one launch per 24 sites instead of one per site. */
typedef struct lq_mirror_job {
    const float* A;   /* [d_in, rank] f32 */
    const float* B;   /* [rank, d_out] f32 */
    int64_t d_in, d_out;
    int32_t rank;
    void* mirror;     /* lq_lora_mirror_bytes(d_in, d_out, rank) bytes, 256-byte aligned */
} lq_mirror_job;
int lq_lora_mirror_update_batch(const lq_mirror_job* jobs, int n_jobs, void* stream);

/* Several sites that read the SAME activation — the reference calls `site()` three times on one x
 * for wq / wk / wv and twice for gate / up (crates/loractl-core/src/mmdit.rs:599-610,701-706) — in
 * one call.  Semantics per site are exactly lq_linear_fwd's (Y_i = X . dequant(W_i)^T + bias_i +
 * s_i (X . A_i) . B_i, H_i = X . A_i).  With int4 weights of one d_in and quant block at <= 16 tokens
 * (LQ_BF16) the whole group is ONE launch of the packed-weight-stream kernel over the concatenated
 * work list of the sites plus one finalize launch, so launch ramp and tail are paid once per group;
 * any other request runs the sites one after the other through lq_linear_fwd.  At most 4 sites take
 * the one-launch path.  `workspace`: at least lq_linear_grouped_workspace_bytes() bytes. */
typedef struct lq_group_site {
    const lq_weight_t* w;
    const float* A;      /* [d_in, rank] f32, NULL when rank == 0 */
    const float* B;      /* [rank, d_out] f32 */
    int32_t rank;
    float scaling;
    void* Y;             /* [n_tokens, d_out] */
    float* H_out;        /* [n_tokens, rank] f32, may be NULL */
} lq_group_site;
size_t lq_linear_grouped_workspace_bytes(const lq_group_site* sites, int n_sites, int64_t n_tokens, int dtype);
int lq_linear_fwd_grouped(const lq_group_site* sites, int n_sites, const void* X, int64_t n_tokens, int dtype,
                          void* workspace, size_t workspace_bytes, void* stream);

/* Builds, once, the transposed copy of a scaled-fp8 weight that the LQ_BF16_W8A8 backward reads
 * ([d_in, d_out] e4m3 bytes, +1 byte per element of resident memory).  Optional: the first
 * LQ_BF16_W8A8 backward builds it on demand (one cudaMalloc); call this at load time to keep the
 * step loop allocation-free.  No counterpart in the reference. */
int lq_weight_prepare_fp8_backward(const lq_weight_t* w, void* stream);

/* ---- step glue on the flat LoRA buffers ---------------------------------------- */

/* crates/loractl-core/src/diffusion_trainer.rs:1708-1725 (the finite check over every adapter
 * gradient): clears the device int `flag`, then sets it to 1 if any of the `n` floats of the flat
 * gradient buffer is NaN or Inf.  One kernel, no host synchronisation. */
int lq_grad_nonfinite_flag(const float* grads, int64_t n, int* flag, void* stream);

/* crates/loractl-core/src/diffusion_trainer.rs:1564-1566,1727-1728 (burn AdamW, decoupled decay)
 * as one pass over flat f32 buffers of every adapter parameter:
 *   p -= lr*wd*p;  m = b1 m + (1-b1) g;  v = b2 v + (1-b2) g^2;
 *   p -= lr * (m / (1-b1^step)) / (sqrt(v / (1-b2^step)) + eps),   g = grad_scale * grads[i].
 * `step` is the 1-based update count.  A non-zero device int at `skip_flag` (may be NULL) makes
 * the call a no-op: the "skip the update" branch of the dynamic loss scale
 * (diffusion_trainer.rs:1732-1742), taken on the device. */
int lq_adamw_step(float* params, const float* grads, float* exp_avg, float* exp_avg_sq, int64_t n,
                  float lr, float beta1, float beta2, float eps, float weight_decay, int64_t step,
                  float grad_scale, const int* skip_flag, void* stream);

/* ---- element-wise companions of the linears inside a DiT block ------------------ */

/* crates/loractl-core/src/mmdit.rs:857-869: the block's `(scale + 1) * norm(x) + shift` prologues
 * and `x + gate * f(..)` residuals, which the reference runs as separate broadcast multiplies and
 * adds.  x, y, out: [samples, tokens, h] contiguous; shift, scale, gate: [samples, h] contiguous,
 * broadcast over the tokens of their sample; `dtype` LQ_F32 or LQ_BF16 for all of them.  The norm is
 * a layer norm over h without affine parameters, statistics in f32; `mean`, `rstd`: f32 [samples *
 * tokens], written by the forward and read by the backward.  The backward's token-axis sums
 * (`dshift`, `dscale`, `dgate`: f32 [samples, h]) are reduced in a fixed order (no atomics) through
 * `ws`, at least lq_block_ops_workspace_bytes() bytes. */
size_t lq_block_ops_workspace_bytes(int64_t samples, int64_t tokens, int64_t h);
int lq_ln_modulate_fwd(const void* x, const void* shift, const void* scale, int dtype, int64_t samples,
                       int64_t tokens, int64_t h, float eps, void* y, float* mean, float* rstd,
                       void* stream);
int lq_ln_modulate_bwd(const void* dy, const void* x, const void* scale, const float* mean,
                       const float* rstd, int dtype, int64_t samples, int64_t tokens, int64_t h,
                       void* dx, float* dshift, float* dscale, void* ws, size_t ws_bytes, void* stream);
/* out = x + gate * y. */
int lq_gate_residual_fwd(const void* x, const void* gate, const void* y, int dtype, int64_t samples,
                         int64_t tokens, int64_t h, void* out, void* stream);
/* dy = gate * dout, dgate = sum over tokens of dout * y (d x is dout itself). */
int lq_gate_residual_bwd(const void* dout, const void* gate, const void* y, int dtype, int64_t samples,
                         int64_t tokens, int64_t h, void* dy, float* dgate, void* ws, size_t ws_bytes,
                         void* stream);

/* The two activations between linears of the reference's own block, one pass forward and one pass
 * backward each, over `n` contiguous elements of type `dtype` (LQ_F32 or LQ_BF16; f32 arithmetic;
 * 16-byte aligned pointers):
 *   SwiGLU (crates/loractl-core/src/mmdit.rs:695-708)            out = silu(gate) * up
 *   attention output gate (crates/loractl-core/src/mmdit.rs:659-664)   out = x * sigmoid(gate)
 * The reference runs each as two or three burn tensor ops (and as many autodiff nodes). */
int lq_swiglu_fwd(const void* gate, const void* up, int dtype, int64_t n, void* out, void* stream);
int lq_swiglu_bwd(const void* dout, const void* gate, const void* up, int dtype, int64_t n,
                  void* dgate, void* dup, void* stream);
int lq_sigmoid_gate_fwd(const void* x, const void* gate, int dtype, int64_t n, void* out, void* stream);
int lq_sigmoid_gate_bwd(const void* dout, const void* x, const void* gate, int dtype, int64_t n,
                        void* dx, void* dgate, void* stream);

/* ZRmsNorm (crates/loractl-core/src/mmdit.rs:282-330): y = x / sqrt(mean(x^2) + eps) * (scale + 1)
 * over rows of `h` contiguous elements (`dtype` LQ_F32 or LQ_BF16; `scale` f32 [h], frozen: the
 * backward yields dx only); `rstd` f32 [rows] is written by the forward (may be NULL when no backward
 * follows) and read by the backward. */
int lq_zrmsnorm_fwd(const void* x, const float* scale, int dtype, int64_t rows, int64_t h, float eps,
                    void* y, float* rstd, void* stream);
int lq_zrmsnorm_bwd(const void* dy, const void* x, const float* scale, const float* rstd, int dtype,
                    int64_t rows, int64_t h, void* dx, void* stream);

/* ---- diagnostics -------------------------------------------------------------- */

/* Device-side waits in the kernels are bounded; one that gives up records a code in a
 * per-device error word instead of hanging.  This call synchronises `stream`, returns
 * LQ_ERR_TIMEOUT (and clears the word) if a kernel gave up since the last call, else
 * LQ_OK.  It is the device-side half of the reference's "fail loudly" policy
 * (crates/loractl-core/src/config.rs:503-512); a trainer calls it where the reference
 * reads the loss back (crates/loractl-core/src/diffusion_trainer.rs:1675). */
int lq_check_device_status(void* stream);

/* Self-test of that mechanism (no reference counterpart; the reference has no device-side waits):
 * launches one warp that waits, with the kernels' own bounded-wait routine and a limit of
 * `limit_ms` (1..1000), on a barrier nothing arrives on.  The wait runs out, the kernel records
 * wait site 90 and returns; the next lq_check_device_status() reports LQ_ERR_TIMEOUT and clears
 * the word, and the context stays usable.  Nothing faults or spins without a limit. */
int lq_selftest_bounded_wait(unsigned limit_ms, void* stream);

/* Launch accounting for benchmarks — the counterpart of the reference's bench probes
 * (crates/loractl-core/src/probe.rs:24-39 phase markers; crates/loractl-bench/src/lib.rs).
 * lq_kernel_launch_count: kernels this library has launched in this process so far.
 * lq_profile_enable(1): from now on every launch is bracketed by a CUDA event pair on its
 * stream; lq_profile_collect synchronises the device and returns, per kernel class
 * (lq_profile_kinds() of them, named by lq_profile_kind_name), the summed milliseconds and
 * the number of timed launches since the last collect, then forgets them. */
uint64_t lq_kernel_launch_count(void);
int lq_profile_enable(int on);
int lq_profile_kinds(void);
const char* lq_profile_kind_name(int kind);
int lq_profile_collect(double* ms_by_kind, uint64_t* launches_by_kind, int n_kinds);

/* Run-time switches of the kernel selection, for A/B measurements and tests (the reference selects
 * code paths through `compute.*` config keys, crates/loractl-core/src/config.rs:704-760; these are
 * the equivalent knobs below the boundary).  Process-wide; initial values come from the environment
 * variables of the same meaning (LQ_W4, LQ_W4_EXACT, LQ_BWD_MN, LQ_TAIL_SPLIT).
 *   "w4"        1: int4 weights at >= 128 tokens are dequantised inside the GEMM mainloop and no bf16
 *               copy of the weight is written to HBM; 0 (default: it measured faster at every size
 *               tried): dequantise into the workspace.
 *   "w4_exact"  how the in-mainloop conversion forms a bf16 weight from (q, scale):
 *               1: bf16(q * scale) with the f32 product, bit-identical to the workspace path;
 *               2: fma(q, s_hi, bf16(q * s_lo)) with the scale split into two bf16 terms — one
 *                  rounding of q * scale except within 2^-18 of a rounding boundary;
 *               0: bf16(q * bf16(scale)).
 *   "bwd_mn"    1: the backward dequantises W in its own orientation and the dX GEMM reads that
 *               scratch as an MN-major operand; 0 (default): transposed scratch, K-major operand.
 *   "tail_split" 1 (default): a frozen GEMM with a long reduction whose last (or only) round of the
 *               persistent grid is at most half full has those tiles cut along k (f32 partial tiles
 *               in the workspace, summed in a fixed order by a second launch); 0: whole tiles only.
 *   "reserve_sms" n (default 0): SMs the persistent GEMM grids leave free, for a trainer whose
 *               collectives run beside them (LQ_RESERVE_SMS).
 * Unknown names are LQ_ERR_INVALID. */
int lq_option_set(const char* name, int value);

/* The bare tcgen05 contraction the hot path is built from, exposed for unit tests and
 * roofline probes: C[Mg, Ng] = A . B^T + bias with bf16 operands and f32 accumulation.
 * An operand is K-major ([rows, Kg], Kg contiguous; *_mn = 0) or MN-major ([Kg, rows], rows
 * contiguous; *_mn = 1); ld* are row strides in elements.  block_n is 64, 128 or 256;
 * splits > 1 needs c_dtype LQ_F32, block_n 64, splits <= ceil(Kg / 64) and `partial_ws` of
 * splits * Mg * roundup(Ng, 64) floats.  The reference has no counterpart: burn's
 * `float_matmul` (crates/loractl-core/src/quant.rs:233,251) is the nearest equivalent. */
int lq_gemm_bf16(const void* A, int a_mn, int64_t lda, const void* B, int b_mn, int64_t ldb,
                 void* C, int c_dtype, int64_t ldc, int64_t Mg, int64_t Ng, int64_t Kg,
                 int block_n, int splits, float* partial_ws, const float* bias, void* stream);

/* Split-K contraction that allocates nothing — it has no counterpart in the reference.
 *
 *     C[Mg, Ng] (f32, row stride ldc) = A . B^T      bf16 operands, f32 accumulation
 *
 * Same arithmetic as lq_gemm_bf16 with c_dtype LQ_F32, block_n 64 and `splits` k-ranges, but the
 * caller passes no partial-sum workspace: the partial tiles live in a fixed 16 MiB array built
 * into the library (one per GPU that loads it, held until the process exits).  It is meant for
 * callers that cannot call cudaMalloc where they need the result — a stream that is being
 * captured, an allocator callback, a loop whose memory was fixed at start-up.  The call itself
 * performs no cudaMalloc / cudaFree and no other allocating device call.
 *
 * Both operands are K-major ([rows, Kg], operands_mn = 0) or both MN-major ([Kg, rows],
 * operands_mn = 1); lda / ldb are their row strides in elements.
 * Limit: splits * Mg * roundup(Ng, 64) must not exceed 4 * 2^20 floats, else LQ_ERR_WORKSPACE.
 * The first call on each device looks up the array's device address (cudaGetSymbolAddress) and
 * the SM count; make that first call before any stream capture begins.
 * Every call on a GPU shares the one array and it keeps the previous call's contents: calls that
 * may overlap on the GPU (different streams without ordering) race and must be serialised by the
 * caller.  If a bounded device-side wait gives up, every element of C is NaN and the next
 * lq_check_device_status() on that device returns LQ_ERR_TIMEOUT. */
int lq_gemm_bf16_splitk_static(const void* A, const void* B, int operands_mn, int64_t lda, int64_t ldb,
                               float* C, int64_t ldc, int64_t Mg, int64_t Ng, int64_t Kg, int splits,
                               void* stream);

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif

#ifdef __cplusplus
}
#endif
#endif /* LORACTL_B200_H */
