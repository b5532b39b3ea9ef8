// C ABI of libloractl_b200: argument validation, handle ownership, dispatch.
//
// Every entry point converts C++ exceptions into an lq_status plus a thread-local
// message; nothing here aborts.  There is no CPU path: requests the GPU kernels cannot
// run are LQ_ERR_UNSUPPORTED.
#include <cstring>
#include <memory>
#include <mutex>
#include <vector>

#include "lq_internal.cuh"
#include "lq_tc.cuh"

namespace {

thread_local std::string g_last_error;

template <typename F>
int guarded(F&& f) {
    try {
        f();
        g_last_error.clear();
        return LQ_OK;
    } catch (const LqError& e) {
        g_last_error = e.what();
        return e.status;
    } catch (const std::exception& e) {
        g_last_error = std::string("internal error: ") + e.what();
        return LQ_ERR_INVALID;
    }
}

struct DeviceGuard {
    int prev = -1;
    explicit DeviceGuard(int dev) {
        LQ_CUDA(cudaGetDevice(&prev));
        if (prev != dev) LQ_CUDA(cudaSetDevice(dev));
        else prev = -1;
    }
    ~DeviceGuard() {
        if (prev >= 0) cudaSetDevice(prev);
    }
};

void check_sm100(int dev) {
    static std::mutex mu;
    static std::vector<int> ok;  // per device: 0 unknown, 1 ok
    std::lock_guard<std::mutex> lk(mu);
    if ((int)ok.size() <= dev) ok.resize(dev + 1, 0);
    if (ok[dev]) return;
    int major = 0, minor = 0;
    LQ_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
    LQ_CUDA(cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev));
    if (major != 10)
        throw LqError(LQ_ERR_UNSUPPORTED, "compute.backend b200 needs an sm_100 device; device " + std::to_string(dev) +
                                              " is sm_" + std::to_string(major) + std::to_string(minor) +
                                              " (no fallback)");
    ok[dev] = 1;
}

std::unique_ptr<lq_weight> new_handle(int scheme, int64_t M, int64_t K, int group, int scale_kind) {
    LQ_CHECK_ARG(M > 0 && K > 0, "weight dims must be positive");
    auto h = std::make_unique<lq_weight>();
    LQ_CUDA(cudaGetDevice(&h->device));
    check_sm100(h->device);
    h->scheme = scheme;
    h->M = M;
    h->K = K;
    h->group = group;
    h->scale_kind = scale_kind;
    if (scheme == LQ_FP8_E4M3) {
        h->m_tiles = h->k_tiles = h->n_groups = 0;
        h->packed_bytes = (size_t)M * (size_t)K;
        h->scale_bytes = sizeof(float) * (scale_kind == LQ_SCALE_PER_CHANNEL ? (size_t)M : 1);
    } else {
        h->m_tiles = (M + LQ_TILE_M - 1) / LQ_TILE_M;
        h->k_tiles = (K + LQ_TILE_K - 1) / LQ_TILE_K;
        h->n_groups = K / group;
        size_t tile_bytes = scheme == LQ_INT4 ? 4096 : 8192;
        h->packed_bytes = (size_t)h->m_tiles * (size_t)h->k_tiles * tile_bytes;
        h->scale_bytes = sizeof(float) * (size_t)h->m_tiles * (size_t)h->n_groups * 128;
    }
    LQ_CUDA(cudaMalloc(&h->packed, h->packed_bytes));
    cudaError_t e = cudaMalloc((void**)&h->scales, h->scale_bytes);
    if (e != cudaSuccess) {
        cudaFree(h->packed);
        throw LqError(LQ_ERR_CUDA, std::string("cudaMalloc(scales): ") + cudaGetErrorString(e));
    }
    return h;
}

void free_handle(lq_weight* h) {
    if (!h) return;
    cudaFree(h->packed);
    cudaFree(h->scales);
    cudaFree(h->bias);
    cudaFree(h->packed_t);
    delete h;
}

void check_int_scheme(int64_t M, int64_t K, int group, int bits) {
    LQ_CHECK_ARG(bits == 4 || bits == 8, "quant bits must be 4 (int4, Q4S) or 8 (int8, Q8S)");
    LQ_CHECK_ARG(group == 32 || group == 64, "quant block must be 32 or 64 elements along d_in");
    if (K % group != 0)
        throw LqError(LQ_ERR_INVALID, "linear weight [" + std::to_string(M) + ", " + std::to_string(K) +
                                          "]: the input dim must be a multiple of the quant block (" +
                                          std::to_string(group) + ")");
}

inline size_t align256(size_t x) { return (x + 255) & ~size_t(255); }

// Carves the caller's workspace; every sub-buffer is 256-byte aligned.
struct Carver {
    char* base;
    size_t cap, used = 0;
    Carver(void* p, size_t c) : base((char*)p), cap(c) {}
    void* take(size_t bytes) {
        size_t off = align256(used);
        used = off + bytes;
        if (base == nullptr) return nullptr;  // sizing pass
        if (used > cap)
            throw LqError(LQ_ERR_WORKSPACE, "workspace too small: need at least " + std::to_string(used) +
                                                " bytes, got " + std::to_string(cap) +
                                                " (query lq_linear_workspace_bytes)");
        return base + off;
    }
};

void check_call(const lq_weight* w, int64_t N, int dtype, const float* A, const float* B, int rank) {
    LQ_CHECK_ARG(w != nullptr, "weight handle is NULL (quant_matmul_t requires a quantized weight)");
    LQ_CHECK_ARG(N >= 0, "n_tokens must be >= 0");
    LQ_CHECK_ARG(dtype == LQ_F32 || dtype == LQ_BF16 || dtype == LQ_BF16_W8A8,
                 "dtype must be LQ_F32, LQ_BF16 or LQ_BF16_W8A8");
    if (dtype == LQ_BF16_W8A8 && !lq_w8a8_supported(w, N, rank))
        throw LqError(LQ_ERR_UNSUPPORTED,
                      "LQ_BF16_W8A8 (native fp8 compute) needs a scaled-fp8 weight with d_in % 16 == 0 and "
                      "d_out % 16 == 0; int4/int8 weights compute in bf16 (no fallback is taken silently)");
    LQ_CHECK_ARG(rank >= 0 && rank <= 256, "LoRA rank must be in [0, 256]");
    if (rank > 0) LQ_CHECK_ARG(A != nullptr && B != nullptr, "rank > 0 needs LoRA factors A [K,r] and B [r,M]");
}

// ---- f32-arithmetic path (SIMT) ---------------------------------------------------

LqSimtArgs simt_base(const void* A, int a_dtype, int64_t sa_i, int64_t sa_k, void* C, int c_dtype, int64_t ldc,
                     int64_t I, int64_t J, int64_t Kred) {
    LqSimtArgs a{};
    a.A = A; a.a_dtype = a_dtype; a.sa_i = sa_i; a.sa_k = sa_k;
    a.C = C; a.c_dtype = c_dtype; a.ldc = ldc;
    a.I = I; a.J = J; a.Kred = Kred;
    a.alpha = 1.f; a.beta = 0; a.bias = nullptr; a.b_mode = 0; a.Bp = nullptr; a.b_dtype = LQ_F32; a.sb_k = a.sb_j = 0;
    return a;
}

void fwd_simt(const lq_weight* w, const void* X, int64_t N, int dtype, const float* A, const float* B, int r,
              float s, void* Y, float* H, cudaStream_t st) {
    const int64_t M = w->M, K = w->K;
    // Y = X . dq^T + bias   (crates/loractl-core/src/mmdit.rs:497-514)
    LqSimtArgs g = simt_base(X, dtype, K, 1, Y, dtype, M, N, M, K);
    g.b_mode = 1; g.W = lq_view(w); g.bias = w->bias;
    lq_launch_simt_gemm(g, st);
    if (r == 0) return;
    // H = X . A ; Y += s * (H . B)   (crates/loractl-core/src/lora.rs:199-203)
    LqSimtArgs h = simt_base(X, dtype, K, 1, H, LQ_F32, r, N, r, K);
    h.Bp = A; h.sb_k = r; h.sb_j = 1;
    lq_launch_simt_gemm(h, st);
    LqSimtArgs d = simt_base(H, LQ_F32, r, 1, Y, dtype, M, N, M, r);
    d.Bp = B; d.sb_k = M; d.sb_j = 1; d.alpha = s; d.beta = 1;
    lq_launch_simt_gemm(d, st);
}

void bwd_simt(const lq_weight* w, const void* dY, const void* X, const float* H, int64_t N, int dtype,
              const float* A, const float* B, int r, float s, void* dX, float* dA, float* dB, int accumulate,
              float* dH, cudaStream_t st) {
    const int64_t M = w->M, K = w->K;
    if (dX) {  // dX = dY . dq   (crates/loractl-core/src/quant.rs:229-234)
        LqSimtArgs g = simt_base(dY, dtype, M, 1, dX, dtype, K, N, K, M);
        g.b_mode = 2; g.W = lq_view(w);
        lq_launch_simt_gemm(g, st);
    }
    if (r == 0) return;
    // dH = s * dY . B^T
    LqSimtArgs h = simt_base(dY, dtype, M, 1, dH, LQ_F32, r, N, r, M);
    h.Bp = B; h.sb_k = 1; h.sb_j = M; h.alpha = s;
    lq_launch_simt_gemm(h, st);
    if (dX) {  // dX += dH . A^T
        LqSimtArgs g = simt_base(dH, LQ_F32, r, 1, dX, dtype, K, N, K, r);
        g.Bp = A; g.sb_k = 1; g.sb_j = r; g.beta = 1;
        lq_launch_simt_gemm(g, st);
    }
    if (dA) {  // dA = X^T . dH
        LqSimtArgs g = simt_base(X, dtype, 1, K, dA, LQ_F32, r, K, r, N);
        g.Bp = dH; g.sb_k = r; g.sb_j = 1; g.beta = accumulate;
        lq_launch_simt_gemm(g, st);
    }
    if (dB) {  // dB = s * H^T . dY
        LqSimtArgs g = simt_base(H, LQ_F32, 1, r, dB, LQ_F32, M, r, M, N);
        g.Bp = dY; g.b_dtype = dtype; g.sb_k = M; g.sb_j = 1; g.alpha = s; g.beta = accumulate;
        lq_launch_simt_gemm(g, st);
    }
}

}  // namespace

// Lets entry points defined in other translation units report through lq_last_error().
void lq_set_last_error(const std::string& msg) { g_last_error = msg; }

// ---- exported symbols ---------------------------------------------------------------

extern "C" {

const char* lq_last_error(void) { return g_last_error.c_str(); }
int lq_abi_version(void) { return LQ_ABI_VERSION; }

int lq_dequant_chunk_rows(uint64_t d_out, uint64_t d_in, uint64_t chunk_bytes, uint64_t* rows, size_t cap,
                          size_t* n_chunks) {
    return guarded([&] {
        LQ_CHECK_ARG(n_chunks != nullptr, "n_chunks is NULL");
        // crates/loractl-core/src/quant.rs:102-117
        uint64_t full = d_out * d_in * 4;
        std::vector<uint64_t> out;
        if (chunk_bytes == 0 || full <= chunk_bytes || d_out <= 1) {
            out.push_back(d_out);
        } else {
            uint64_t row_bytes = d_in * 4;
            uint64_t max_rows = chunk_bytes / row_bytes;
            if (max_rows < 1) max_rows = 1;
            uint64_t n = (d_out + max_rows - 1) / max_rows;
            uint64_t base = d_out / n, rem = d_out % n;
            for (uint64_t i = 0; i < n; ++i) out.push_back(i < rem ? base + 1 : base);
        }
        *n_chunks = out.size();
        if (rows)
            for (size_t i = 0; i < out.size() && i < cap; ++i) rows[i] = out[i];
    });
}

int lq_quantize(const void* w, int w_dtype, int64_t d_out, int64_t d_in, int group, int bits, void* stream,
                lq_weight_t** out) {
    return guarded([&] {
        LQ_CHECK_ARG(out != nullptr, "out is NULL");
        *out = nullptr;
        LQ_CHECK_ARG(w != nullptr, "weight pointer is NULL");
        LQ_CHECK_ARG(w_dtype == LQ_F32 || w_dtype == LQ_BF16, "w_dtype must be LQ_F32 or LQ_BF16");
        check_int_scheme(d_out, d_in, group, bits);
        auto h = new_handle(bits == 4 ? LQ_INT4 : LQ_INT8, d_out, d_in, group, LQ_SCALE_SCALAR);
        try {
            lq_launch_quantize(w, w_dtype, h.get(), bits, (cudaStream_t)stream);
        } catch (...) {
            free_handle(h.release());
            throw;
        }
        *out = h.release();
    });
}

int lq_quantize_from_fp8(const uint8_t* bytes, const float* scale, int scale_kind, int64_t d_out, int64_t d_in, int group,
                         int bits, void* stream, lq_weight_t** out) {
    return guarded([&] {
        LQ_CHECK_ARG(out != nullptr, "out is NULL");
        *out = nullptr;
        LQ_CHECK_ARG(bytes != nullptr && scale != nullptr, "fp8 bytes / weight_scale pointer is NULL");
        LQ_CHECK_ARG(scale_kind == LQ_SCALE_SCALAR || scale_kind == LQ_SCALE_PER_CHANNEL,
                     "weight_scale must be scalar ([] or [1]) or per-out-channel ([out_features])");
        check_int_scheme(d_out, d_in, group, bits);
        auto h = new_handle(bits == 4 ? LQ_INT4 : LQ_INT8, d_out, d_in, group, LQ_SCALE_SCALAR);
        try {
            lq_launch_quantize_fp8(bytes, scale, scale_kind == LQ_SCALE_PER_CHANNEL, h.get(), bits, (cudaStream_t)stream);
        } catch (...) {
            free_handle(h.release());
            throw;
        }
        *out = h.release();
    });
}

int lq_weight_from_codes(const int8_t* codes, const float* scales, int64_t d_out, int64_t d_in, int group, int bits,
                         void* stream, lq_weight_t** out) {
    return guarded([&] {
        LQ_CHECK_ARG(out != nullptr, "out is NULL");
        *out = nullptr;
        LQ_CHECK_ARG(codes != nullptr && scales != nullptr, "codes/scales pointer is NULL");
        check_int_scheme(d_out, d_in, group, bits);
        auto h = new_handle(bits == 4 ? LQ_INT4 : LQ_INT8, d_out, d_in, group, LQ_SCALE_SCALAR);
        try {
            lq_launch_pack_codes(codes, scales, h.get(), (cudaStream_t)stream);
        } catch (...) {
            free_handle(h.release());
            throw;
        }
        *out = h.release();
    });
}

int lq_weight_from_fp8(const uint8_t* bytes, const float* scale, int scale_kind, int64_t d_out, int64_t d_in,
                       void* stream, lq_weight_t** out) {
    return guarded([&] {
        LQ_CHECK_ARG(out != nullptr, "out is NULL");
        *out = nullptr;
        LQ_CHECK_ARG(bytes != nullptr && scale != nullptr, "fp8 bytes / weight_scale pointer is NULL");
        LQ_CHECK_ARG(scale_kind == LQ_SCALE_SCALAR || scale_kind == LQ_SCALE_PER_CHANNEL,
                     "weight_scale must be scalar ([] or [1]) or per-out-channel ([out_features])");
        auto h = new_handle(LQ_FP8_E4M3, d_out, d_in, 0, scale_kind);
        cudaStream_t st = (cudaStream_t)stream;
        cudaError_t e = cudaMemcpyAsync(h->packed, bytes, h->packed_bytes, cudaMemcpyDeviceToDevice, st);
        if (e == cudaSuccess) e = cudaMemcpyAsync(h->scales, scale, h->scale_bytes, cudaMemcpyDeviceToDevice, st);
        if (e != cudaSuccess) {
            free_handle(h.release());
            throw LqError(LQ_ERR_CUDA, std::string("copying fp8 storage: ") + cudaGetErrorString(e));
        }
        *out = h.release();
    });
}

int lq_fp8_quantize(const float* w, int64_t d_out, int64_t d_in, int per_channel, void* stream, lq_weight_t** out) {
    return guarded([&] {
        LQ_CHECK_ARG(out != nullptr, "out is NULL");
        *out = nullptr;
        LQ_CHECK_ARG(w != nullptr, "weight pointer is NULL");
        auto h = new_handle(LQ_FP8_E4M3, d_out, d_in, 0, per_channel ? LQ_SCALE_PER_CHANNEL : LQ_SCALE_SCALAR);
        try {
            lq_launch_fp8_quantize(w, d_out, d_in, per_channel, (uint8_t*)h->packed, h->scales, (cudaStream_t)stream);
        } catch (...) {
            free_handle(h.release());
            throw;
        }
        *out = h.release();
    });
}

int lq_weight_set_bias(lq_weight_t* w, const float* bias, void* stream) {
    return guarded([&] {
        LQ_CHECK_ARG(w != nullptr, "weight handle is NULL");
        DeviceGuard dg(w->device);
        if (!bias) {
            LQ_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
            cudaFree(w->bias);
            w->bias = nullptr;
            return;
        }
        if (!w->bias) LQ_CUDA(cudaMalloc((void**)&w->bias, sizeof(float) * (size_t)w->M));
        LQ_CUDA(cudaMemcpyAsync(w->bias, bias, sizeof(float) * (size_t)w->M, cudaMemcpyDeviceToDevice,
                                (cudaStream_t)stream));
    });
}

int lq_weight_info_get(const lq_weight_t* w, lq_weight_info* info) {
    return guarded([&] {
        LQ_CHECK_ARG(w != nullptr && info != nullptr, "NULL argument");
        std::memset(info, 0, sizeof(*info));
        info->d_out = w->M;
        info->d_in = w->K;
        info->scheme = w->scheme;
        info->group = w->group;
        info->scale_kind = w->scale_kind;
        info->has_bias = w->bias != nullptr;
        info->device = w->device;
        info->packed_bytes = w->packed_bytes;
        info->scale_bytes = w->scale_bytes;
    });
}

int lq_weight_destroy(lq_weight_t* w) {
    return guarded([&] {
        if (!w) return;
        DeviceGuard dg(w->device);
        free_handle(w);
    });
}

int lq_unpack(const lq_weight_t* w, int8_t* codes, float* scales, void* stream) {
    return guarded([&] {
        LQ_CHECK_ARG(w != nullptr && codes != nullptr && scales != nullptr, "NULL argument");
        DeviceGuard dg(w->device);
        lq_launch_unpack(w, codes, scales, (cudaStream_t)stream);
    });
}

int lq_dequantize(const lq_weight_t* w, void* out, int out_dtype, void* stream) {
    return guarded([&] {
        LQ_CHECK_ARG(w != nullptr && out != nullptr, "NULL argument");
        LQ_CHECK_ARG(out_dtype == LQ_F32 || out_dtype == LQ_BF16, "out_dtype must be LQ_F32 or LQ_BF16");
        DeviceGuard dg(w->device);
        lq_launch_dequant(w, out, out_dtype, w->K, 0, (cudaStream_t)stream);
    });
}

size_t lq_linear_workspace_bytes(const lq_weight_t* w, int64_t n_tokens, int rank, int dtype) {
    if (!w || n_tokens < 0 || rank < 0) return 0;
    Carver c(nullptr, 0);
    if (dtype == LQ_BF16_W8A8)
        return lq_w8a8_supported(w, n_tokens, rank) ? align256(lq_w8a8_workspace_bytes(w, n_tokens, rank)) + 256 : 0;
    if (dtype == LQ_BF16 && lq_tc_supported(w, n_tokens, rank)) {
        size_t need = lq_tc_workspace_bytes(w, n_tokens, rank);  // backward (and forward for N > 64)
        if (lq_fused_supported(w, n_tokens, rank)) need = std::max(need, lq_fused_workspace_bytes(w, n_tokens, rank));
        if (lq_small_bwd_supported(w, n_tokens, rank)) need = std::max(need, lq_small_bwd_workspace_bytes(w, n_tokens, rank));
        return align256(need) + 256;
    }
    c.take(sizeof(float) * (size_t)n_tokens * (size_t)(rank > 0 ? rank : 1));  // H
    c.take(sizeof(float) * (size_t)n_tokens * (size_t)(rank > 0 ? rank : 1));  // dH
    return align256(c.used) + 256;
}

size_t lq_weight_bf16_copy_bytes(const lq_weight_t* w) { return w ? (size_t)w->M * (size_t)w->K * 2 : 0; }

int lq_weight_attach_bf16_copy(lq_weight_t* w, void* buffer, void* stream) {
    return guarded([&] {
        LQ_CHECK_ARG(w != nullptr, "weight handle is NULL");
        if (!buffer) {  // detach: per-call dequantisation again
            w->bf16_copy = nullptr;
            return;
        }
        LQ_CHECK_ARG(((uintptr_t)buffer & 15) == 0, "bf16 copy must be 16-byte aligned");
        LQ_CHECK_ARG(w->K % 8 == 0, "bf16 copy needs d_in % 8 == 0 (16-byte rows)");
        DeviceGuard dg(w->device);
        lq_launch_dequant(w, buffer, LQ_BF16, w->K, 0, (cudaStream_t)stream);
        w->bf16_copy = buffer;
    });
}

size_t lq_lora_mirror_bytes(int64_t d_in, int64_t d_out, int rank) {
    if (d_in <= 0 || d_out <= 0 || rank <= 0 || rank > 256) return 0;
    return lq_tc_mirror_bytes(d_in, d_out, rank);
}

int lq_lora_mirror_update(const float* A, const float* B, int64_t d_in, int64_t d_out, int rank, void* mirror,
                          void* stream) {
    return guarded([&] {
        LQ_CHECK_ARG(A && B && mirror, "NULL argument");
        LQ_CHECK_ARG(d_in > 0 && d_out > 0 && rank >= 1 && rank <= 256, "d_in, d_out must be positive and rank in [1, 256]");
        LQ_CHECK_ARG(((uintptr_t)mirror & 255) == 0, "mirror must be 256-byte aligned");
        int dev = 0;
        LQ_CUDA(cudaGetDevice(&dev));
        check_sm100(dev);
        lq_tc_mirror_build(A, B, d_in, d_out, rank, mirror, (cudaStream_t)stream);
    });
}

int lq_lora_mirror_update_batch(const lq_mirror_job* jobs, int n_jobs, void* stream) {
    return guarded([&] {
        LQ_CHECK_ARG(n_jobs >= 0 && (n_jobs == 0 || jobs != nullptr), "jobs is NULL");
        for (int i = 0; i < n_jobs; ++i) {
            const lq_mirror_job& q = jobs[i];
            LQ_CHECK_ARG(q.A && q.B && q.mirror, "NULL pointer in a mirror job");
            LQ_CHECK_ARG(q.d_in > 0 && q.d_out > 0 && q.rank >= 1 && q.rank <= 256,
                         "d_in, d_out must be positive and rank in [1, 256]");
            LQ_CHECK_ARG(((uintptr_t)q.mirror & 255) == 0, "mirror must be 256-byte aligned");
        }
        if (n_jobs == 0) return;
        int dev = 0;
        LQ_CUDA(cudaGetDevice(&dev));
        check_sm100(dev);
        lq_tc_mirror_build_batch(jobs, n_jobs, (cudaStream_t)stream);
    });
}

int lq_linear_fwd(const lq_weight_t* w, const void* X, int64_t n_tokens, int dtype, const float* A, const float* B,
                  int rank, float scaling, void* Y, float* H_out, void* workspace, size_t workspace_bytes,
                  void* stream, const void* lora_mirror) {
    return guarded([&] {
        check_call(w, n_tokens, dtype, A, B, rank);
        LQ_CHECK_ARG(n_tokens == 0 || (X != nullptr && Y != nullptr), "X / Y pointer is NULL");
        if (n_tokens == 0) return;
        DeviceGuard dg(w->device);
        cudaStream_t st = (cudaStream_t)stream;
        if (dtype == LQ_BF16_W8A8) {
            lq_w8a8_fwd(w, X, n_tokens, A, B, rank, scaling, Y, H_out, workspace, workspace_bytes, st);
            return;
        }
        if (dtype == LQ_BF16 && lq_fused_supported(w, n_tokens, rank)) {
            // packed-weight-stream regime: the weight is converted on chip, no bf16 weight in HBM
            lq_fused_fwd(w, X, n_tokens, A, B, rank, scaling, Y, H_out, workspace, workspace_bytes, st);
            return;
        }
        if (dtype == LQ_BF16 && lq_tc_supported(w, n_tokens, rank)) {
            LQ_CHECK_ARG(((uintptr_t)lora_mirror & 255) == 0, "lora_mirror must be 256-byte aligned");
            lq_tc_fwd(w, X, n_tokens, A, B, rank, scaling, Y, H_out, workspace, workspace_bytes, st,
                      rank > 0 ? lora_mirror : nullptr);
            return;
        }
        LQ_CHECK_ARG(rank == 0 || workspace != nullptr || H_out != nullptr, "workspace is NULL");
        Carver c(workspace ? workspace : (void*)H_out, workspace ? workspace_bytes : ~size_t(0));
        float* H = H_out;
        if (rank > 0 && !H) H = (float*)c.take(sizeof(float) * (size_t)n_tokens * rank);
        fwd_simt(w, X, n_tokens, dtype, A, B, rank, scaling, Y, H, st);
    });
}

int lq_linear_bwd(const lq_weight_t* w, const void* dY, const void* X, const float* H, int64_t n_tokens, int dtype,
                  const float* A, const float* B, int rank, float scaling, void* dX, float* dA, float* dB,
                  int accumulate, void* workspace, size_t workspace_bytes, void* stream, const void* lora_mirror) {
    return guarded([&] {
        check_call(w, n_tokens, dtype, A, B, rank);
        if (n_tokens == 0) {
            // Empty batch: gradients of an empty sum are zero.
            DeviceGuard dg(w->device);
            if (rank > 0 && !accumulate) {
                if (dA) LQ_CUDA(cudaMemsetAsync(dA, 0, sizeof(float) * (size_t)w->K * rank, (cudaStream_t)stream));
                if (dB) LQ_CUDA(cudaMemsetAsync(dB, 0, sizeof(float) * (size_t)w->M * rank, (cudaStream_t)stream));
            }
            return;
        }
        LQ_CHECK_ARG(dY != nullptr, "dY pointer is NULL");
        LQ_CHECK_ARG(rank == 0 || X != nullptr, "X is needed for the LoRA gradients");
        DeviceGuard dg(w->device);
        cudaStream_t st = (cudaStream_t)stream;
        if (dtype == LQ_BF16_W8A8) {
            lq_w8a8_bwd(w, dY, X, H, n_tokens, A, B, rank, scaling, dX, dA, dB, accumulate, workspace, workspace_bytes,
                        st);
            return;
        }
        if (dtype == LQ_BF16 && lq_tc_supported(w, n_tokens, rank) && lq_small_bwd_supported(w, n_tokens, rank)) {
            // packed-weight-stream regime of the backward: no bf16 image of W^T is written
            lq_small_bwd(w, dY, X, H, n_tokens, A, B, rank, scaling, dX, dA, dB, accumulate, workspace, workspace_bytes,
                         st);
            return;
        }
        if (dtype == LQ_BF16 && lq_tc_supported(w, n_tokens, rank)) {
            LQ_CHECK_ARG(((uintptr_t)lora_mirror & 255) == 0, "lora_mirror must be 256-byte aligned");
            lq_tc_bwd(w, dY, X, H, n_tokens, A, B, rank, scaling, dX, dA, dB, accumulate, workspace, workspace_bytes,
                      st, rank > 0 ? lora_mirror : nullptr);
            return;
        }
        LQ_CHECK_ARG(rank == 0 || workspace != nullptr, "workspace is NULL");
        Carver c(workspace, workspace_bytes);
        float* Hbuf = nullptr;
        float* dH = nullptr;
        if (rank > 0) {
            Hbuf = (float*)c.take(sizeof(float) * (size_t)n_tokens * rank);
            dH = (float*)c.take(sizeof(float) * (size_t)n_tokens * rank);
        }
        const float* Huse = H;
        if (rank > 0 && !H && dB) {  // recompute H = X . A
            LqSimtArgs h = simt_base(X, dtype, w->K, 1, Hbuf, LQ_F32, rank, n_tokens, rank, w->K);
            h.Bp = A; h.sb_k = rank; h.sb_j = 1;
            lq_launch_simt_gemm(h, st);
            Huse = Hbuf;
        }
        bwd_simt(w, dY, X, Huse, n_tokens, dtype, A, B, rank, scaling, dX, dA, dB, accumulate, dH, st);
    });
}

size_t lq_linear_grouped_workspace_bytes(const lq_group_site* sites, int n_sites, int64_t n_tokens, int dtype) {
    if (!sites || n_sites < 1 || n_tokens < 0) return 0;
    if (dtype == LQ_BF16 && lq_fused_group_supported(sites, n_sites, n_tokens))
        return align256(lq_fused_group_workspace_bytes(sites, n_sites, n_tokens)) + 256;
    size_t need = 0;
    for (int i = 0; i < n_sites; ++i) need = std::max(need, lq_linear_workspace_bytes(sites[i].w, n_tokens, sites[i].rank, dtype));
    return need;
}

int lq_linear_fwd_grouped(const lq_group_site* sites, int n_sites, const void* X, int64_t n_tokens, int dtype,
                          void* workspace, size_t workspace_bytes, void* stream) {
    int rc = guarded([&] {
        LQ_CHECK_ARG(sites != nullptr && n_sites >= 1, "no sites");
        for (int i = 0; i < n_sites; ++i) {
            check_call(sites[i].w, n_tokens, dtype, sites[i].A, sites[i].B, sites[i].rank);
            LQ_CHECK_ARG(sites[i].w->K == sites[0].w->K, "the sites of a group share X: their d_in must agree");
        }
        LQ_CHECK_ARG(n_tokens == 0 || X != nullptr, "X pointer is NULL");
    });
    if (rc != LQ_OK || n_tokens == 0) return rc;
    if (dtype == LQ_BF16 && lq_fused_group_supported(sites, n_sites, n_tokens)) {
        return guarded([&] {
            DeviceGuard dg(sites[0].w->device);
            lq_fused_fwd_grouped(sites, n_sites, X, n_tokens, workspace, workspace_bytes, (cudaStream_t)stream);
        });
    }
    for (int i = 0; i < n_sites; ++i) {  // one after the other; the stream orders their use of the workspace
        rc = lq_linear_fwd(sites[i].w, X, n_tokens, dtype, sites[i].A, sites[i].B, sites[i].rank, sites[i].scaling,
                           sites[i].Y, sites[i].H_out, workspace, workspace_bytes, stream, nullptr);
        if (rc != LQ_OK) return rc;
    }
    return LQ_OK;
}

int lq_weight_prepare_fp8_backward(const lq_weight_t* w, void* stream) {
    return guarded([&] {
        LQ_CHECK_ARG(w != nullptr, "weight handle is NULL");
        LQ_CHECK_ARG(w->scheme == LQ_FP8_E4M3, "only scaled-fp8 weights have an fp8 backward operand");
        DeviceGuard dg(w->device);
        lq_w8a8_prepare_backward(w, (cudaStream_t)stream);
    });
}

int lq_check_device_status(void* stream) {
    return guarded([&] {
        int dev = 0;
        LQ_CUDA(cudaGetDevice(&dev));
        int code = lq_tc_read_status(dev, (cudaStream_t)stream);
        if (code != 0)
            throw LqError(LQ_ERR_TIMEOUT, "a kernel's bounded wait gave up (wait site " + std::to_string(code) +
                                              "); its outputs are invalid");
    });
}

int lq_selftest_bounded_wait(unsigned limit_ms, void* stream) {
    return guarded([&] {
        LQ_CHECK_ARG(limit_ms >= 1 && limit_ms <= 1000, "limit_ms must be in [1, 1000]");
        int dev = 0;
        LQ_CUDA(cudaGetDevice(&dev));
        check_sm100(dev);
        lq_tc_selftest_wait(dev, limit_ms, (cudaStream_t)stream);
    });
}

int lq_option_set(const char* name, int value) {
    return guarded([&] {
        LQ_CHECK_ARG(name != nullptr, "option name is NULL");
        if (!lq_w4_option_set(name, value) && !lq_tc_option_set(name, value))
            throw LqError(LQ_ERR_INVALID, std::string("unknown option '") + name + "' (known: w4, w4_exact, bwd_mn, tail_split, reserve_sms)");
    });
}

int lq_gemm_bf16(const void* A, int a_mn, int64_t lda, const void* B, int b_mn, int64_t ldb, void* C, int c_dtype,
                 int64_t ldc, int64_t Mg, int64_t Ng, int64_t Kg, int block_n, int splits, float* partial_ws,
                 const float* bias, void* stream) {
    return guarded([&] {
        LQ_CHECK_ARG(A && B && C, "NULL operand");
        LQ_CHECK_ARG(Mg > 0 && Ng > 0 && Kg > 0, "gemm dims must be positive");
        LQ_CHECK_ARG(c_dtype == LQ_F32 || c_dtype == LQ_BF16, "c_dtype must be LQ_F32 or LQ_BF16");
        LQ_CHECK_ARG(splits >= 1 && splits <= 64, "splits must be in [1, 64]");
        int dev = 0;
        LQ_CUDA(cudaGetDevice(&dev));
        check_sm100(dev);
        lq_tc_gemm_bf16(A, a_mn, lda, B, b_mn, ldb, C, c_dtype, ldc, Mg, Ng, Kg, block_n, splits, partial_ws, bias,
                        (cudaStream_t)stream);
    });
}

}  // extern "C"
