#include "lq_prof.cuh"

#include <atomic>
#include <mutex>
#include <utility>
#include <vector>

#include "lq_internal.cuh"

namespace {
std::atomic<uint64_t> g_launches[LQ_K_COUNT];
std::atomic<int> g_enabled{0};
std::mutex g_mu;
std::vector<std::pair<cudaEvent_t, cudaEvent_t>> g_events[LQ_K_COUNT];
thread_local cudaEvent_t t_open = nullptr;
}  // namespace

void lq_prof_begin(int kind, cudaStream_t st) {
    g_launches[kind].fetch_add(1, std::memory_order_relaxed);
    if (!g_enabled.load(std::memory_order_relaxed)) return;
    cudaEvent_t e = nullptr;
    if (cudaEventCreate(&e) != cudaSuccess) return;
    cudaEventRecord(e, st);
    t_open = e;
}

void lq_prof_end(int kind, cudaStream_t st) {
    if (!t_open) return;
    cudaEvent_t b = t_open, e = nullptr;
    t_open = nullptr;
    if (cudaEventCreate(&e) != cudaSuccess) {
        cudaEventDestroy(b);
        return;
    }
    cudaEventRecord(e, st);
    std::lock_guard<std::mutex> lk(g_mu);
    g_events[kind].emplace_back(b, e);
}

extern "C" {

uint64_t lq_kernel_launch_count(void) {
    uint64_t n = 0;
    for (int k = 0; k < LQ_K_COUNT; ++k) n += g_launches[k].load(std::memory_order_relaxed);
    return n;
}

int lq_profile_enable(int on) {
    g_enabled.store(on ? 1 : 0);
    return LQ_OK;
}

int lq_profile_kinds(void) { return LQ_K_COUNT; }

const char* lq_profile_kind_name(int kind) {
    static const char* names[LQ_K_COUNT] = {"quantize", "dequant", "prep", "gemm_main", "gemm_down",
                                            "gemm_grad", "reduce", "simt_gemm"};
    return (kind >= 0 && kind < LQ_K_COUNT) ? names[kind] : "";
}

int lq_profile_collect(double* ms_by_kind, uint64_t* timed_by_kind, int n_kinds) {
    if (cudaDeviceSynchronize() != cudaSuccess) return LQ_ERR_CUDA;
    std::lock_guard<std::mutex> lk(g_mu);
    for (int k = 0; k < LQ_K_COUNT; ++k) {
        double ms = 0.0;
        uint64_t n = 0;
        for (auto& pr : g_events[k]) {
            float t = 0.f;
            if (cudaEventElapsedTime(&t, pr.first, pr.second) == cudaSuccess) {
                ms += t;
                ++n;
            }
            cudaEventDestroy(pr.first);
            cudaEventDestroy(pr.second);
        }
        g_events[k].clear();
        if (k < n_kinds) {
            if (ms_by_kind) ms_by_kind[k] = ms;
            if (timed_by_kind) timed_by_kind[k] = n;
        }
    }
    return LQ_OK;
}
}
