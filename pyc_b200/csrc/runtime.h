// Per-device context of the backend: stream, status word, device arena, pinned
// staging buffer, CUDA-graph cache.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "internal.h"

namespace b200 {

constexpr int kMaxDevices = 16;

struct CachedGraph {
    cudaGraphExec_t exec = nullptr;
    size_t kernels = 0;
    size_t replays = 0;
    uint64_t check = 0;           // second hash of the key material, compared on every hit
    std::shared_ptr<void> plan;   // the dispatch layer's step list for this key (opaque here)
};

struct DeviceContext {
    int device = 0;
    int sm_count = 148;
    int cc_major = 0, cc_minor = 0;
    std::mutex mu;                 // serialises dispatch on this device
    cudaStream_t stream = nullptr; // private non-blocking stream
    cudaStream_t user_stream = nullptr;
    bool use_user_stream = false;
    bool async = false;
    int* status_dev = nullptr;     // device status word written by kernels on a timed-out wait
    int* status_host = nullptr;    // pinned mirror
    void* arena = nullptr;         // single device arena; the lifetime plan hands out offsets
    size_t arena_bytes = 0;
    void* pinned = nullptr;        // host staging for host-pointer tensors
    size_t pinned_bytes = 0;
    // Side streams + events for the host-tensor pipeline (uploads, kernels and downloads of one call overlap).
    cudaStream_t copy_in = nullptr, copy_out = nullptr;
    std::vector<cudaEvent_t> events;
    std::map<uint64_t, CachedGraph> graphs;
    size_t graph_replays = 0;
    uint64_t last_base = 0;      // module+descriptor hash of the previous run
    uint64_t resident_base = 0;  // hash whose static host operands are still in the arena
    size_t last_plan_peak = 0, last_plan_total = 0, last_graph_kernels = 0;

    int ensure_arena(size_t bytes);
    int ensure_pinned(size_t bytes);
    int ensure_pipeline(size_t event_count);
    void drop_graphs();
    cudaStream_t active_stream() const { return use_user_stream ? user_stream : stream; }
};

DeviceContext* current_context();
std::string gemm_symbol(pyc_dtype d, const GemmConfig& c);
bool has_gemm_winner(pyc_dtype dtype, int M, int N, int K);
int autotune_gemm_unlocked(DeviceContext* ctx, pyc_dtype dtype, int M, int N, int K, int iters, std::string* best_symbol, double* best_ms,
                           int add_mode = PYC_B200_ADD_NONE, int act = PYC_B200_ACT_NONE);

}  // namespace b200
