// Per-device runtime state, tensor-map encoding, the kernel registry bridge and
// the symbol-addressed / extension C entry points.
//
// Replaces the process-global workspace of PyC's CUDA backend
// (src/compiler/runtime/cuda_backend.c:137-180: three device buffers, cuBLAS
// handles, one stream, one captured graph behind one global mutex) with one
// context per device, and the registration code of
// src/compiler/cutlass_kernels/registry/init.cu:32-92.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <fcntl.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/file.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <map>
#include <mutex>
#include <string>
#include <tuple>
#include <vector>

#include "internal.h"
#include "ptx_sm100.cuh"
#include "runtime.h"

// PyC's kernel registry (src/compiler/runtime/kernel_registry.c) is looked up at run time in the process's global symbol
// scope: present when this library sits next to PyC's front half (linked together, or both loaded RTLD_GLOBAL, in either
// order), absent stand-alone.
#include <dlfcn.h>
namespace {
struct PycRegistryApi {
    int (*reg)(const pyc_kernel_desc*) = nullptr;
    size_t (*collect)(const char*, pyc_backend, pyc_kernel_desc*, size_t) = nullptr;
    int (*promote)(const char*, pyc_backend, const char*) = nullptr;
    int (*promoted)(const char*, pyc_backend, char*, size_t) = nullptr;
    int (*bench_update)(const char*, pyc_backend, const char*, double) = nullptr;
    int (*coselect)(const char*, pyc_backend, pyc_objective_mode, const pyc_kernel_coselect_context*, pyc_kernel_desc*, pyc_kernel_selection_trace*) = nullptr;
};
// Resolved again on every call until PyC's registry shows up (it may be loaded after this library).
const PycRegistryApi& pyc_registry() {
    static PycRegistryApi api;
    static std::mutex mu;
    std::lock_guard<std::mutex> lk(mu);
    if (!api.reg) {
        void* f = dlsym(RTLD_DEFAULT, "pyc_kernel_register");
        if (f) {
            *reinterpret_cast<void**>(&api.reg) = f;
            *reinterpret_cast<void**>(&api.collect) = dlsym(RTLD_DEFAULT, "pyc_kernel_collect");
            *reinterpret_cast<void**>(&api.promote) = dlsym(RTLD_DEFAULT, "pyc_kernel_promote_symbol");
            *reinterpret_cast<void**>(&api.promoted) = dlsym(RTLD_DEFAULT, "pyc_kernel_promoted_symbol");
            *reinterpret_cast<void**>(&api.bench_update) = dlsym(RTLD_DEFAULT, "pyc_kernel_benchmark_update_symbol");
            *reinterpret_cast<void**>(&api.coselect) = dlsym(RTLD_DEFAULT, "pyc_kernel_coselect_with_context");
        }
    }
    return api;
}
}  // namespace

namespace b200 {

// ------------------------------------------------------------------ errors --
static thread_local char g_err[512] = "";
void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}
const char* last_error() { return g_err; }

static std::atomic<size_t> g_launches{0};
void count_launch(size_t n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
size_t launches_total() { return g_launches.load(std::memory_order_relaxed); }

// ---------------------------------------------------------------- contexts --
static std::mutex g_ctx_mu;
static DeviceContext* g_ctx[kMaxDevices] = {};

DeviceContext* current_context() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        cudaGetLastError();
        set_error("no usable CUDA device");
        return nullptr;
    }
    std::lock_guard<std::mutex> lk(g_ctx_mu);
    if (g_ctx[dev]) return g_ctx[dev];
    DeviceContext* c = new DeviceContext();
    c->device = dev;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, dev) != cudaSuccess) { cudaGetLastError(); delete c; set_error("cudaGetDeviceProperties failed"); return nullptr; }
    c->sm_count = prop.multiProcessorCount;
    c->cc_major = prop.major;
    c->cc_minor = prop.minor;
    if (cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking) != cudaSuccess ||
        cudaMalloc(&c->status_dev, 256) != cudaSuccess ||
        cudaMemset(c->status_dev, 0, 256) != cudaSuccess ||
        cudaMallocHost(&c->status_host, 256) != cudaSuccess) {
        set_error("context setup failed: %s", cudaGetErrorString(cudaGetLastError()));
        delete c;
        return nullptr;
    }
    *c->status_host = 0;
    g_ctx[dev] = c;
    return c;
}

int sm_count() {
    DeviceContext* c = current_context();
    return c ? c->sm_count : 148;
}
int* device_status_word() {
    DeviceContext* c = current_context();
    return c ? c->status_dev : nullptr;
}
int read_device_status(cudaStream_t stream) {
    DeviceContext* c = current_context();
    if (!c) return -1;
    if (cudaMemcpyAsync(c->status_host, c->status_dev, sizeof(int), cudaMemcpyDeviceToHost, stream) != cudaSuccess) return -1;
    if (cudaStreamSynchronize(stream) != cudaSuccess) return -1;
    const int st = *c->status_host;
    if (st != 0) {  // read-and-clear, so one timed-out wait is reported once
        cudaMemsetAsync(c->status_dev, 0, sizeof(int), stream);
        cudaStreamSynchronize(stream);
        *c->status_host = 0;
    }
    return st;
}

int DeviceContext::ensure_arena(size_t bytes) {
    if (bytes <= arena_bytes) return 0;
    // Grow-only, like PyC's workspace (cuda_backend.c:303-420); cached graphs hold arena addresses.
    drop_graphs();
    if (arena) cudaFree(arena);
    arena = nullptr; arena_bytes = 0;
    size_t want = (bytes + (size_t(1) << 20) - 1) & ~((size_t(1) << 20) - 1);
    B200_CUDA_OK(cudaMalloc(&arena, want));
    arena_bytes = want;
    return 0;
}
int DeviceContext::ensure_pinned(size_t bytes) {
    if (bytes <= pinned_bytes) return 0;
    drop_graphs();
    if (pinned) cudaFreeHost(pinned);
    pinned = nullptr; pinned_bytes = 0;
    size_t want = (bytes + (size_t(1) << 20) - 1) & ~((size_t(1) << 20) - 1);
    B200_CUDA_OK(cudaMallocHost(&pinned, want));
    pinned_bytes = want;
    return 0;
}
int DeviceContext::ensure_pipeline(size_t event_count) {
    if (!copy_in) B200_CUDA_OK(cudaStreamCreateWithFlags(&copy_in, cudaStreamNonBlocking));
    if (!copy_out) B200_CUDA_OK(cudaStreamCreateWithFlags(&copy_out, cudaStreamNonBlocking));
    while (events.size() < event_count) {
        cudaEvent_t e = nullptr;
        B200_CUDA_OK(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
        events.push_back(e);
    }
    return 0;
}
void DeviceContext::drop_graphs() {
    for (auto& kv : graphs) {
        if (kv.second.exec) cudaGraphExecDestroy(kv.second.exec);
    }
    graphs.clear();
}

// ------------------------------------------------------------- tensor maps --
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
        else
            cudaGetLastError();
    });
    return fn;
}

int encode_tmap(CUtensorMap* out, const void* base, int elem_bytes, int rank, const uint64_t* dims,
                const uint64_t* strides_bytes, const uint32_t* box, bool swizzle128) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) { set_error("cuTensorMapEncodeTiled is not available from this driver"); return -1; }
    if (reinterpret_cast<uintptr_t>(base) % 16 != 0) { set_error("tensor map: base address not 16-byte aligned"); return -1; }
    cuuint64_t gdim[5]; cuuint64_t gstr[4]; cuuint32_t bx[5]; cuuint32_t es[5];
    for (int i = 0; i < rank; ++i) { gdim[i] = dims[i]; bx[i] = box[i]; es[i] = 1; }
    for (int i = 0; i + 1 < rank; ++i) {
        if (strides_bytes[i] % 16 != 0) { set_error("tensor map: stride %llu not a multiple of 16 bytes", (unsigned long long)strides_bytes[i]); return -1; }
        gstr[i] = strides_bytes[i];
    }
    const CUtensorMapDataType dt = elem_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_UINT16 : CU_TENSOR_MAP_DATA_TYPE_UINT32;
    const CUresult r = fn(out, dt, static_cast<cuuint32_t>(rank), const_cast<void*>(base), gdim, gstr, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled failed with code %d", static_cast<int>(r)); return -1; }
    return 0;
}

int encode_tmap_2d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t rows, uint64_t cols,
                   uint64_t row_stride_bytes, uint32_t box_rows, uint32_t box_cols) {
    const uint64_t dims[2] = {cols, rows};
    const uint64_t strides[1] = {row_stride_bytes};
    const uint32_t box[2] = {box_cols, box_rows};
    return encode_tmap(out, base, elem_bytes, 2, dims, strides, box, true);
}

// ---------------------------------------------------------------- registry --
struct RegEntry {
    pyc_kernel_desc desc;
    double best_ms;
};
// Function-local statics: registration runs from a load-time constructor, which may
// come before this file's namespace-scope objects are constructed.
struct RegState {
    std::mutex mu;
    std::vector<RegEntry> entries;
    std::map<std::string, std::string> promoted;  // op_key -> symbol (stand-alone mode)
    bool done = false;
    bool mirrored = false;   // entries copied into PyC's registry (which may be loaded after this library)
};
static RegState& reg_state() { static RegState* s = new RegState(); return *s; }
#define g_reg_mu (reg_state().mu)
#define g_reg (reg_state().entries)
#define g_promoted (reg_state().promoted)
#define g_reg_done (reg_state().done)

// Priorities are TIERS, not a ranking: PyC's score is priority * 100 + affinities (+36 for a matching workload family,
// -18 for a different one) - 100 * best measured ms (kernel_registry.c:48-57, 125-158), so any priority step outweighs
// every measurement.  All tensor-core tiles therefore share one priority and their declared workload family plus the
// measured times decide between them; the SIMT tiles sit in a lower tier (fp32, or 16-bit shapes TMA cannot take).
static const GemmConfig kGemmConfigs[] = {
    // symbol suffix           kind       dtypes                                     bm   bn   bk  st  prio  smem    workload
    {"tc2_256x256x64_s6", GEMM_TC_PAIR, (1 << PYC_DTYPE_BF16) | (1 << PYC_DTYPE_F16), 256, 256, 64, 6, 100, 230576, PYC_KERNEL_WORKLOAD_LARGE_SQUARE},
    {"tc2_256x256x64_s7", GEMM_TC_PAIR, (1 << PYC_DTYPE_BF16) | (1 << PYC_DTYPE_F16), 256, 256, 64, 7, 100, 230560, PYC_KERNEL_WORKLOAD_LARGE_SQUARE},
    {"tc_128x256x64_s4", GEMM_TC, (1 << PYC_DTYPE_BF16) | (1 << PYC_DTYPE_F16), 128, 256, 64, 4, 100, 197744, PYC_KERNEL_WORKLOAD_SQUARE},
    {"tc_128x128x64_s6", GEMM_TC, (1 << PYC_DTYPE_BF16) | (1 << PYC_DTYPE_F16), 128, 128, 64, 6, 100, 197776, PYC_KERNEL_WORKLOAD_TALL_SKINNY},
    {"tc_128x64x64_s8", GEMM_TC, (1 << PYC_DTYPE_BF16) | (1 << PYC_DTYPE_F16), 128, 64, 64, 8, 100, 197808, PYC_KERNEL_WORKLOAD_SMALL},
    {"simt_x2_128x128x32", GEMM_SIMT, (1 << PYC_DTYPE_F32), 128, 128, 32, 2, 30, 66560, PYC_KERNEL_WORKLOAD_LARGE_SQUARE},
    {"simt_128x128x16", GEMM_SIMT, (1 << PYC_DTYPE_F32) | (1 << PYC_DTYPE_BF16) | (1 << PYC_DTYPE_F16), 128, 128, 16, 2, 30, 33792, PYC_KERNEL_WORKLOAD_LARGE_SQUARE},
    {"simt_64x64x16", GEMM_SIMT, (1 << PYC_DTYPE_F32) | (1 << PYC_DTYPE_BF16) | (1 << PYC_DTYPE_F16), 64, 64, 16, 2, 30, 17408, PYC_KERNEL_WORKLOAD_SQUARE},
    {"simt_async_32x64x32", GEMM_SIMT, (1 << PYC_DTYPE_F32), 32, 64, 32, 3, 30, 38400, PYC_KERNEL_WORKLOAD_SMALL},
    {"simt_32x64x16", GEMM_SIMT, (1 << PYC_DTYPE_F32) | (1 << PYC_DTYPE_BF16) | (1 << PYC_DTYPE_F16), 32, 64, 16, 2, 20, 13312, PYC_KERNEL_WORKLOAD_SMALL},
};
const GemmConfig* gemm_configs(int* count) {
    *count = static_cast<int>(sizeof(kGemmConfigs) / sizeof(kGemmConfigs[0]));
    return kGemmConfigs;
}
static const char* dtype_token(pyc_dtype d) { return d == PYC_DTYPE_F32 ? "f32" : d == PYC_DTYPE_BF16 ? "bf16" : d == PYC_DTYPE_F16 ? "f16" : "?"; }
std::string gemm_symbol(pyc_dtype d, const GemmConfig& c) { return std::string("b200_gemm_") + dtype_token(d) + "_" + c.symbol; }

// "b200_gemm_<dtype>_<suffix>" -> (dtype, config)
static const GemmConfig* parse_gemm_symbol(const char* symbol, pyc_dtype* dt) {
    static const char kPrefix[] = "b200_gemm_";
    if (strncmp(symbol, kPrefix, sizeof(kPrefix) - 1) != 0) return nullptr;
    const char* rest = symbol + sizeof(kPrefix) - 1;
    const pyc_dtype cands[3] = {PYC_DTYPE_F32, PYC_DTYPE_BF16, PYC_DTYPE_F16};
    for (pyc_dtype d : cands) {
        const char* tok = dtype_token(d);
        const size_t n = strlen(tok);
        if (strncmp(rest, tok, n) == 0 && rest[n] == '_') {
            for (const GemmConfig& c : kGemmConfigs)
                if (strcmp(rest + n + 1, c.symbol) == 0 && (c.dtype_mask & (1 << d))) { *dt = d; return &c; }
        }
    }
    return nullptr;
}
const GemmConfig* find_gemm_config(const char* symbol) {
    pyc_dtype d;
    return parse_gemm_symbol(symbol, &d);
}

static void reg_add(const char* op_key, const std::string& symbol, int priority, double occ, int tc, size_t smem, int regclass,
                    pyc_kernel_workload_family wf) {
    RegEntry e;
    memset(&e, 0, sizeof(e));
    strncpy(e.desc.op_key, op_key, PYC_KERNEL_OP_KEY_MAX - 1);
    strncpy(e.desc.symbol, symbol.c_str(), PYC_KERNEL_SYMBOL_MAX - 1);
    e.desc.backend = PYC_BACKEND_CUDA;
    e.desc.priority = priority;
    e.desc.estimated_occupancy = occ;
    e.desc.tensor_core_eligible = tc;
    e.desc.shared_mem_bytes = smem;
    e.desc.reg_pressure_class = regclass;
    e.desc.preferred_workload_family = wf;
    // PyC's enum stops at HOPPER and maps compute capability >= 9 to it
    // (cuda_backend.c:279-285), so that is the family a B200 reports.
    e.desc.preferred_hardware_family = PYC_KERNEL_HARDWARE_HOPPER;
    e.best_ms = 0.0;
    g_reg.push_back(e);
    
}

static void registry_fill_locked();
// Mirror this library's descriptors (and a PYC_PROMOTED_GEMM_SYMBOL promotion) into PyC's registry once it is reachable.
static void registry_mirror_locked() {
    RegState& st = reg_state();
    if (st.mirrored || !pyc_registry().reg) return;
    st.mirrored = true;
    for (const RegEntry& e : st.entries) pyc_registry().reg(&e.desc);
    auto it = st.promoted.find("matmul");
    if (it != st.promoted.end() && pyc_registry().promote) pyc_registry().promote("matmul", PYC_BACKEND_CUDA, it->second.c_str());
    if (pyc_registry().bench_update)
        for (const RegEntry& e : st.entries) if (e.best_ms > 0.0) pyc_registry().bench_update(e.desc.op_key, PYC_BACKEND_CUDA, e.desc.symbol, e.best_ms);
}
void registry_init_once() {
    bool first = false;
    {
        std::lock_guard<std::mutex> lk(g_reg_mu);
        if (!g_reg_done) { g_reg_done = true; first = true; registry_fill_locked(); }
        registry_mirror_locked();
    }
    // Timings and per-shape winners persisted by an earlier process (PYC_AUTOTUNE_DB_PATH); outside the lock because
    // loading reports timings through the registry.
    if (first) autotune_db_load(nullptr);
}
static void registry_fill_locked() {
    for (const GemmConfig& c : kGemmConfigs) {
        const pyc_dtype cands[3] = {PYC_DTYPE_BF16, PYC_DTYPE_F16, PYC_DTYPE_F32};
        for (pyc_dtype d : cands) {
            if (!(c.dtype_mask & (1 << d))) continue;
            // One CTA per SM (persistent) for the tensor-core kernels; SIMT tiles run 2-4 CTAs per SM.
            int prio = c.priority;
            if (c.kind == GEMM_SIMT && d != PYC_DTYPE_F32) prio -= 5;  // any-shape path for 16-bit types
            // PyC adds 6 x estimated occupancy to a score and breaks exact ties by symbol name: the packed-FMA tile gets
            // a slightly higher estimate than the scalar tile of the same shape, priority and workload family, so that it
            // is the one proposed for large fp32 problems (when it cannot take a problem the next check falls through).
            const double occ = c.kind != GEMM_SIMT ? 0.09 : (c.bm == 128 && c.bk == 32) ? 0.55 : 0.5;
            reg_add("matmul", gemm_symbol(d, c), prio, occ, c.kind != GEMM_SIMT ? 1 : 0, c.smem_bytes,
                    c.kind != GEMM_SIMT ? 2 : 1, c.workload);
            // The same descriptor under a dtype-qualified key: PyC's selection returns ONE winner per op key, and a
            // winner of another dtype is of no use to a GEMM that has to run now.
            reg_add((std::string("matmul.") + dtype_token(d)).c_str(), gemm_symbol(d, c), prio, occ,
                    c.kind != GEMM_SIMT ? 1 : 0, c.smem_bytes, c.kind != GEMM_SIMT ? 2 : 1, c.workload);
        }
    }
    reg_add("conv2d", "b200_conv2d_fprop_bf16", 100, 0.09, 1, 197744, 2, PYC_KERNEL_WORKLOAD_ANY);
    reg_add("conv2d", "b200_conv2d_fprop_f16", 90, 0.09, 1, 197744, 2, PYC_KERNEL_WORKLOAD_ANY);
    reg_add("attention", "b200_attention_bf16", 100, 0.09, 1, 200000, 3, PYC_KERNEL_WORKLOAD_ANY);
    reg_add("attention", "b200_attention_bf16_causal", 95, 0.09, 1, 200000, 3, PYC_KERNEL_WORKLOAD_ANY);
    reg_add("attention", "b200_attention_f16", 90, 0.09, 1, 200000, 3, PYC_KERNEL_WORKLOAD_ANY);
    reg_add("attention", "b200_attention_f16_causal", 85, 0.09, 1, 200000, 3, PYC_KERNEL_WORKLOAD_ANY);

    const char* promoted = getenv("PYC_PROMOTED_GEMM_SYMBOL");
    if (promoted && promoted[0]) {
        bool known = false;
        for (const RegEntry& e : g_reg) known = known || (strcmp(e.desc.op_key, "matmul") == 0 && strcmp(e.desc.symbol, promoted) == 0);
        if (known) {
            g_promoted["matmul"] = promoted;

        }
    }
}

int registry_count(const char* op_key) {
    registry_init_once();
    if (!op_key) return 0;
    if (pyc_registry().collect) {
        std::vector<pyc_kernel_desc> tmp(PYC_KERNEL_MAX);
        return static_cast<int>(pyc_registry().collect(op_key, PYC_BACKEND_CUDA, tmp.data(), tmp.size()));
    }
    std::lock_guard<std::mutex> lk(g_reg_mu);
    int n = 0;
    for (const RegEntry& e : g_reg) n += strcmp(e.desc.op_key, op_key) == 0;
    return n;
}

bool registry_promoted_symbol(const char* op_key, std::string* out) {
    registry_init_once();
    if (pyc_registry().promoted) {
        char buf[PYC_KERNEL_SYMBOL_MAX] = "";
        if (pyc_registry().promoted(op_key, PYC_BACKEND_CUDA, buf, sizeof(buf)) == 0 && buf[0]) { *out = buf; return true; }
    }
    std::lock_guard<std::mutex> lk(g_reg_mu);
    auto it = g_promoted.find(op_key);
    if (it == g_promoted.end()) return false;
    *out = it->second;
    return true;
}

void registry_report_ms(const char* op_key, const char* symbol, double ms) {
    registry_init_once();
    {
        std::lock_guard<std::mutex> lk(g_reg_mu);
        for (RegEntry& e : g_reg)
            if (strcmp(e.desc.op_key, op_key) == 0 && strcmp(e.desc.symbol, symbol) == 0 && (e.best_ms == 0.0 || ms < e.best_ms)) e.best_ms = ms;
    }
    if (auto update = pyc_registry().bench_update) {
        update(op_key, PYC_BACKEND_CUDA, symbol, ms);
        // GEMM kernels are also registered under "matmul.<dtype>" (the key the backend's own selection asks for)
        pyc_dtype d;
        if (strcmp(op_key, "matmul") == 0 && parse_gemm_symbol(symbol, &d))
            update((std::string("matmul.") + dtype_token(d)).c_str(), PYC_BACKEND_CUDA, symbol, ms);
    }
}

// ------------------------------------------------------- GEMM config choice --
// Who picks the tile configuration of a GEMM, in this order:
//   1. a measured winner for exactly this (dtype, M, N, K): autotuned in this process or read from the autotune DB;
//   2. PYC_CUDA_BF16_GEMM_SYMBOL for bf16 problems (PyC: cuda_backend.c:671-699) when it names one of this library's
//      kernels (PyC's legacy name "cutlass_gemm_tensorcore_bf16" means "the default");
//   3. the symbol promoted in the kernel registry (PYC_PROMOTED_GEMM_SYMBOL, pyc_kernel_promote_symbol), unless
//      PYC_CUDA_ENABLE_PROMOTED_GEMM is set to 0/false (PyC: cuda_backend.c:2640-2645 consults the promotion only when
//      that switch is on; here a promotion is honoured by default and the switch can turn it off);
//   4. PyC's own scoring, pyc_kernel_coselect_with_context (kernel_registry.c:374-454), asked for the dtype-qualified
//      key with the workload family PyC derives from M, N, K (compiler_api.c:1141-1170) and the device's hardware
//      family, when PyC's registry is linked into the process.  Its proposal is taken unless the wave-count model below
//      puts it more than 25 % behind the model's own best (the registry knows families, not wave quantisation);
//      PYC_B200_REGISTRY_SELECT=0 skips this step;
//   5. the wave-count model.
// Function-local (heap) singletons: the autotune DB is read from the load-time constructor, which can run before this
// file's namespace-scope objects are constructed.
struct WinnerState {
    std::mutex mu;
    std::map<std::tuple<int, int, int, int>, const GemmConfig*> winners;
};
static WinnerState& winner_state() { static WinnerState* s = new WinnerState(); return *s; }
#define g_win_mu (winner_state().mu)
#define g_winners (winner_state().winners)
static std::atomic<uint64_t> g_selection_epoch{1};
static thread_local char g_selection_source[32] = "";

uint64_t selection_epoch() { return g_selection_epoch.load(std::memory_order_relaxed); }
const char* last_selection_source() { return g_selection_source; }
static void note_source(const char* s) { strncpy(g_selection_source, s, sizeof(g_selection_source) - 1); g_selection_source[sizeof(g_selection_source) - 1] = 0; }

void remember_gemm_winner(pyc_dtype dtype, int M, int N, int K, const GemmConfig* cfg) {
    std::lock_guard<std::mutex> lk(g_win_mu);
    const GemmConfig*& slot = g_winners[std::make_tuple(static_cast<int>(dtype), M, N, K)];
    if (slot != cfg) g_selection_epoch.fetch_add(1, std::memory_order_relaxed);   // graphs captured with the old choice go stale
    slot = cfg;
}

bool gemm_config_supports(const GemmConfig& cfg, const GemmProblem& p) {
    if (!(cfg.dtype_mask & (1 << p.dtype))) return false;
    if (cfg.kind == GEMM_SIMT) {
        if (cfg.bk == 32)  // the cp.async tiles (latency tile, packed-FMA tile): 16-byte loads of row-major operands
            return !p.b_col_major && p.K % 4 == 0 && p.N % 4 == 0 && reinterpret_cast<uintptr_t>(p.A) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(p.B) % 16 == 0 && reinterpret_cast<uintptr_t>(p.D) % 16 == 0;
        return true;
    }
    // TMA: 16-byte aligned bases and row strides.
    if (p.K % 8 != 0) return false;
    if (!p.b_col_major && p.N % 8 != 0) return false;
    if (reinterpret_cast<uintptr_t>(p.A) % 16 || reinterpret_cast<uintptr_t>(p.B) % 16) return false;
    DeviceContext* c = current_context();
    return c && c->cc_major == 10;
}

// Relative efficiency of the CTA-pair tile in the wave-count model (the 128x256 single-CTA tile is 1.0).
// Measured on 8192^3: 1450-1499 TFLOP/s against 1434-1472 for the single-CTA tile.
static constexpr double kPairEfficiency = 1.02;

// Estimated time of `c` on `p` in arbitrary units: waves * tile work / relative efficiency of the tile.
static double model_cost(const GemmConfig& c, const GemmProblem& p, int sms) {
    const double tiles = static_cast<double>((p.M + c.bm - 1) / c.bm) * ((p.N + c.bn - 1) / c.bn);
    double eff, slots;
    if (c.kind == GEMM_TC) { eff = c.bn == 256 ? 1.0 : c.bn == 128 ? 0.85 : 0.6; slots = sms; }
    else if (c.kind == GEMM_TC_PAIR) { eff = kPairEfficiency; slots = sms / 2; }
    else { eff = ((c.bm == 128 && c.bk == 32) ? 2.7 : c.bm == 128 ? 1.0 : c.bm == 64 ? 0.8 : c.bk == 32 ? 0.75 : 0.55) / 24.0; slots = sms * (c.bm == 128 ? 2.0 : 4.0); }  // packed-FMA tile: 51 TFLOP/s measured against 30 for 64 x 64
    const double waves = static_cast<double>(static_cast<long long>((tiles + slots - 1) / slots));
    return waves * c.bm * c.bn / eff / (c.kind == GEMM_TC_PAIR ? 2.0 : 1.0);  // a pair tile is the work of two SMs
}

// PyC's workload classes (compiler_api.c:1141-1170), restated: the registry's affinity scores are keyed on them.
pyc_kernel_workload_family matmul_workload_family(size_t m, size_t n, size_t k) {
    if (m == 0 || n == 0 || k == 0) return PYC_KERNEL_WORKLOAD_ANY;
    const size_t major = m > n ? m : n, minor = m < n ? m : n;
    if (major <= 512 || m * n * k <= static_cast<size_t>(512) * 512 * 512) return PYC_KERNEL_WORKLOAD_SMALL;
    if (m >= n * 3) return PYC_KERNEL_WORKLOAD_TALL_SKINNY;
    if (n >= m * 3) return PYC_KERNEL_WORKLOAD_WIDE_SKINNY;
    if (minor >= 1024 && major <= minor * 2 && k >= 512) return PYC_KERNEL_WORKLOAD_LARGE_SQUARE;
    return PYC_KERNEL_WORKLOAD_SQUARE;
}

static bool env_is_false(const char* name) {
    const char* v = getenv(name);
    return v && (!strcmp(v, "0") || !strcmp(v, "false") || !strcmp(v, "FALSE"));
}

const GemmConfig* choose_gemm_config(const GemmProblem& p) {
    {
        std::lock_guard<std::mutex> lk(g_win_mu);
        auto it = g_winners.find(std::make_tuple(static_cast<int>(p.dtype), p.M, p.N, p.K));
        if (it != g_winners.end() && gemm_config_supports(*it->second, p)) { note_source("autotune"); return it->second; }
    }
    if (p.dtype == PYC_DTYPE_BF16) {
        const char* forced = getenv("PYC_CUDA_BF16_GEMM_SYMBOL");
        if (forced && forced[0]) {
            pyc_dtype d;
            const GemmConfig* c = parse_gemm_symbol(forced, &d);
            if (c && d == p.dtype && gemm_config_supports(*c, p)) { note_source("env"); return c; }
        }
    }
    if (!env_is_false("PYC_CUDA_ENABLE_PROMOTED_GEMM")) {
        std::string promoted;
        if (registry_promoted_symbol("matmul", &promoted)) {
            pyc_dtype d;
            const GemmConfig* c = parse_gemm_symbol(promoted.c_str(), &d);
            if (c && d == p.dtype && gemm_config_supports(*c, p)) { note_source("promoted"); return c; }
        }
    }
    const int sms = sm_count();
    const GemmConfig* best = nullptr;
    double best_cost = 0.0;
    for (const GemmConfig& c : kGemmConfigs) {
        if (!gemm_config_supports(c, p)) continue;
        const double cost = model_cost(c, p, sms);
        if (!best || cost < best_cost) { best = &c; best_cost = cost; }
    }
    if (best && pyc_registry().coselect && !env_is_false("PYC_B200_REGISTRY_SELECT")) {
        registry_init_once();
        pyc_kernel_coselect_context ctx;
        memset(&ctx, 0, sizeof(ctx));
        ctx.workload_family = matmul_workload_family(static_cast<size_t>(p.M), static_cast<size_t>(p.N), static_cast<size_t>(p.K));
        ctx.hardware_family = pyc_cuda_current_hardware_family();
        pyc_kernel_desc pick;
        pyc_kernel_selection_trace tr;
        const std::string key = std::string("matmul.") + dtype_token(p.dtype);
        if (pyc_registry().coselect(key.c_str(), PYC_BACKEND_CUDA, PYC_MODE_BALANCED, &ctx, &pick, &tr) == 0) {
            pyc_dtype d;
            const GemmConfig* c = parse_gemm_symbol(pick.symbol, &d);
            if (c && d == p.dtype && gemm_config_supports(*c, p) && model_cost(*c, p, sms) <= 1.25 * best_cost) { note_source("registry"); return c; }
        }
    }
    note_source("model");
    return best;
}

int launch_gemm(const GemmConfig& cfg, const GemmProblem& p, cudaStream_t stream) {
    if (p.M <= 0 || p.N <= 0 || p.K <= 0 || !p.A || !p.B || !p.D) { set_error("gemm: bad shape or NULL pointer"); return -1; }
    if (!gemm_config_supports(cfg, p)) { set_error("gemm: configuration %s does not support this dtype/shape/alignment", cfg.symbol); return -1; }
    if (cfg.kind == GEMM_TC || cfg.kind == GEMM_TC_PAIR) {
        int* st = device_status_word();
        if (!st) return -1;
        return cfg.kind == GEMM_TC ? launch_gemm_tc(cfg, p, stream, st) : launch_gemm_tc_pair(cfg, p, stream, st);
    }
    return launch_gemm_simt(cfg, p, stream);
}

bool has_gemm_winner(pyc_dtype dtype, int M, int N, int K) {
    std::lock_guard<std::mutex> lk(g_win_mu);
    return g_winners.count(std::make_tuple(static_cast<int>(dtype), M, N, K)) != 0;
}

// ------------------------------------------------------------ autotune DB --
// Persisted timings, in the line format of PyC's autotune DB (compiler_api.c:2145-2305: "op|backend|symbol|best_ms",
// writers serialised by flock on "<path>.lock", the file compacted to one line per (op, backend, symbol) keeping the
// smallest time).  Two kinds of line are written for every timed configuration:
//     matmul|1|<symbol>|<ms>                          what PyC's own loader feeds to its registry (per symbol)
//     matmul@<dtype>:<M>x<N>x<K>|1|<symbol>|<ms>      the same timing keyed by shape: the fastest symbol of a shape
//                                                     becomes that shape's winner in the next process
// PyC's loader skips op keys it does not ask for, so both kinds live in one file.  The path is PYC_AUTOTUNE_DB_PATH
// (compiler_api.c:2124-2143); without it nothing is read or written.
struct DbLine { std::string op, symbol; int backend; double ms; };

static bool parse_db_line(const char* line, DbLine* out) {
    char op[PYC_KERNEL_OP_KEY_MAX], sym[PYC_KERNEL_SYMBOL_MAX];
    int backend = 0; double ms = 0.0;
    if (sscanf(line, "%63[^|]|%d|%127[^|]|%lf", op, &backend, sym, &ms) != 4 || ms <= 0.0) return false;
    out->op = op; out->symbol = sym; out->backend = backend; out->ms = ms;
    return true;
}

static std::string shape_key(pyc_dtype dtype, int M, int N, int K) {
    char buf[PYC_KERNEL_OP_KEY_MAX];
    snprintf(buf, sizeof(buf), "matmul@%s:%dx%dx%d", dtype_token(dtype), M, N, K);
    return buf;
}

static const char* autotune_db_path() {
    const char* p = getenv("PYC_AUTOTUNE_DB_PATH");
    return p && p[0] ? p : nullptr;
}

// Append `lines`, then compact, all under the lock file.
static int db_append(const char* path, const std::vector<DbLine>& lines) {
    const std::string lock_path = std::string(path) + ".lock";
    const int fd = open(lock_path.c_str(), O_CREAT | O_RDWR, 0644);
    if (fd < 0) { set_error("autotune DB: cannot open %s", lock_path.c_str()); return -1; }
    if (flock(fd, LOCK_EX) != 0) { close(fd); set_error("autotune DB: flock failed"); return -1; }
    std::vector<DbLine> all;
    if (FILE* in = fopen(path, "r")) {
        char buf[512];
        DbLine l;
        while (fgets(buf, sizeof(buf), in)) if (parse_db_line(buf, &l)) all.push_back(l);
        fclose(in);
    }
    for (const DbLine& l : lines) all.push_back(l);
    std::vector<DbLine> kept;
    for (const DbLine& l : all) {
        bool found = false;
        for (DbLine& k : kept)
            if (k.op == l.op && k.backend == l.backend && k.symbol == l.symbol) { if (l.ms < k.ms) k.ms = l.ms; found = true; break; }
        if (!found) kept.push_back(l);
    }
    int rc = 0;
    const std::string tmp = std::string(path) + ".tmp";
    if (FILE* out = fopen(tmp.c_str(), "w")) {
        for (const DbLine& k : kept) if (fprintf(out, "%s|%d|%s|%.6f\n", k.op.c_str(), k.backend, k.symbol.c_str(), k.ms) < 0) rc = -1;
        if (fclose(out) != 0) rc = -1;
        if (rc == 0 && rename(tmp.c_str(), path) != 0) rc = -1;
    } else rc = -1;
    if (rc != 0) set_error("autotune DB: cannot write %s", path);
    flock(fd, LOCK_UN);
    close(fd);
    return rc;
}

// Read the DB: per-symbol timings go to the registry, the fastest symbol of every shape key becomes that shape's winner.
// Returns the number of shape winners installed (0 when there is no file), -1 on a NULL path.
int autotune_db_load(const char* path) {
    if (!path) path = autotune_db_path();
    if (!path) return -1;
    FILE* in = fopen(path, "r");
    if (!in) return 0;
    std::map<std::string, std::pair<std::string, double>> best;   // shape key -> (symbol, ms)
    char buf[512];
    DbLine l;
    while (fgets(buf, sizeof(buf), in)) {
        if (!parse_db_line(buf, &l) || l.backend != static_cast<int>(PYC_BACKEND_CUDA)) continue;
        if (l.op == "matmul") { registry_report_ms("matmul", l.symbol.c_str(), l.ms); continue; }
        if (l.op.compare(0, 7, "matmul@") != 0) continue;
        auto it = best.find(l.op);
        if (it == best.end() || l.ms < it->second.second) best[l.op] = std::make_pair(l.symbol, l.ms);
    }
    fclose(in);
    int installed = 0;
    for (const auto& kv : best) {
        char tok[8]; int M = 0, N = 0, K = 0;
        if (sscanf(kv.first.c_str(), "matmul@%7[^:]:%dx%dx%d", tok, &M, &N, &K) != 4) continue;
        pyc_dtype d;
        const GemmConfig* c = parse_gemm_symbol(kv.second.first.c_str(), &d);
        if (!c || strcmp(dtype_token(d), tok) != 0 || M <= 0 || N <= 0 || K <= 0) continue;
        remember_gemm_winner(d, M, N, K, c);
        ++installed;
    }
    return installed;
}

// ------------------------------------------------------- wait self-test ------
// One CTA waits on an mbarrier that nobody arrives at, with a limit of `limit_cycles`: the wait gives up by itself,
// records ST_WAIT_TIMEOUT with site 0x7f in the device status word and the kernel returns.  This is the path every
// kernel's bounded waits take when a producer never shows up, exercised without making anything hang.
__global__ void wait_selftest_kernel(int* status, long long limit_cycles) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        fence_barrier_init();
        mbar_wait(smem_u32(&bar), 0, status, 0x7f, limit_cycles);
    }
}

// ------------------------------------------------------------- autotune ------
// Operands for timing: values ~ N(0, 0.02^2) (sum of four uniforms, counter-based hash of the element index), so that the
// tensor cores toggle as they do on real activations/weights.  All-zero operands draw less power and clock higher on a
// power-capped part, which can reorder tile configurations that are within a few percent of each other.
__global__ void autotune_fill_kernel(void* dst, size_t n, int dtype, uint32_t seed, float std) {
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n; i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        uint64_t z = (i + 1) * 0x9E3779B97F4A7C15ull + seed;
        z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull; z = (z ^ (z >> 27)) * 0x94D049BB133111EBull; z ^= z >> 31;
        float s = 0.0f;
#pragma unroll
        for (int k = 0; k < 4; ++k) s += static_cast<float>((z >> (16 * k)) & 0xffff) * (1.0f / 65536.0f);
        const float v = (s - 2.0f) * 1.7320508f * std;    // variance of the sum of four U(0,1) is 1/3
        if (dtype == PYC_DTYPE_F32) static_cast<float*>(dst)[i] = v;
        else if (dtype == PYC_DTYPE_BF16) static_cast<unsigned short*>(dst)[i] = static_cast<unsigned short>((__float_as_uint(v) + 0x7fffu + ((__float_as_uint(v) >> 16) & 1u)) >> 16);
        else static_cast<unsigned short*>(dst)[i] = __half_as_ushort(__float2half_rn(v));
    }
}

// Times every tile configuration that supports (dtype, M, N, K) on the context's stream with CUDA events (median of
// `iters` >= 5 launches, with the epilogue that will run: add_mode / act), remembers the fastest, feeds every timing to
// the registry and, when PYC_AUTOTUNE_DB_PATH is set, to the autotune DB.  The caller holds ctx->mu.  Must not be called
// while a stream capture is open (it allocates and synchronises).
int autotune_gemm_unlocked(DeviceContext* ctx, pyc_dtype dtype, int M, int N, int K, int iters, std::string* best_symbol, double* best_ms,
                           int add_mode, int act) {
    if (!ctx || M <= 0 || N <= 0 || K <= 0) return -1;
    if (iters < 5) iters = 5;
    const size_t es = dtype_size(dtype);
    if (!es) { set_error("autotune: unsupported dtype"); return -1; }
    void *A = nullptr, *B = nullptr, *D = nullptr, *C = nullptr;
    const size_t add_elems = add_mode == PYC_B200_ADD_MATRIX ? static_cast<size_t>(M) * N : add_mode == PYC_B200_ADD_ROW_BIAS ? N : add_mode == PYC_B200_ADD_SCALAR ? 1 : 0;
    if (cudaMalloc(&A, es * M * K) != cudaSuccess || cudaMalloc(&B, es * K * N) != cudaSuccess || cudaMalloc(&D, es * M * N) != cudaSuccess ||
        (add_elems && cudaMalloc(&C, es * add_elems + 16) != cudaSuccess)) {
        cudaGetLastError(); cudaFree(A); cudaFree(B); cudaFree(D); cudaFree(C); set_error("autotune: out of device memory"); return -1;
    }
    autotune_fill_kernel<<<1024, 256, 0, ctx->stream>>>(A, static_cast<size_t>(M) * K, dtype, 0x5EEDA001u, 0.02f);
    autotune_fill_kernel<<<1024, 256, 0, ctx->stream>>>(B, static_cast<size_t>(K) * N, dtype, 0x5EEDA002u, 0.02f);
    if (add_elems) autotune_fill_kernel<<<64, 256, 0, ctx->stream>>>(C, add_elems, dtype, 0x5EEDA003u, 0.02f);
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0); cudaEventCreate(&e1);
    GemmProblem p;
    p.dtype = dtype; p.M = M; p.N = N; p.K = K; p.A = A; p.B = B; p.D = D;
    p.add_mode = add_elems ? add_mode : PYC_B200_ADD_NONE; p.add = C; p.act = act;
    int timed = 0;
    const GemmConfig* best = nullptr;
    double best_t = 0.0;
    int n = 0;
    const GemmConfig* cfgs = gemm_configs(&n);
    std::vector<DbLine> lines;
    std::vector<float> samples(iters);
    for (int i = 0; i < n; ++i) {
        if (!gemm_config_supports(cfgs[i], p)) continue;
        // The SIMT tiles are only worth timing for fp32 or when no tensor-core tile fits.
        if (cfgs[i].kind == GEMM_SIMT && dtype != PYC_DTYPE_F32 && best) continue;
        if (launch_gemm(cfgs[i], p, ctx->stream) != 0) continue;  // warm-up
        bool ok = true;
        for (int it = 0; it < iters && ok; ++it) {
            cudaEventRecord(e0, ctx->stream);
            launch_gemm(cfgs[i], p, ctx->stream);
            cudaEventRecord(e1, ctx->stream);
            ok = cudaEventSynchronize(e1) == cudaSuccess;
            if (ok) cudaEventElapsedTime(&samples[it], e0, e1);
        }
        if (!ok) { cudaGetLastError(); continue; }
        std::sort(samples.begin(), samples.end());
        const double t = samples[iters / 2];
        const std::string sym = gemm_symbol(dtype, cfgs[i]);
        registry_report_ms("matmul", sym.c_str(), t);
        lines.push_back({"matmul", sym, static_cast<int>(PYC_BACKEND_CUDA), t});
        lines.push_back({shape_key(dtype, M, N, K), sym, static_cast<int>(PYC_BACKEND_CUDA), t});
        ++timed;
        if (!best || t < best_t) { best = &cfgs[i]; best_t = t; }
    }
    cudaEventDestroy(e0); cudaEventDestroy(e1);
    cudaFree(A); cudaFree(B); cudaFree(D); cudaFree(C);
    if (!best) { set_error("autotune: no configuration ran"); return -1; }
    remember_gemm_winner(dtype, M, N, K, best);
    if (const char* path = autotune_db_path()) db_append(path, lines);   // a DB that cannot be written does not fail the tuning
    if (best_symbol) *best_symbol = gemm_symbol(dtype, *best);
    if (best_ms) *best_ms = best_t;
    return timed;
}

}  // namespace b200

// ======================================================================== C API
using namespace b200;

extern "C" {

void pyc_cutlass_registry_init(void) { registry_init_once(); }

__attribute__((constructor)) static void b200_auto_register(void) { registry_init_once(); }

int pyc_cutlass_kernel_count(const char* op_key) { return registry_count(op_key); }

const char* pyc_b200_last_error(void) { return last_error(); }

int pyc_cutlass_gemm_dispatch(const char* symbol, int M, int N, int K, const void* A, const void* B, void* C,
                              float alpha, float beta, void* stream) {
    if (!symbol) return -1;
    GemmProblem p;
    p.M = M; p.N = N; p.K = K; p.A = A; p.B = B; p.D = C; p.alpha = alpha;
    if (beta != 0.0f) { p.add_mode = PYC_B200_ADD_MATRIX; p.add = C; p.add_scale = beta; }
    const GemmConfig* cfg = nullptr;
    pyc_dtype dt = PYC_DTYPE_UNKNOWN;
    if ((cfg = parse_gemm_symbol(symbol, &dt)) != nullptr) {
        p.dtype = dt;
    } else if (strcmp(symbol, "cutlass_gemm_tensorcore_bf16") == 0) {
        p.dtype = PYC_DTYPE_BF16;
    } else if (strcmp(symbol, "cutlass_gemm_tensorcore_f16") == 0) {
        p.dtype = PYC_DTYPE_F16; p.b_col_major = true;  // RowMajor x ColumnMajor, gemm/kernel.cu:48-65
    } else if (strcmp(symbol, "cutlass_gemm_simt_f32") == 0 || strcmp(symbol, "ada_gemm_k64_warp32_async_f32") == 0) {
        p.dtype = PYC_DTYPE_F32;
    } else {
        set_error("unknown GEMM symbol %s", symbol);
        return -1;
    }
    if (!cfg) cfg = choose_gemm_config(p);
    if (!cfg) { set_error("no GEMM configuration for this problem"); return -1; }
    return launch_gemm(*cfg, p, static_cast<cudaStream_t>(stream));
}

int pyc_b200_gemm(const pyc_b200_gemm_args* a, void* stream) {
    if (!a) return -1;
    GemmProblem p;
    p.dtype = a->dtype; p.M = a->M; p.N = a->N; p.K = a->K; p.A = a->A; p.B = a->B; p.D = a->D;
    p.b_col_major = a->b_col_major != 0; p.alpha = a->alpha; p.add_mode = a->add_mode; p.add = a->add; p.act = a->act;
    const GemmConfig* cfg = nullptr;
    if (a->symbol && a->symbol[0]) {
        pyc_dtype dt;
        cfg = parse_gemm_symbol(a->symbol, &dt);
        if (!cfg || dt != a->dtype) { set_error("GEMM symbol %s does not exist for this dtype", a->symbol); return -1; }
    } else {
        cfg = choose_gemm_config(p);
    }
    if (!cfg) { set_error("no GEMM configuration for this problem"); return -1; }
    return launch_gemm(*cfg, p, static_cast<cudaStream_t>(stream));
}

int pyc_b200_add(pyc_dtype dtype, const void* a, const void* b, void* out, size_t elems, void* stream) {
    return launch_add(dtype, a, b, out, elems, static_cast<cudaStream_t>(stream));
}
int pyc_b200_bias_act(pyc_dtype dtype, const void* x, const void* add, pyc_b200_add_mode add_mode, pyc_b200_activation act,
                      void* out, size_t rows, size_t cols, void* stream) {
    return launch_bias_act(dtype, x, add, add_mode, act, out, rows, cols, static_cast<cudaStream_t>(stream));
}
int pyc_b200_layernorm(pyc_dtype dtype, const void* x, const void* gamma, const void* beta, void* out, size_t rows, size_t cols,
                       float eps, void* stream) {
    return launch_layernorm(dtype, x, gamma, beta, out, rows, cols, eps, static_cast<cudaStream_t>(stream));
}
int pyc_b200_softmax(pyc_dtype dtype, const void* x, void* out, size_t rows, size_t cols, void* stream) {
    return launch_softmax(dtype, x, out, rows, cols, static_cast<cudaStream_t>(stream));
}
int pyc_b200_reduce_sum(pyc_dtype dtype, const void* x, void* out, size_t rows, size_t cols, void* stream) {
    return launch_reduce_sum(dtype, x, out, rows, cols, static_cast<cudaStream_t>(stream));
}

int pyc_b200_autotune_gemm(pyc_dtype dtype, int M, int N, int K, int iters, char* best_symbol, size_t best_symbol_size, double* best_ms) {
    DeviceContext* ctx = current_context();
    if (!ctx) return -1;
    std::lock_guard<std::mutex> lk(ctx->mu);
    std::string best;
    double ms = 0.0;
    const int n = autotune_gemm_unlocked(ctx, dtype, M, N, K, iters, &best, &ms);
    if (n < 0) return -1;
    if (best_symbol && best_symbol_size) { strncpy(best_symbol, best.c_str(), best_symbol_size - 1); best_symbol[best_symbol_size - 1] = 0; }
    if (best_ms) *best_ms = ms;
    return n;
}

int pyc_b200_autotune_db_load(const char* path) { return autotune_db_load(path); }

int pyc_b200_selftest_wait_timeout(int limit_us, void* stream) {
    DeviceContext* c = current_context();
    if (!c) return -1;
    if (limit_us < 1 || limit_us > 1000000) { set_error("wait self-test: limit must be 1 .. 1000000 us"); return -1; }
    wait_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(c->status_dev, static_cast<long long>(limit_us) * 2000);   // ~2 GHz
    B200_CUDA_OK(cudaGetLastError());
    return 0;
}

int pyc_b200_get_runtime_info(pyc_b200_runtime_info* out) {
    if (!out) return -1;
    memset(out, 0, sizeof(*out));
    out->kernel_launches_total = launches_total();
    DeviceContext* c = current_context();
    if (!c) return -1;
    std::lock_guard<std::mutex> lk(c->mu);
    out->arena_bytes = c->arena_bytes;
    out->plan_peak_bytes = c->last_plan_peak;
    out->plan_total_bytes = c->last_plan_total;
    out->graphs_cached = c->graphs.size();
    out->graph_replays = c->graph_replays;
    out->kernels_per_graph = c->last_graph_kernels;
    return 0;
}

int pyc_b200_set_stream(void* stream, int async) {
    DeviceContext* c = current_context();
    if (!c) return -1;
    std::lock_guard<std::mutex> lk(c->mu);
    c->user_stream = static_cast<cudaStream_t>(stream);
    c->use_user_stream = stream != nullptr || async != 0;
    c->async = async != 0;
    return 0;
}

int pyc_b200_device_status(void) {
    DeviceContext* c = current_context();
    if (!c) return -1;
    std::lock_guard<std::mutex> lk(c->mu);
    return read_device_status(c->stream);
}

void pyc_b200_shutdown(void) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) { cudaGetLastError(); return; }
    DeviceContext* c = nullptr;
    {
        std::lock_guard<std::mutex> lk(g_ctx_mu);
        c = g_ctx[dev];
        g_ctx[dev] = nullptr;
    }
    if (!c) return;
    cudaDeviceSynchronize();
    c->drop_graphs();
    if (c->arena) cudaFree(c->arena);
    if (c->pinned) cudaFreeHost(c->pinned);
    if (c->status_dev) cudaFree(c->status_dev);
    if (c->status_host) cudaFreeHost(c->status_host);
    for (cudaEvent_t e : c->events) cudaEventDestroy(e);
    if (c->copy_in) cudaStreamDestroy(c->copy_in);
    if (c->copy_out) cudaStreamDestroy(c->copy_out);
    if (c->stream) cudaStreamDestroy(c->stream);
    delete c;
}

}  // extern "C"
