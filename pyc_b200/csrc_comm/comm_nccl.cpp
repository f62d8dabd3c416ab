// libpyc_b200_comm_nccl.so -- an NCCL backend for PyC's collective interface.
//
// PyC loads collective backends as shared libraries that export pyc_comm_backend_create / pyc_comm_backend_destroy and
// return a pyc_collective_comm vtable (include/pyc/collective_comm.h:30-101, loader
// src/compiler/runtime/comm_backend_loader.c).  PyC's own NCCL shim (src/compiler/runtime/comm_backend_nccl.c) maps only
// I8/I32/F16/F32 (:139-150), so the bf16 partial sums of the tensor-parallel FFN block cannot go through it, and its
// barrier all-reduces a host integer.  This backend is the same interface with
//   * bf16 (ncclBfloat16) and the other PyC dtypes mapped,
//   * a barrier on a device word,
//   * NCCL found at run time (dlopen; an already loaded libnccl.so.2 -- e.g. the one a framework in the process brought --
//     is reused so that one process holds one NCCL), nothing linked at build time,
// plus three bootstrap helpers for a launcher that has no communicator yet (unique id on rank 0, ncclCommInitRank on
// every rank, destroy).  The communicator is passed to every vtable call as the pyc_comm_handle_t, as PyC does with
// "comm_handle" (src/compiler/runtime/distributed_runtime.c:16-42).
//
// config_json keys (all optional): "nccl_library": "<path>"  library to dlopen instead of the default names;
//                                  "strict": true           creation fails when NCCL cannot be loaded.
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <string>

#include "pyc_b200_abi.h"

namespace {

typedef int nccl_result;
typedef void* nccl_comm;
struct NcclId { char bytes[128]; };

struct Ctx {
    void* lib = nullptr;
    bool owns_lib = false;
    nccl_result (*all_reduce)(const void*, void*, size_t, int, int, nccl_comm, cudaStream_t) = nullptr;
    nccl_result (*all_gather)(const void*, void*, size_t, int, nccl_comm, cudaStream_t) = nullptr;
    nccl_result (*reduce_scatter)(const void*, void*, size_t, int, int, nccl_comm, cudaStream_t) = nullptr;
    nccl_result (*broadcast)(const void*, void*, size_t, int, int, nccl_comm, cudaStream_t) = nullptr;
    nccl_result (*send)(const void*, size_t, int, int, nccl_comm, cudaStream_t) = nullptr;
    nccl_result (*recv)(void*, size_t, int, int, nccl_comm, cudaStream_t) = nullptr;
    nccl_result (*get_unique_id)(NcclId*) = nullptr;
    nccl_result (*comm_init_rank)(nccl_comm*, int, NcclId, int) = nullptr;
    nccl_result (*comm_destroy)(nccl_comm) = nullptr;
    const char* (*get_error_string)(nccl_result) = nullptr;
    int* barrier_word[16] = {};     // one device int per device, allocated at the first barrier there
    char last_error[256] = "";
};

bool map_dtype(pyc_dtype d, int* out) {      // ncclDataType_t values
    switch (d) {
        case PYC_DTYPE_I8: *out = 0; return true;      // ncclInt8
        case PYC_DTYPE_I32: *out = 2; return true;     // ncclInt32
        case PYC_DTYPE_F16: *out = 6; return true;     // ncclFloat16
        case PYC_DTYPE_F32: *out = 7; return true;     // ncclFloat32
        case PYC_DTYPE_BF16: *out = 9; return true;    // ncclBfloat16
        default: return false;
    }
}
bool map_op(pyc_reduce_op op, int* out) {    // ncclRedOp_t values
    switch (op) {
        case PYC_REDUCE_SUM: *out = 0; return true;
        case PYC_REDUCE_PROD: *out = 1; return true;
        case PYC_REDUCE_MAX: *out = 2; return true;
        case PYC_REDUCE_MIN: *out = 3; return true;
        case PYC_REDUCE_AVG: *out = 4; return true;
        default: return false;
    }
}

std::string json_string(const char* json, const char* key) {
    if (!json) return "";
    const std::string pat = std::string("\"") + key + "\"";
    const char* k = strstr(json, pat.c_str());
    if (!k) return "";
    const char* c = strchr(k + pat.size(), ':');
    if (!c) return "";
    const char* q0 = strchr(c, '"');
    if (!q0) return "";
    const char* q1 = strchr(q0 + 1, '"');
    if (!q1) return "";
    return std::string(q0 + 1, q1);
}
bool json_true(const char* json, const char* key) {
    if (!json) return false;
    const std::string pat = std::string("\"") + key + "\"";
    const char* k = strstr(json, pat.c_str());
    if (!k) return false;
    const char* c = strchr(k + pat.size(), ':');
    if (!c) return false;
    ++c;
    while (*c == ' ' || *c == '\t') ++c;
    return strncmp(c, "true", 4) == 0 || *c == '1';
}

bool load_nccl(Ctx* ctx, const char* config_json) {
    const std::string wanted = json_string(config_json, "nccl_library");
    const char* env = getenv("PYC_B200_NCCL_LIBRARY");
    void* h = nullptr;
    if (!wanted.empty()) h = dlopen(wanted.c_str(), RTLD_NOW | RTLD_LOCAL);
    else if (env && env[0]) h = dlopen(env, RTLD_NOW | RTLD_LOCAL);
    else {
        h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_LOCAL | RTLD_NOLOAD);     // the one the process already has
        if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_LOCAL);
        if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_LOCAL);
    }
    if (!h) { snprintf(ctx->last_error, sizeof(ctx->last_error), "NCCL not found: %s", dlerror()); return false; }
    ctx->lib = h; ctx->owns_lib = true;
#define LOAD(field, name) *reinterpret_cast<void**>(&ctx->field) = dlsym(h, name)
    LOAD(all_reduce, "ncclAllReduce"); LOAD(all_gather, "ncclAllGather"); LOAD(reduce_scatter, "ncclReduceScatter");
    LOAD(broadcast, "ncclBroadcast"); LOAD(send, "ncclSend"); LOAD(recv, "ncclRecv");
    LOAD(get_unique_id, "ncclGetUniqueId"); LOAD(comm_init_rank, "ncclCommInitRank"); LOAD(comm_destroy, "ncclCommDestroy");
    LOAD(get_error_string, "ncclGetErrorString");
#undef LOAD
    return ctx->all_reduce && ctx->all_gather && ctx->reduce_scatter && ctx->broadcast;
}

pyc_comm_status check(Ctx* ctx, pyc_comm_handle_t comm, size_t count, pyc_dtype dtype, int* nccl_dtype) {
    if (!ctx || !comm || count == 0) return PYC_COMM_ERR_INVALID;
    if (!map_dtype(dtype, nccl_dtype)) return PYC_COMM_ERR_INVALID;
    if (!ctx->lib) return PYC_COMM_ERR_HARDWARE;
    return PYC_COMM_OK;
}
pyc_comm_status result(Ctx* ctx, nccl_result r) {
    if (r == 0) return PYC_COMM_OK;
    snprintf(ctx->last_error, sizeof(ctx->last_error), "NCCL error %d: %s", r, ctx->get_error_string ? ctx->get_error_string(r) : "?");
    return PYC_COMM_ERR_HARDWARE;
}

pyc_comm_status v_all_reduce(void* bc, pyc_comm_handle_t comm, const void* send, void* recv, size_t count, pyc_dtype dtype, pyc_reduce_op op, void* stream) {
    Ctx* ctx = static_cast<Ctx*>(bc);
    int dt = 0, ro = 0;
    const pyc_comm_status st = check(ctx, comm, count, dtype, &dt);
    if (st != PYC_COMM_OK) return st;
    if (!send || !recv || !map_op(op, &ro)) return PYC_COMM_ERR_INVALID;
    return result(ctx, ctx->all_reduce(send, recv, count, dt, ro, comm, static_cast<cudaStream_t>(stream)));
}
pyc_comm_status v_all_gather(void* bc, pyc_comm_handle_t comm, const void* send, void* recv, size_t count, pyc_dtype dtype, void* stream) {
    Ctx* ctx = static_cast<Ctx*>(bc);
    int dt = 0;
    const pyc_comm_status st = check(ctx, comm, count, dtype, &dt);
    if (st != PYC_COMM_OK) return st;
    if (!send || !recv) return PYC_COMM_ERR_INVALID;
    return result(ctx, ctx->all_gather(send, recv, count, dt, comm, static_cast<cudaStream_t>(stream)));
}
pyc_comm_status v_reduce_scatter(void* bc, pyc_comm_handle_t comm, const void* send, void* recv, size_t count, pyc_dtype dtype, pyc_reduce_op op, void* stream) {
    Ctx* ctx = static_cast<Ctx*>(bc);
    int dt = 0, ro = 0;
    const pyc_comm_status st = check(ctx, comm, count, dtype, &dt);
    if (st != PYC_COMM_OK) return st;
    if (!send || !recv || !map_op(op, &ro)) return PYC_COMM_ERR_INVALID;
    return result(ctx, ctx->reduce_scatter(send, recv, count, dt, ro, comm, static_cast<cudaStream_t>(stream)));
}
pyc_comm_status v_broadcast(void* bc, pyc_comm_handle_t comm, const void* send, void* recv, size_t count, pyc_dtype dtype, int root, void* stream) {
    Ctx* ctx = static_cast<Ctx*>(bc);
    int dt = 0;
    const pyc_comm_status st = check(ctx, comm, count, dtype, &dt);
    if (st != PYC_COMM_OK) return st;
    if (!send || !recv || root < 0) return PYC_COMM_ERR_INVALID;
    return result(ctx, ctx->broadcast(send, recv, count, dt, root, comm, static_cast<cudaStream_t>(stream)));
}
pyc_comm_status v_send(void* bc, pyc_comm_handle_t comm, const void* send, size_t count, pyc_dtype dtype, int peer, void* stream) {
    Ctx* ctx = static_cast<Ctx*>(bc);
    int dt = 0;
    const pyc_comm_status st = check(ctx, comm, count, dtype, &dt);
    if (st != PYC_COMM_OK) return st;
    if (!send || peer < 0) return PYC_COMM_ERR_INVALID;
    if (!ctx->send) return PYC_COMM_ERR_HARDWARE;
    return result(ctx, ctx->send(send, count, dt, peer, comm, static_cast<cudaStream_t>(stream)));
}
pyc_comm_status v_recv(void* bc, pyc_comm_handle_t comm, void* recv, size_t count, pyc_dtype dtype, int peer, void* stream) {
    Ctx* ctx = static_cast<Ctx*>(bc);
    int dt = 0;
    const pyc_comm_status st = check(ctx, comm, count, dtype, &dt);
    if (st != PYC_COMM_OK) return st;
    if (!recv || peer < 0) return PYC_COMM_ERR_INVALID;
    if (!ctx->recv) return PYC_COMM_ERR_HARDWARE;
    return result(ctx, ctx->recv(recv, count, dt, peer, comm, static_cast<cudaStream_t>(stream)));
}
// Stream-ordered barrier: a one-word all-reduce completes on this rank's stream only after every rank's stream has
// reached its own call.
pyc_comm_status v_barrier(void* bc, pyc_comm_handle_t comm, void* stream) {
    Ctx* ctx = static_cast<Ctx*>(bc);
    int dt = 0;
    const pyc_comm_status st = check(ctx, comm, 1, PYC_DTYPE_I32, &dt);
    if (st != PYC_COMM_OK) return st;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 16) return PYC_COMM_ERR_HARDWARE;
    if (!ctx->barrier_word[dev]) {
        if (cudaMalloc(&ctx->barrier_word[dev], 256) != cudaSuccess || cudaMemset(ctx->barrier_word[dev], 0, 256) != cudaSuccess) {
            cudaGetLastError();
            return PYC_COMM_ERR_HARDWARE;
        }
    }
    return result(ctx, ctx->all_reduce(ctx->barrier_word[dev], ctx->barrier_word[dev], 1, dt, 2 /* max */, comm, static_cast<cudaStream_t>(stream)));
}

}  // namespace

extern "C" {

__attribute__((visibility("default"))) pyc_collective_comm* pyc_comm_backend_create(const char* config_json) {
    pyc_collective_comm* comm = static_cast<pyc_collective_comm*>(calloc(1, sizeof(pyc_collective_comm)));
    Ctx* ctx = new Ctx();
    if (!comm) { delete ctx; return nullptr; }
    const bool ok = load_nccl(ctx, config_json);
    if (!ok) {
        if (ctx->lib) { dlclose(ctx->lib); ctx->lib = nullptr; }
        if (json_true(config_json, "strict")) { delete ctx; free(comm); return nullptr; }
    }
    comm->backend_ctx = ctx;
    comm->all_reduce = v_all_reduce; comm->all_gather = v_all_gather; comm->reduce_scatter = v_reduce_scatter;
    comm->broadcast = v_broadcast; comm->send = v_send; comm->recv = v_recv; comm->barrier = v_barrier;
    return comm;
}

__attribute__((visibility("default"))) void pyc_comm_backend_destroy(pyc_collective_comm* comm) {
    if (!comm) return;
    Ctx* ctx = static_cast<Ctx*>(comm->backend_ctx);
    if (ctx) {
        // barrier words are left to the CUDA context's teardown when no device is current any more
        for (int* w : ctx->barrier_word) if (w) cudaFree(w);
        cudaGetLastError();
        if (ctx->lib && ctx->owns_lib) dlclose(ctx->lib);
        delete ctx;
    }
    free(comm);
}

// ---- bootstrap helpers (no counterpart in PyC, whose launcher is expected to bring a communicator) -----------------
// Rank 0 makes the 128-byte id and sends it to the others by whatever channel the launcher has; every rank then calls
// pyc_b200_nccl_comm_init_rank with its CUDA device current.  Return 0 / -1; text in pyc_b200_nccl_last_error().
__attribute__((visibility("default"))) int pyc_b200_nccl_unique_id(pyc_collective_comm* comm, unsigned char id_out[128]) {
    Ctx* ctx = comm ? static_cast<Ctx*>(comm->backend_ctx) : nullptr;
    if (!ctx || !ctx->get_unique_id || !id_out) return -1;
    NcclId id;
    if (result(ctx, ctx->get_unique_id(&id)) != PYC_COMM_OK) return -1;
    memcpy(id_out, id.bytes, 128);
    return 0;
}
__attribute__((visibility("default"))) int pyc_b200_nccl_comm_init_rank(pyc_collective_comm* comm, const unsigned char id_in[128], int world, int rank,
                                                                        pyc_comm_handle_t* handle_out) {
    Ctx* ctx = comm ? static_cast<Ctx*>(comm->backend_ctx) : nullptr;
    if (!ctx || !ctx->comm_init_rank || !id_in || !handle_out || world < 1 || rank < 0 || rank >= world) return -1;
    NcclId id;
    memcpy(id.bytes, id_in, 128);
    nccl_comm c = nullptr;
    if (result(ctx, ctx->comm_init_rank(&c, world, id, rank)) != PYC_COMM_OK) return -1;
    *handle_out = c;
    return 0;
}
__attribute__((visibility("default"))) int pyc_b200_nccl_comm_destroy(pyc_collective_comm* comm, pyc_comm_handle_t handle) {
    Ctx* ctx = comm ? static_cast<Ctx*>(comm->backend_ctx) : nullptr;
    if (!ctx || !ctx->comm_destroy || !handle) return -1;
    return result(ctx, ctx->comm_destroy(handle)) == PYC_COMM_OK ? 0 : -1;
}
__attribute__((visibility("default"))) const char* pyc_b200_nccl_last_error(pyc_collective_comm* comm) {
    Ctx* ctx = comm ? static_cast<Ctx*>(comm->backend_ctx) : nullptr;
    return ctx ? ctx->last_error : "no backend";
}

}  // extern "C"
