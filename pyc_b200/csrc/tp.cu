// Tensor-parallel plumbing that is not a GEMM: the reduction of the per-rank partial sums a rank has received, with the
// all-gather folded in (the reduced rows are stored into every rank's output over NVLink), and the CUDA-IPC helpers
// that make a buffer writable by the other processes of the node.  No kernel here waits on another GPU.
#include <cuda_bf16.h>
#include <string.h>

#include "internal.h"

namespace b200 {
namespace {

struct ReduceArgs {
    const __nv_bfloat16* recv;                       // [world][rows][hidden], local
    __nv_bfloat16* outs[PYC_B200_TP_MAX_RANKS];      // [world * rows][hidden] of every rank
    int world, rank, rows, hidden;
};

// One thread = 8 consecutive bf16 of one owned row: read that 16-byte piece from each of the world slots, add in fp32,
// round once, store to the same place of every rank's output.  HBM-bound on the local reads (world x the slice) and
// NVLink-bound on the (world - 1) remote copies of the slice.
__global__ void __launch_bounds__(256) tp_reduce_broadcast_kernel(ReduceArgs a) {
    const size_t vec_per_row = static_cast<size_t>(a.hidden) / 8;
    const size_t total = static_cast<size_t>(a.rows) * vec_per_row;
    const size_t slot_vecs = total;
    const uint4* recv = reinterpret_cast<const uint4*>(a.recv);
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total; i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        float acc[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll 4
        for (int s = 0; s < a.world; ++s) {
            const uint4 u = __ldg(recv + static_cast<size_t>(s) * slot_vecs + i);
            const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
            for (int t = 0; t < 4; ++t) { acc[2 * t] += __uint_as_float(w[t] << 16); acc[2 * t + 1] += __uint_as_float(w[t] & 0xffff0000u); }
        }
        uint4 o;
        __nv_bfloat162 p0 = __floats2bfloat162_rn(acc[0], acc[1]), p1 = __floats2bfloat162_rn(acc[2], acc[3]);
        __nv_bfloat162 p2 = __floats2bfloat162_rn(acc[4], acc[5]), p3 = __floats2bfloat162_rn(acc[6], acc[7]);
        o.x = *reinterpret_cast<uint32_t*>(&p0); o.y = *reinterpret_cast<uint32_t*>(&p1);
        o.z = *reinterpret_cast<uint32_t*>(&p2); o.w = *reinterpret_cast<uint32_t*>(&p3);
        const size_t dst = static_cast<size_t>(a.rank) * total + i;   // owned rows start at rank * rows
        for (int r = 0; r < a.world; ++r) reinterpret_cast<uint4*>(a.outs[r])[dst] = o;
    }
}

}  // namespace
}  // namespace b200

extern "C" {

int pyc_b200_tp_reduce_broadcast(const void* recv_local, void* const* outs, int world, int rank, int rows_per_rank, int hidden, void* stream) {
    using namespace b200;
    if (!recv_local || !outs || world < 1 || world > PYC_B200_TP_MAX_RANKS || rank < 0 || rank >= world || rows_per_rank <= 0 || hidden <= 0) {
        set_error("tp reduce: bad arguments"); return -1;
    }
    if (hidden % 8 != 0 || reinterpret_cast<uintptr_t>(recv_local) % 16) { set_error("tp reduce: hidden must be a multiple of 8 and the buffers 16-byte aligned"); return -1; }
    ReduceArgs a;
    a.recv = static_cast<const __nv_bfloat16*>(recv_local);
    a.world = world; a.rank = rank; a.rows = rows_per_rank; a.hidden = hidden;
    for (int i = 0; i < PYC_B200_TP_MAX_RANKS; ++i) {
        a.outs[i] = i < world ? static_cast<__nv_bfloat16*>(outs[i]) : nullptr;
        if (i < world && (!outs[i] || reinterpret_cast<uintptr_t>(outs[i]) % 16)) { set_error("tp reduce: output %d is NULL or not 16-byte aligned", i); return -1; }
    }
    const size_t total = static_cast<size_t>(rows_per_rank) * (hidden / 8);
    size_t blocks = (total + 255) / 256;
    const size_t cap = static_cast<size_t>(sm_count()) * 8;
    if (blocks > cap) blocks = cap;
    tp_reduce_broadcast_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(a);
    B200_CUDA_OK(cudaGetLastError());
    count_launch();
    return 0;
}

int pyc_b200_symm_alloc(size_t bytes, void** ptr, unsigned char handle[64]) {
    using namespace b200;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "CUDA IPC handle size");
    if (!ptr || !handle || bytes == 0) { set_error("symm alloc: bad arguments"); return -1; }
    void* p = nullptr;
    B200_CUDA_OK(cudaMalloc(&p, bytes));
    cudaIpcMemHandle_t h;
    const cudaError_t e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) { cudaFree(p); cudaGetLastError(); set_error("cudaIpcGetMemHandle failed: %s", cudaGetErrorString(e)); return -1; }
    memcpy(handle, &h, 64);
    *ptr = p;
    return 0;
}
int pyc_b200_symm_open(const unsigned char handle[64], void** ptr) {
    using namespace b200;
    if (!ptr || !handle) { set_error("symm open: bad arguments"); return -1; }
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, 64);
    B200_CUDA_OK(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
    return 0;
}
int pyc_b200_symm_close(void* ptr) {
    using namespace b200;
    if (!ptr) return 0;
    B200_CUDA_OK(cudaIpcCloseMemHandle(ptr));
    return 0;
}
int pyc_b200_symm_free(void* ptr) {
    using namespace b200;
    if (!ptr) return 0;
    B200_CUDA_OK(cudaFree(ptr));
    return 0;
}

}  // extern "C"
