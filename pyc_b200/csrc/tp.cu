// Tensor-parallel plumbing that is not a GEMM: the reduction of the per-rank partial sums a rank has received, with the
// all-gather folded in (the reduced rows are stored into every rank's output over NVLink), and the CUDA-IPC helpers
// that make a buffer writable by the other processes of the node.  No kernel here waits on another GPU.
#include <cuda_bf16.h>
#include <stdlib.h>
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

// ---- all-reduce inside the NVSwitch (multimem) ---------------------------------------------------------------------
// Every rank's [rows][hidden] bf16 partial sum lives at the same offset of a buffer that is bound to one NVLink
// multicast object; `mc` is the multicast address of that buffer.  A rank owns 1/world of the 16-byte pieces: for each
// it issues multimem.ld_reduce (the switch fetches the piece from every GPU, adds in fp32, returns one bf16x2 x 4) and
// multimem.st (the switch stores the result into every GPU's copy).  Per GPU and direction ~(1 + 1/world) x the tensor
// crosses NVLink, against 2 (world-1)/world for a ring, and the sum is rounded once.
// Two rendezvous per call, block b of a rank with block b of every other rank: before the reads (every rank's producer
// kernel has finished: stream order on each rank + this flag exchange) and after the stores (every rank's pieces have
// been written everywhere).  A flag is a 32-bit epoch in the RECEIVER's memory with one writer, (block, sender); epochs
// come from a per-block counter in local memory that the kernel advances itself, so a captured graph replays correctly.
// Waits are bounded (about two seconds of clock64); a wait that runs out records (site << 8) | 1 in the status word and
// the kernel carries on to its end, so the counter stays in step with the other ranks.
constexpr int MM_BLOCKS = PYC_B200_TP_MULTIMEM_BLOCKS, MM_MAX_THREADS = 1024;

struct MultimemArgs {
    char* mc;                                   // multicast address of the [rows][hidden] bf16 buffer
    uint32_t* flags[PYC_B200_TP_MAX_RANKS];     // [MM_BLOCKS][PYC_B200_TP_MAX_RANKS] of every rank (own and peer-mapped)
    uint32_t* epochs;                           // [MM_BLOCKS], local
    int* status;
    int world, rank;
    size_t vec_begin, vec_end;                  // this rank's 16-byte pieces
};

__device__ __forceinline__ void mm_rendezvous(const MultimemArgs& a, uint32_t epoch, int site) {
    __syncthreads();
    const int peer = threadIdx.x;
    if (peer < a.world && peer != a.rank) {
        __threadfence_system();
        uint32_t* theirs = a.flags[peer] + blockIdx.x * PYC_B200_TP_MAX_RANKS + a.rank;
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(theirs), "r"(epoch) : "memory");
        const uint32_t* mine = a.flags[a.rank] + blockIdx.x * PYC_B200_TP_MAX_RANKS + peer;
        const long long t0 = clock64();
        for (;;) {
            uint32_t v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
            if (static_cast<int32_t>(v - epoch) >= 0) break;
            if (clock64() - t0 > 4000000000ll) { atomicCAS(a.status, 0, (site << 8) | 1); break; }
        }
    }
    __syncthreads();
}

template <int MM_UNROLL>
__global__ void __launch_bounds__(MM_MAX_THREADS) tp_allreduce_multimem_kernel(MultimemArgs a) {
    const uint32_t epoch = a.epochs[blockIdx.x];
    mm_rendezvous(a, epoch + 1, 40);
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    for (size_t i0 = a.vec_begin + blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i0 < a.vec_end; i0 += stride * MM_UNROLL) {
        uint32_t v[MM_UNROLL][4];
#pragma unroll
        for (int u = 0; u < MM_UNROLL; ++u) {
            const size_t i = i0 + u * stride;
            if (i < a.vec_end)
                asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                             : "=r"(v[u][0]), "=r"(v[u][1]), "=r"(v[u][2]), "=r"(v[u][3]) : "l"(a.mc + i * 16) : "memory");
        }
#pragma unroll
        for (int u = 0; u < MM_UNROLL; ++u) {
            const size_t i = i0 + u * stride;
            if (i < a.vec_end)
                asm volatile("multimem.st.relaxed.sys.global.v4.bf16x2 [%0], {%1, %2, %3, %4};"
                             ::"l"(a.mc + i * 16), "r"(v[u][0]), "r"(v[u][1]), "r"(v[u][2]), "r"(v[u][3]) : "memory");
        }
    }
    mm_rendezvous(a, epoch + 2, 41);
    if (threadIdx.x == 0) a.epochs[blockIdx.x] = epoch + 2;
}

}  // namespace
}  // namespace b200

extern "C" {

int pyc_b200_tp_allreduce_multimem(void* multicast_ptr, void* const* flag_ptrs, void* epoch_counters, int world, int rank,
                                   size_t rows, size_t hidden, void* stream) {
    using namespace b200;
    if (!multicast_ptr || !flag_ptrs || !epoch_counters || world < 2 || world > PYC_B200_TP_MAX_RANKS || rank < 0 || rank >= world || rows == 0 || hidden == 0) {
        set_error("tp multimem all-reduce: bad arguments"); return -1;
    }
    if (hidden % 8 != 0 || reinterpret_cast<uintptr_t>(multicast_ptr) % 16) { set_error("tp multimem all-reduce: hidden must be a multiple of 8 and the buffer 16-byte aligned"); return -1; }
    MultimemArgs a;
    a.mc = static_cast<char*>(multicast_ptr);
    for (int i = 0; i < PYC_B200_TP_MAX_RANKS; ++i) {
        a.flags[i] = i < world ? static_cast<uint32_t*>(flag_ptrs[i]) : nullptr;
        if (i < world && !flag_ptrs[i]) { set_error("tp multimem all-reduce: flag buffer %d is NULL", i); return -1; }
    }
    a.epochs = static_cast<uint32_t*>(epoch_counters);
    a.status = device_status_word();
    if (!a.status) return -1;
    a.world = world; a.rank = rank;
    const size_t total = rows * (hidden / 8);
    a.vec_begin = total * static_cast<size_t>(rank) / world;
    a.vec_end = total * static_cast<size_t>(rank + 1) / world;
    if (sm_count() < MM_BLOCKS) { set_error("tp multimem all-reduce: needs %d co-resident blocks, the device has %d SMs", MM_BLOCKS, sm_count()); return -1; }
    int threads = 128, unroll = 2;   // measured on 4 GPUs, 64 MB: 0.170 ms; 512 x 4: 0.182; 1024 x 8: 0.200 (the switch, not the latency, is the limit)
    if (const char* e = getenv("PYC_B200_TP_MULTIMEM_THREADS")) { const int v = atoi(e); if (v >= 32 && v <= MM_MAX_THREADS && v % 32 == 0) threads = v; }
    if (const char* e = getenv("PYC_B200_TP_MULTIMEM_UNROLL")) unroll = atoi(e);
    if (unroll == 8) tp_allreduce_multimem_kernel<8><<<MM_BLOCKS, threads, 0, static_cast<cudaStream_t>(stream)>>>(a);
    else if (unroll == 4) tp_allreduce_multimem_kernel<4><<<MM_BLOCKS, threads, 0, static_cast<cudaStream_t>(stream)>>>(a);
    else tp_allreduce_multimem_kernel<2><<<MM_BLOCKS, threads, 0, static_cast<cudaStream_t>(stream)>>>(a);
    B200_CUDA_OK(cudaGetLastError());
    count_launch();
    return 0;
}

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
