// Entry points whose kernels live in files that are not built yet.
#include "internal.h"
namespace b200 {
int launch_attention(pyc_dtype, int, int, int, const void*, const void*, const void*, void*, float, int, cudaStream_t, int*) { set_error("attention kernel not built"); return -1; }
int launch_conv2d(pyc_dtype, int, int, int, int, int, int, int, int, int, int, int, const void*, const void*, const void*, int, void*, cudaStream_t, int*) { set_error("conv2d kernel not built"); return -1; }
}
extern "C" {
int pyc_cutlass_conv2d_dispatch(const char*, int, int, int, int, int, int, int, int, int, int, int, const void*, const void*, void*, void*) { return -1; }
int pyc_cutlass_attention_dispatch(const char*, int, int, const void*, const void*, const void*, void*, float, void*) { return -1; }
int pyc_b200_attention(pyc_dtype, int, int, int, const void*, const void*, const void*, void*, float, int, void*) { return -1; }
int pyc_b200_conv2d(pyc_dtype, int, int, int, int, int, int, int, int, int, int, int, const void*, const void*, const void*, int, void*, void*) { return -1; }
}
