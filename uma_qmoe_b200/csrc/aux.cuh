// Host launchers of the supporting kernels (aux.cu).
#pragma once
#include <cuda_runtime.h>

namespace umaq {
int launch_quantize_groups(const void* src_bf16, long long elements, int enc, void* codes, float* scales,
                           cudaStream_t stream);
}
