// Host-visible entry points of the loop kernel translation unit.
#pragma once
#include <cuda_runtime.h>

#include "program.h"

namespace arkb {
size_t loop_kernel_smem_bytes();
cudaError_t loop_kernel_prepare();
// smem_bytes: dynamic shared memory the program's stages need (0: the kernel's maximum)
cudaError_t loop_kernel_launch(const LaunchParams &P, int grid, cudaStream_t stream, size_t smem_bytes);
}  // namespace arkb
