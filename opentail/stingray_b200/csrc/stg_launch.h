// Launchers implemented in the .cu files, called by the C-ABI layer.
#pragma once
#include <cuda_runtime.h>

#include "stg_types.h"

namespace stg {

// shared memory a row-type work item needs: sort keys + exp-value histogram
constexpr size_t kRowArenaBytes = (size_t)kSortCap * 4 + 2048 * 4 + 2048 * 8;

cudaError_t launch_sample(const SampleArgs &a, int grid, size_t smem, cudaStream_t stream);

}  // namespace stg
