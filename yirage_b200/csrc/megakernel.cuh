// The variants of the persistent megakernel (one translation unit each, megakernel_*.cu):
// one-GPU decode with at most 8 tokens per iteration, the same under tensor parallelism, the
// variant for more than 8 tokens (16-token and tcgen05 LINEAR paths, tensor memory), and the
// one for graphs with mixture-of-experts layers.
#pragma once
#include "device_common.cuh"

namespace ypk {

__global__ void ypk_megakernel_decode(const __grid_constant__ Runtime rt);
__global__ void ypk_megakernel_decode_tp(const __grid_constant__ Runtime rt);
__global__ void ypk_megakernel_wide(const __grid_constant__ Runtime rt);
__global__ void ypk_megakernel_moe(const __grid_constant__ Runtime rt);

}  // namespace ypk
