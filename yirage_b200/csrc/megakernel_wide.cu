// Kernel for graphs with more than 8 tokens per iteration (16-token and tcgen05 LINEAR paths,
// tensor memory), with or without tensor parallelism.
#include "megakernel_body.cuh"

namespace ypk {

__global__ void __launch_bounds__(kBlockThreads, 1) ypk_megakernel_wide(const __grid_constant__ Runtime rt) {
  megakernel_body<true, true>(rt);
}

}  // namespace ypk
