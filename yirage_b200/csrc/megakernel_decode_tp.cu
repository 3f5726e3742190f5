// Tensor-parallel decode kernel (at most 8 tokens per iteration).
#include "megakernel_body.cuh"

namespace ypk {

__global__ void __launch_bounds__(kBlockThreads, 1) ypk_megakernel_decode_tp(const __grid_constant__ Runtime rt) {
  megakernel_body<true, false>(rt);
}

}  // namespace ypk
