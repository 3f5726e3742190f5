// One-GPU decode kernel (at most 8 tokens per iteration, no tensor parallelism): the
// configuration the headline benchmark runs.  The runners it calls are this unit's own copies.
#include "megakernel_body.cuh"

namespace ypk {

__global__ void __launch_bounds__(kBlockThreads, 1) ypk_megakernel_decode(const __grid_constant__ Runtime rt) {
  megakernel_body<false, false>(rt);
}

}  // namespace ypk
