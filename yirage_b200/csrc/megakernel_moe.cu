// Kernel for graphs with mixture-of-experts layers (LINEAR tasks whose expert is picked at run
// time, YPK_F_MOE), one GPU, any number of tokens per iteration.  A kernel of its own so that
// the expert lookup is not part of the other kernels' worker loops.
#include "megakernel_body.cuh"

namespace ypk {

__global__ void __launch_bounds__(kBlockThreads, 1) ypk_megakernel_moe(const __grid_constant__ Runtime rt) {
  megakernel_body<false, true, true>(rt);
}

}  // namespace ypk
