// Warp-specialised kernel instantiations: RmsNormFwdOp.
#include <cuda_bf16.h>

#include "../../include/credit_b200.h"
#include "kernel_tables.h"
#include "ws_tables.h"

namespace credit {

const void* ws_rmsnorm_kernel_for(int dtype, int out_warps, int vpt, bool full) {
    return dtype == CREDIT_F32 ? ws_pick_warps<RmsNormFwdOp, float, false>(out_warps, vpt, full)
                               : ws_pick_warps<RmsNormFwdOp, __nv_bfloat16, false>(out_warps, vpt, full);
}

}  // namespace credit
