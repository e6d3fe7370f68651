// Warp-specialised kernel instantiations: LayerNorm backward without column sums, with given
// statistics (LayerNormBwdDxOp) and with the statistics recomputed from the row
// (LayerNormBwdRecomputeOp, 8 output warps only).
#include <cuda_bf16.h>

#include "../../include/credit_b200.h"
#include "kernel_tables.h"
#include "ws_tables.h"

namespace credit {

const void* ws_layernorm_bwd_dx_kernel_for(int dtype, int out_warps, int vpt, bool full, bool recompute) {
    if (recompute) {
        if (out_warps != 8) return nullptr;
        constexpr int kMaxElems = ws_max_elems_per_thread(false, true);
        return dtype == CREDIT_F32 ? ws_pick<LayerNormBwdRecomputeOp, float, 8, kMaxElems>(vpt, full)
                                   : ws_pick<LayerNormBwdRecomputeOp, __nv_bfloat16, 8, kMaxElems>(vpt, full);
    }
    return dtype == CREDIT_F32 ? ws_pick_warps<LayerNormBwdDxOp, float, false>(out_warps, vpt, full)
                               : ws_pick_warps<LayerNormBwdDxOp, __nv_bfloat16, false>(out_warps, vpt, full);
}

}  // namespace credit
