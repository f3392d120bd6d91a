// Translation unit of the tcgen05 forward kernels for one 16-bit element type
// (-DNA2D_TC_DT=1: bf16, 2: fp16).
#include "na2d_tc_entry.h"
#include "na2d_tc_fwd1.cuh"
#include "na2d_tc_fwd.cuh"

namespace na2d_tc {

#if NA2D_TC_DT == 1
#define NA2D_TC_TYPE __nv_bfloat16
#define NA2D_TC_NAME(base) base##_bf16
#elif NA2D_TC_DT == 2
#define NA2D_TC_TYPE __half
#define NA2D_TC_NAME(base) base##_f16
#else
#error "compile with -DNA2D_TC_DT=1 (bf16) or 2 (fp16)"
#endif

int NA2D_TC_NAME(forward)(const LaunchCtx& lc, const TensorArg& q, const TensorArg& k, const TensorArg& v,
                          const TensorArg& o, float* lse) {
    const Na2dGeom& g = lc.g;
    NA2D_TC_DISPATCH_D(launch_forward, NA2D_TC_TYPE, lc, q, k, v, o, lse)
}

}  // namespace na2d_tc
