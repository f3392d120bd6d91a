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

#ifdef NA2D_TRACE
// Development aid: the trace CTA 0 of this unit's kernels recorded (see na2d_tc.cuh).
extern "C" int NA2D_TC_NAME(na2d_debug_trace_fwd)(unsigned long long* out, int max_entries) {
    return na2d_tc::copy_trace(out, max_entries);
}
#endif
