// Host entry points of the tcgen05 kernel families.  Each family is compiled in a translation
// unit of its own, once per 16-bit element type (na2d_tc_fwd.cu, na2d_tc_dq.cu, na2d_tc_dkdv.cu
// with -DNA2D_TC_DT=1 for bf16 and 2 for fp16), so that the library builds in parallel.
#pragma once

#include "na2d_tc.cuh"

namespace na2d_tc {

int forward_bf16(const LaunchCtx& lc, const TensorArg& q, const TensorArg& k, const TensorArg& v, const TensorArg& o,
                 float* lse);
int forward_f16(const LaunchCtx& lc, const TensorArg& q, const TensorArg& k, const TensorArg& v, const TensorArg& o,
                float* lse);

// dQ (d_q.ptr may be null: delta only).  The exact row deltas are written to `delta`.  delta_in, if
// not null (it may be `delta` itself), holds an estimate of them (dO . o); the kernels of the
// larger windows then walk their key box once and correct the result, instead of walking twice.
int backward_dq_bf16(const LaunchCtx& lc, const TensorArg& q, const TensorArg& k, const TensorArg& v, const float* lse,
                     const TensorArg& d_o, const TensorArg& d_q, float* delta, const float* delta_in);
int backward_dq_f16(const LaunchCtx& lc, const TensorArg& q, const TensorArg& k, const TensorArg& v, const float* lse,
                    const TensorArg& d_o, const TensorArg& d_q, float* delta, const float* delta_in);

int backward_dkdv_bf16(const LaunchCtx& lc, const TensorArg& q, const TensorArg& k, const TensorArg& v,
                       const float* lse, const TensorArg& d_o, const float* delta, const TensorArg& d_k,
                       const TensorArg& d_v);
int backward_dkdv_f16(const LaunchCtx& lc, const TensorArg& q, const TensorArg& k, const TensorArg& v,
                      const float* lse, const TensorArg& d_o, const float* delta, const TensorArg& d_k,
                      const TensorArg& d_v);

}  // namespace na2d_tc
