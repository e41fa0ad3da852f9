// Device helpers shared by the bandwidth-bound kernels and the fused attention kernels: warp and CTA
// reductions in a fixed order, and the reference's Schraudolph exponential.
#pragma once
#include "tl_kernels.h"
#include <cfloat>

namespace tl {

__device__ __forceinline__ float warp_sum(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
// Sum over the whole CTA; every thread gets the result.  `red` holds >= 33 floats.
__device__ __forceinline__ float block_sum(float v, float *red)
{
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red[wid] = v;
    __syncthreads();
    float t = (threadIdx.x < nw) ? red[threadIdx.x] : 0.f;
    if (wid == 0) { t = warp_sum(t); if (lane == 0) red[32] = t; }
    __syncthreads();
    return red[32];
}
__device__ __forceinline__ float block_max(float v, float *red)
{
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) red[wid] = v;
    __syncthreads();
    float t = (threadIdx.x < nw) ? red[threadIdx.x] : -FLT_MAX;
    if (wid == 0) { t = warp_max(t); if (lane == 0) red[32] = t; }
    __syncthreads();
    return red[32];
}

// Schraudolph exponential exactly as the reference computes it: multiply and add are
// rounded separately, the float is truncated to an unsigned and reinterpreted
// [ref: lib/sources/pulp_train_utils_fp32.c:1223-1231].
__device__ __forceinline__ float fastexp_gist_dev(float x)
{
    x = __fadd_rn(__fmul_rn(GIST_A, x), GIST_B);
    if (x < (float)GIST_C || x > (float)GIST_D) x = (x < (float)GIST_C) ? 0.0f : (float)GIST_D;
    return __uint_as_float((unsigned)x);
}

} // namespace tl
