// seq_common.cuh -- helpers shared by the ragged-batch sequence ops (seq_ops.cu, diff_attention.cu, moe_ops.cu).
// Activations come in one of two element types, selected at run time by `elem` (bytes per element): 4 = float,
// 2 = bfloat16.  Everything that is accumulated, normalised or carried as state is float.
#pragma once
#include <cuda_bf16.h>

#include "pa_common.cuh"

namespace pa {

typedef __nv_bfloat16 bf16_t;

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<bf16_t>(bf16_t v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16_t from_f32<bf16_t>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float sigmoid_f32(float v) { return 1.0f / (1.0f + expf(-v)); }
__device__ __forceinline__ float silu_f32(float v) { return v / (1.0f + expf(-v)); }
__device__ __forceinline__ float gelu_erf_f32(float v) { return 0.5f * v * (1.0f + erff(v * 0.70710678118654752440f)); }

// Sum over a CTA of up to 1024 threads (whole warps); every thread gets the result.  `sm` holds 32 floats.
__device__ __forceinline__ float block_sum(float v, float* sm) {
    v = warp_sum(v);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
    __syncthreads();  // a previous use of `sm` is over
    if (lane == 0) sm[warp] = v;
    __syncthreads();
    float r = (lane < nw) ? sm[lane] : 0.f;
    return warp_sum(r);
}

#define PA_DISPATCH_ELEM(elem, ...)                          \
    do {                                                     \
        if ((elem) == 4) { typedef float T; __VA_ARGS__; }   \
        else if ((elem) == 2) { typedef bf16_t T; __VA_ARGS__; } \
        else return PA_ERR_UNSUPPORTED;                      \
    } while (0)

}  // namespace pa
