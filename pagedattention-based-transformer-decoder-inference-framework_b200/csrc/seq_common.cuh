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

// ---- legacy tensor-core path (mma.sync, bfloat16 operands, float accumulation) ----------------------------------------
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 16-byte asynchronous copy global -> shared; !ok writes zeros and reads nothing
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, bool ok) {
    const int n = ok ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

// eight bfloat16 values in one 16-byte word <-> eight floats
__device__ __forceinline__ void bf16x8_unpack(const uint4& v, float (&f)[8]) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        f[2 * i] = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}
__device__ __forceinline__ uint4 bf16x8_pack(const float (&f)[8]) {
    return make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]));
}

#define PA_DISPATCH_ELEM(elem, ...)                          \
    do {                                                     \
        if ((elem) == 4) { typedef float T; __VA_ARGS__; }   \
        else if ((elem) == 2) { typedef bf16_t T; __VA_ARGS__; } \
        else return PA_ERR_UNSUPPORTED;                      \
    } while (0)

}  // namespace pa
