// Shared device helpers for the sm_100a decode kernels.
//
// Numerics contract for every kernel in this directory: the library is compiled with -fmad=false
// and without fast-math, so a*b+c is two roundings unless written as __fmaf_rn, '/' and sqrtf are
// IEEE, and roundf rounds half away from zero — the same choices the reference CPU engine makes
// (src/runtime/TenzoEngine.cpp of catdlia/tenzo), which is what keeps quantised values identical.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace tz {

constexpr int kWarp = 32;

// dp4a with unsigned bytes in `a` and signed bytes in `b` (PTX dp4a.u32.s32), accumulating in s32.
__device__ __forceinline__ int dp4a_us(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ int dp4a_ss(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) { return __byte_perm(a, b, sel); }

// 128-bit streaming load that does not allocate in L1: weights and KV are read once per token.
__device__ __forceinline__ uint4 ld_stream_u4(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
// Coherent (L2) loads for data another CTA of the same kernel may have just written.
__device__ __forceinline__ uint4 ld_cg_u4(const void* p) { return __ldcg(reinterpret_cast<const uint4*>(p)); }

// Programmatic dependent launch: wait until the kernels this one depends on have completed and
// their memory is visible / allow the next kernel in the stream to begin its own prologue.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) v += __shfl_xor_sync(0xffffffffu, v, m);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, m));
    return v;
}
__device__ __forceinline__ int warp_sum_i(int v) {
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) v += __shfl_xor_sync(0xffffffffu, v, m);
    return v;
}

// Block-wide reductions whose result is bit-identical in every thread and every CTA: warp
// butterflies, then each thread adds the per-warp partials in index order. `scratch` holds at
// least blockDim.x/32 floats; two barriers per call.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float t = 0.0f;
    for (int i = 0; i < nw; ++i) t += scratch[i];
    return t;
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float t = scratch[0];
    for (int i = 1; i < nw; ++i) t = fmaxf(t, scratch[i]);
    return t;
}

// y_i = x_i * inv_rms * w_i evaluated left to right (TenzoEngine.cpp:158); w may be null (:163).
__device__ __forceinline__ float rms_apply(float x, float inv_rms, const float* w, int i) {
    float y = x * inv_rms;
    return w ? y * w[i] : y;
}
// inv_rms = 1 / sqrt(sum_sq/dim + eps) (TenzoEngine.cpp:154).
__device__ __forceinline__ float rms_inv(float sum_sq, int dim, float eps) {
    return 1.0f / sqrtf((sum_sq / static_cast<float>(dim)) + eps);
}

}  // namespace tz
