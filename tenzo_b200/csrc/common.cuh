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

// Ask L2 to fetch [base, base+bytes) ahead of use: the kernels of a decode step run one after another
// on data-dependent vectors, so each kernel requests the NEXT kernel's weights while it works and
// HBM keeps streaming across kernel boundaries. Work is spread over the whole grid, one line per thread.
__device__ __forceinline__ void l2_prefetch_slice(const void* base, size_t bytes) {
    if (!base) return;
    const size_t n_lines = (bytes + 127) / 128;
    const size_t cta = blockIdx.x + (size_t)gridDim.x * (blockIdx.y + (size_t)gridDim.y * blockIdx.z);
    const size_t n_threads = (size_t)gridDim.x * gridDim.y * gridDim.z * blockDim.x;
    for (size_t c = cta * blockDim.x + threadIdx.x; c < n_lines; c += n_threads)
        asm volatile("prefetch.global.L2 [%0];" ::"l"(static_cast<const char*>(base) + c * 128));
}

// ---- bulk asynchronous copy (TMA, 1-D) global -> shared with mbarrier completion ---------------------
// A bulk copy keeps tens of kilobytes in flight per SM from a single instruction; ordinary loads
// are capped by the load/store unit's request queue long before HBM latency is covered.
__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_init_fence() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
// dst and src 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, unsigned bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_addr(dst)), "l"(src), "r"(bytes), "r"(smem_addr(bar)) : "memory");
}
// Wait for phase `parity` of an mbarrier, giving up after a bounded number of polls (each poll
// already blocks for a hardware-defined interval). Returns false on give-up so the caller can flag
// the failure and leave instead of hanging the GPU.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, unsigned parity) {
    const uint32_t addr = smem_addr(bar);
    for (int it = 0; it < (1 << 20); ++it) {
        uint32_t done;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(done) : "r"(addr), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}

// Barrier among `count` threads (a multiple of 32) of the CTA; id 1..15 (0 is __syncthreads).
__device__ __forceinline__ void named_barrier_sync(int id, int count) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory"); }

// One non-blocking look at phase `parity` of an mbarrier.
__device__ __forceinline__ bool mbar_test(uint64_t* bar, unsigned parity) {
    uint32_t done;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(done) : "r"(smem_addr(bar)), "r"(parity) : "memory");
    return done != 0;
}

// Bounded wait by polling test_wait (no hardware suspend between polls): lower wake-up latency than
// mbar_wait_bounded, for the hand-offs inside a software pipeline. Returns false on give-up.
__device__ __forceinline__ bool mbar_spin_bounded(uint64_t* bar, unsigned parity) {
    for (int it = 0; it < (1 << 24); ++it)
        if (mbar_test(bar, parity)) return true;
    return false;
}

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
__device__ __forceinline__ int warp_sum_i(int v) { return __reduce_add_sync(0xffffffffu, v); }   // one redux.sync
// Maximum over the warp of values that are >= 0 and not NaN (running maxima of |x| that started at 0: fmaxf drops NaN):
// for those the order of the floats is the order of their bit patterns, so one integer redux.sync replaces five shuffles.
__device__ __forceinline__ float warp_max_nonneg(float v) {
    return __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(v)));
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
// The same for values >= 0 that are not NaN (see warp_max_nonneg).
__device__ __forceinline__ float block_max_nonneg(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_max_nonneg(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    return warp_max_nonneg(scratch[lane < nw ? lane : 0]);
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    // the per-warp maxima are reduced by a second butterfly (a maximum does not depend on the order; as a loop of
    // dependent loads over up to 16 slots this step alone took some 500 cycles)
    return warp_max(scratch[lane < nw ? lane : 0]);
}

// Sum of squares in the exact order of the reference's vectorised loop (TenzoEngine.cpp:149-153 as
// gcc compiles it for AVX2): eight lanes, lane j accumulating x[j], x[j+8], ... with a separately
// rounded product and sum (no FMA), then the lanes added left to right starting from lane 0; any
// tail beyond a multiple of eight follows in index order. fp32 addition is not associative, and
// this value feeds a quantiser, so the order is part of the result. `x` is in shared memory and
// complete (caller has synchronised); every thread returns the same bits. Two barriers.
__device__ __forceinline__ float sumsq_reference_order(const float* x, int dim, float* scratch) {
    const int n8 = dim & ~7;
    if (threadIdx.x < 8) {
        float s = 0.0f;
        int i = threadIdx.x;
        // 16 loads in flight ahead of the dependent adds: the chain runs at add latency, not load latency
        for (; i + 8 * 15 < n8; i += 8 * 16) {
            float v[16];
#pragma unroll
            for (int u = 0; u < 16; ++u) v[u] = x[i + 8 * u];
#pragma unroll
            for (int u = 0; u < 16; ++u) v[u] = __fmul_rn(v[u], v[u]);
#pragma unroll
            for (int u = 0; u < 16; ++u) s = __fadd_rn(s, v[u]);
        }
        for (; i < n8; i += 8) {
            const float v = x[i];
            s = __fadd_rn(s, __fmul_rn(v, v));
        }
        scratch[threadIdx.x] = s;
    }
    __syncthreads();
    float t = scratch[0];
#pragma unroll
    for (int j = 1; j < 8; ++j) t = __fadd_rn(t, scratch[j]);
    for (int i = n8; i < dim; ++i) t = __fadd_rn(t, __fmul_rn(x[i], x[i]));
    __syncthreads();
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

// expf with the bits glibc's expf returns for x <= 0 (the softmax arguments, TenzoEngine.cpp:826).
// It is the published table-driven algorithm glibc uses (Szabolcs Nagy's exp2f/expf from ARM's
// optimized-routines: 32-entry table of 2^(i/32), cubic in double precision, k = round(x*32/ln2)
// through the 1.5*2^52 shift), with the reduced argument formed by one fused multiply-add as the
// FMA build of the library does. Checked against the host's expf on every float in [-104.5, -0]:
// zero differences. Inputs above 0 are outside its use here.
static __device__ __constant__ unsigned long long kExp2fTab[32] = {
    0x3ff0000000000000ull, 0x3fefd9b0d3158574ull, 0x3fefb5586cf9890full, 0x3fef9301d0125b51ull,
    0x3fef72b83c7d517bull, 0x3fef54873168b9aaull, 0x3fef387a6e756238ull, 0x3fef1e9df51fdee1ull,
    0x3fef06fe0a31b715ull, 0x3feef1a7373aa9cbull, 0x3feedea64c123422ull, 0x3feece086061892dull,
    0x3feebfdad5362a27ull, 0x3feeb42b569d4f82ull, 0x3feeab07dd485429ull, 0x3feea47eb03a5585ull,
    0x3feea09e667f3bcdull, 0x3fee9f75e8ec5f74ull, 0x3feea11473eb0187ull, 0x3feea589994cce13ull,
    0x3feeace5422aa0dbull, 0x3feeb737b0cdc5e5ull, 0x3feec49182a3f090ull, 0x3feed503b23e255dull,
    0x3feee89f995ad3adull, 0x3feeff76f2fb5e47ull, 0x3fef199bdd85529cull, 0x3fef3720dcef9069ull,
    0x3fef5818dcfba487ull, 0x3fef7c97337b9b5full, 0x3fefa4afa2a490daull, 0x3fefd0765b6e4540ull};

__device__ __forceinline__ float expf_reference_bits(float x) {
    if (x < -0x1.9fe368p6f) return 0.0f;                       // underflow to zero below about -103.97
    const double inv_ln2_n = 0x1.71547652b82fep+0 * 32.0, shift = 0x1.8p+52;
    const double c0 = 0x1.c6af84b912394p-5 / 32 / 32 / 32, c1 = 0x1.ebfce50fac4f3p-3 / 32 / 32, c2 = 0x1.62e42ff0c52d6p-1 / 32;
    const double xd = (double)x;
    const double z = __dmul_rn(inv_ln2_n, xd);
    double kd = __dadd_rn(z, shift);
    const unsigned long long ki = (unsigned long long)__double_as_longlong(kd);
    kd = __dadd_rn(kd, -shift);
    const double r = __fma_rn(inv_ln2_n, xd, -kd);
    const unsigned long long t = kExp2fTab[ki & 31] + (ki << 47);
    const double s = __longlong_as_double((long long)t);
    const double zz = __fma_rn(c0, r, c1);
    const double r2 = __dmul_rn(r, r);
    double y = __fma_rn(c2, r, 1.0);
    y = __fma_rn(zz, r2, y);
    y = __dmul_rn(y, s);
    return __double2float_rn(y);
}

// Same bits as expf_reference_bits, with the 32-entry table held one entry per lane (tab_lo/tab_hi =
// the two halves of kExp2fTab[lane]) and fetched by shuffle instead of a data-dependent constant
// load. Every lane of the warp must make the call.
__device__ __forceinline__ float expf_reference_bits_lanes(float x, uint32_t tab_lo, uint32_t tab_hi) {
    const double inv_ln2_n = 0x1.71547652b82fep+0 * 32.0, shift = 0x1.8p+52;
    const double c0 = 0x1.c6af84b912394p-5 / 32 / 32 / 32, c1 = 0x1.ebfce50fac4f3p-3 / 32 / 32, c2 = 0x1.62e42ff0c52d6p-1 / 32;
    const double xd = (double)x;
    const double z = __dmul_rn(inv_ln2_n, xd);
    double kd = __dadd_rn(z, shift);
    const unsigned long long ki = (unsigned long long)__double_as_longlong(kd);
    kd = __dadd_rn(kd, -shift);
    const double r = __fma_rn(inv_ln2_n, xd, -kd);
    const int sel = (int)(ki & 31);
    const uint32_t lo = __shfl_sync(0xffffffffu, tab_lo, sel), hi = __shfl_sync(0xffffffffu, tab_hi, sel);
    const unsigned long long t = (((unsigned long long)hi << 32) | lo) + (ki << 47);
    const double s = __longlong_as_double((long long)t);
    const double zz = __fma_rn(c0, r, c1);
    const double r2 = __dmul_rn(r, r);
    double y = __fma_rn(c2, r, 1.0);
    y = __fma_rn(zz, r2, y);
    y = __dmul_rn(y, s);
    return x < -0x1.9fe368p6f ? 0.0f : __double2float_rn(y);
}

}  // namespace tz
