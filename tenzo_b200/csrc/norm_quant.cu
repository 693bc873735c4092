// Standalone fused RMSNorm + per-token absmax quantiser (both flavours the reference uses).
//
// qmax = 31 : the quantiser half of build_lut — floor 1e-6, q = round(y*(31/m)), scale m/31
//             (src/runtime/TenzoEngine.cpp:27-42 of the reference).
// qmax = 127: compute_logits' quantiser — floor 1e-8, s = amax/127, q = clamp(round(y*(1/s)))
//             (:1666-1678).
// The GEMV and LM-head kernels carry the same code in their prologues; this entry exists for the
// backend class's executeRMSNorm and for checking the quantiser on its own.
#include "common.cuh"
#include "attn_common.cuh"
#include "../../include/tenzo_kernels.h"

namespace tz {

constexpr int kNqThreads = 256;

__global__ void __launch_bounds__(kNqThreads) rmsnorm_quant_kernel(
    const float* __restrict__ x, const float* __restrict__ norm_w, int do_norm, float eps, int dim, int qmax,
    int x_stride, float* y_out, int8_t* q_out, float* scale_out) {
    extern __shared__ float s_y[];            // dim floats + 32 scratch
    float* s_f = s_y + dim;
    const int tid = threadIdx.x, seq = blockIdx.x;
    const float* xs = x + (size_t)seq * x_stride;

    for (int i = tid; i < dim; i += kNqThreads) s_y[i] = xs[i];
    float m = 0.0f;
    if (do_norm) {
        __syncthreads();
        const float ss = sumsq_reference_order(s_y, dim, s_f);
        const float inv_rms = rms_inv(ss, dim, eps);
        for (int i = tid; i < dim; i += kNqThreads) {
            const float y = rms_apply(s_y[i], inv_rms, norm_w, i);
            s_y[i] = y;
            m = fmaxf(m, fabsf(y));
        }
    } else {
        for (int i = tid; i < dim; i += kNqThreads) m = fmaxf(m, fabsf(s_y[i]));
    }
    if (y_out)
        for (int i = tid; i < dim; i += kNqThreads) y_out[(size_t)seq * dim + i] = s_y[i];
    if (!q_out && !scale_out) return;
    m = block_max_nonneg(m, s_f);      // m: running maximum of |y| from 0
    if (qmax == 31) {
        m = fmaxf(m, 1e-6f);
        const float to_q = 31.0f / m;
        if (q_out)
            for (int i = tid; i < dim; i += kNqThreads)
                q_out[(size_t)seq * dim + i] = (int8_t)(int)roundf(s_y[i] * to_q);
        if (scale_out && tid == 0) scale_out[seq] = m / 31.0f;
    } else {
        m = fmaxf(m, 1e-8f);
        const float s = m / 127.0f, inv = 1.0f / s;
        if (q_out)
            for (int i = tid; i < dim; i += kNqThreads)
                q_out[(size_t)seq * dim + i] = (int8_t)(int)fminf(fmaxf(roundf(s_y[i] * inv), -128.0f), 127.0f);
        if (scale_out && tid == 0) scale_out[seq] = s;
    }
}

// Batched front half of the TL1 GEMM: per sequence RMSNorm + absmax(31) quantiser, written as the
// packed tensor-core B fragments tl1_mma_kernel consumes: words[seq][set][t][0] holds 4*a for the
// even columns of column pairs 16*set + 4*i + t (byte i = 0..3), words[seq][set][t][1] the odd
// columns unscaled; columns beyond K are zero. inv[seq] = max|y|/31. `words` may be null (tensor-core GEMM
// path: it takes the plain int8 matrix a_out [batch][K] and sum_out[seq] = sum_k a_k instead).
#ifdef TZ_AQ_TRACE
__device__ long long g_aq_trace[8];
#define AQT(i) do { if (blockIdx.x == 0 && threadIdx.x == 0) g_aq_trace[i] = clock64(); } while (0)
#else
#define AQT(i) ((void)0)
#endif
constexpr int kAqVec = 7;     // float4 values a thread of act_quant_kernel holds: rows up to 7168 floats stay in registers

__global__ void __launch_bounds__(kNqThreads) act_quant_kernel(
    const float* x, const float* __restrict__ norm_w, int do_norm, float eps, int K, int x_stride,
    uint32_t* words, float* inv, int8_t* a_out, int* sum_out, int use_pdl) {
    extern __shared__ __align__(16) float s_y[];   // K floats (or eight padded rows of K/8 squares) + 32 scratch
    float* s_f = s_y + K + 64;
    const int tid = threadIdx.x, seq = blockIdx.x;
    // Let the GEMM that consumes this kernel's output start at once: its prologue (tensor-memory allocation, the first
    // weight copies, expanding the first weight chunks) depends on nothing here and takes as long as this whole kernel;
    // it waits for this grid's completion before it touches the activations.
    AQT(0);
    if (use_pdl) pdl_launch_dependents();
    const float* xs = x + (size_t)seq * x_stride;
    // The whole row in registers as 16-byte loads, all in flight at once; shared memory is only touched where another
    // thread needs the value (the sum of squares in reference order, the packed fragments of the mma.sync path), instead
    // of four passes over a staged copy.
    const bool vec = (K & 3) == 0 && K <= 4 * kAqVec * kNqThreads && (x_stride & 3) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 &&
                     (!norm_w || (reinterpret_cast<uintptr_t>(norm_w) & 15) == 0) && (!a_out || (reinterpret_cast<uintptr_t>(a_out) & 3) == 0);
    if (vec) {
        const int k4 = K >> 2;
        float4 w4[kAqVec], v[kAqVec];
        const bool has_w = do_norm && norm_w;
        if (has_w) {                                    // model constants: no need to wait for the previous kernel
#pragma unroll
            for (int r = 0; r < kAqVec; ++r) {
                const int i = tid + r * kNqThreads;
                w4[r] = i < k4 ? __ldg(reinterpret_cast<const float4*>(norm_w) + i) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
        if (use_pdl) pdl_wait();
        AQT(1);
#pragma unroll
        for (int r = 0; r < kAqVec; ++r) {
            const int i = tid + r * kNqThreads;
            v[r] = i < k4 ? __ldcg(reinterpret_cast<const float4*>(xs) + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        float m = 0.0f;
        if (do_norm) {
            float ss;
            if ((K & 7) == 0) {
                // Squares from every thread, stored chain-major (lane j's x[j]^2, x[j+8]^2, ... contiguous, rows padded so
                // that the eight lanes' 16-byte loads fall in different banks); the eight chains of the reference's order
                // then cost one load per four adds and one add per element. The chain shares its SM with the
                // consuming GEMM's first round of weight expansion, and every instruction it does not have to issue is
                // one it does not have to queue for (load + square + add per element ran at 10.6 cycles per step there).
                const int rows = K >> 3, stride = ((rows + 3) & ~3) + 4;
#pragma unroll
                for (int r = 0; r < kAqVec; ++r) {
                    const int i = tid + r * kNqThreads;
                    if (i < k4) {
                        float* d = s_y + (4 * (i & 1)) * stride + (i >> 1);      // element 4i + c: row (4i + c) & 7, column (4i + c) >> 3
                        d[0] = __fmul_rn(v[r].x, v[r].x);
                        d[stride] = __fmul_rn(v[r].y, v[r].y);
                        d[2 * stride] = __fmul_rn(v[r].z, v[r].z);
                        d[3 * stride] = __fmul_rn(v[r].w, v[r].w);
                    }
                }
                __syncthreads();
                AQT(2);
                if (tid < 8) s_f[tid] = sequential_sum(s_y + tid * stride, rows);
                __syncthreads();
                ss = s_f[0];
#pragma unroll
                for (int j = 1; j < 8; ++j) ss = __fadd_rn(ss, s_f[j]);        // lanes added left to right, from lane 0
            } else {
#pragma unroll
                for (int r = 0; r < kAqVec; ++r) {
                    const int i = tid + r * kNqThreads;
                    if (i < k4) reinterpret_cast<float4*>(s_y)[i] = v[r];
                }
                __syncthreads();
                AQT(2);
                ss = sumsq_reference_order(s_y, K, s_f);
            }
            AQT(3);
            const float inv_rms = rms_inv(ss, K, eps);
#pragma unroll
            for (int r = 0; r < kAqVec; ++r) {          // y = (x * inv_rms) * w, left to right (rms_apply)
                v[r].x *= inv_rms; v[r].y *= inv_rms; v[r].z *= inv_rms; v[r].w *= inv_rms;
                if (has_w) { v[r].x *= w4[r].x; v[r].y *= w4[r].y; v[r].z *= w4[r].z; v[r].w *= w4[r].w; }
            }
        }
#pragma unroll
        for (int r = 0; r < kAqVec; ++r) m = fmaxf(fmaxf(m, fmaxf(fabsf(v[r].x), fabsf(v[r].y))), fmaxf(fabsf(v[r].z), fabsf(v[r].w)));
        m = fmaxf(block_max_nonneg(m, s_f), 1e-6f);      // TenzoEngine.cpp:28-32
        AQT(4);
        const float to_q = 31.0f / m;             // :34
        if (tid == 0) inv[seq] = m / 31.0f;       // :35
        if (words) {                              // the packed fragments gather arbitrary columns: through shared memory
            __syncthreads();
#pragma unroll
            for (int r = 0; r < kAqVec; ++r) {
                const int i = tid + r * kNqThreads;
                if (i < k4) reinterpret_cast<float4*>(s_y)[i] = v[r];
            }
            __syncthreads();
            const int nsets = ((K >> 1) + 15) / 16;
            for (int wd = tid; wd < nsets * 8; wd += kNqThreads) {
                const int s = wd >> 3, tt = (wd >> 1) & 3, odd = wd & 1;
                uint32_t word = 0;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int col = 2 * (16 * s + 4 * i + tt) + odd;
                    const int q = col < K ? (int)roundf(s_y[col] * to_q) : 0;   // :41-42
                    word |= (uint32_t)(uint8_t)(int8_t)(odd ? q : 4 * q) << (8 * i);
                }
                words[(size_t)seq * nsets * 8 + wd] = word;
            }
        }
        if (a_out || sum_out) {
            int part = 0;
#pragma unroll
            for (int r = 0; r < kAqVec; ++r) {
                const int i = tid + r * kNqThreads;
                const int q0 = (int)roundf(v[r].x * to_q), q1 = (int)roundf(v[r].y * to_q), q2 = (int)roundf(v[r].z * to_q), q3 = (int)roundf(v[r].w * to_q);
                if (i < k4) {
                    if (a_out)
                        reinterpret_cast<uint32_t*>(a_out + (size_t)seq * K)[i] =
                            (uint32_t)(uint8_t)(int8_t)q0 | ((uint32_t)(uint8_t)(int8_t)q1 << 8) | ((uint32_t)(uint8_t)(int8_t)q2 << 16) | ((uint32_t)(uint8_t)(int8_t)q3 << 24);
                    part += q0 + q1 + q2 + q3;
                }
            }
            if (sum_out) {                        // sum_k a_k, for kernels that multiply by the unsigned codes w+1
                int* s_i = reinterpret_cast<int*>(s_f);
                __syncthreads();
                if (tid == 0) s_i[0] = 0;
                __syncthreads();
                part = __reduce_add_sync(0xffffffffu, part);
                if ((tid & 31) == 0) atomicAdd(&s_i[0], part);
                __syncthreads();
                if (tid == 0) sum_out[seq] = s_i[0];
            }
        }
        AQT(5);
        return;
    }
    // rows that are longer, or not aligned for 16-byte loads: element by element through shared memory
    if (use_pdl) pdl_wait();
    for (int i = tid; i < K; i += kNqThreads) s_y[i] = __ldcg(xs + i);
    __syncthreads();
    float m = 0.0f;
    if (do_norm) {
        const float ss = sumsq_reference_order(s_y, K, s_f);
        const float inv_rms = rms_inv(ss, K, eps);
        for (int i = tid; i < K; i += kNqThreads) {
            const float y = rms_apply(s_y[i], inv_rms, norm_w, i);
            s_y[i] = y;
            m = fmaxf(m, fabsf(y));
        }
    } else {
        for (int i = tid; i < K; i += kNqThreads) m = fmaxf(m, fabsf(s_y[i]));
    }
    m = fmaxf(block_max_nonneg(m, s_f), 1e-6f);      // TenzoEngine.cpp:28-32
    const float to_q = 31.0f / m;             // :34
    const int nsets = ((K >> 1) + 15) / 16;
    for (int wd = tid; words && wd < nsets * 8; wd += kNqThreads) {
        const int s = wd >> 3, tt = (wd >> 1) & 3, odd = wd & 1;
        uint32_t word = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int col = 2 * (16 * s + 4 * i + tt) + odd;
            const int q = col < K ? (int)roundf(s_y[col] * to_q) : 0;   // :41-42
            word |= (uint32_t)(uint8_t)(int8_t)(odd ? q : 4 * q) << (8 * i);
        }
        words[(size_t)seq * nsets * 8 + wd] = word;
    }
    if (tid == 0) inv[seq] = m / 31.0f;       // :35
    if (a_out || sum_out) {
        int part = 0;
        for (int i = tid; i < K; i += kNqThreads) {
            const int q = (int)roundf(s_y[i] * to_q);
            if (a_out) a_out[(size_t)seq * K + i] = (int8_t)q;
            part += q;
        }
        if (sum_out) {                        // sum_k a_k, for kernels that multiply by the unsigned codes w+1
            int* s_i = reinterpret_cast<int*>(s_f);
            __syncthreads();
            if (tid == 0) s_i[0] = 0;
            __syncthreads();
            part = __reduce_add_sync(0xffffffffu, part);
            if ((tid & 31) == 0) atomicAdd(&s_i[0], part);
            __syncthreads();
            if (tid == 0) sum_out[seq] = s_i[0];
        }
    }
}

cudaError_t launch_act_quant(const float* x, const float* norm_w, int do_norm, float eps, int K, int batch, int x_stride,
                             uint32_t* words, float* inv, int8_t* a_out, int* sum_out, int use_pdl, cudaStream_t st) {
    const size_t smem = (size_t)(K + 96) * sizeof(float);
    if (smem > 48 * 1024) {
        cudaError_t ea = cudaFuncSetAttribute(act_quant_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 80 * 1024);
        if (ea != cudaSuccess) return ea;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)batch, 1, 1);
    cfg.blockDim = dim3(kNqThreads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = use_pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, act_quant_kernel, x, norm_w, do_norm, eps, K, x_stride, words, inv, a_out, sum_out, use_pdl);
}

}  // namespace tz

#ifdef TZ_AQ_TRACE
extern "C" __attribute__((visibility("default"))) int tenzo_trace_act_quant(long long* out) {
    return (int)cudaMemcpyFromSymbol(out, tz::g_aq_trace, sizeof(long long) * 8);
}
#endif

extern "C" int tenzo_cuda_rmsnorm_quant(const float* x, const float* norm_w, int do_norm, float eps, int dim,
                                        int qmax, int batch, int x_stride, float* y_out, int8_t* q_out,
                                        float* scale_out, void* stream) {
    if (!x || dim <= 0 || batch <= 0 || (qmax != 31 && qmax != 127)) return -1;
    if (dim > 16384) return -5;
    const size_t smem = (size_t)(dim + 32) * sizeof(float);
    if (smem > 48 * 1024) {
        cudaError_t ea = cudaFuncSetAttribute(tz::rmsnorm_quant_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 80 * 1024);
        if (ea != cudaSuccess) return (int)ea;
    }
    tz::rmsnorm_quant_kernel<<<batch, tz::kNqThreads, smem, static_cast<cudaStream_t>(stream)>>>(
        x, norm_w, do_norm, eps, dim, qmax, x_stride, y_out, q_out, scale_out);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : (int)e;
}
