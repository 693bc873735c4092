// INT8 LM-head GEMV with fused final RMSNorm + absmax(127) quantiser and greedy argmax; INT8
// embedding-row dequantisation; checkpoint-rows -> TL1 repack.
//
// Replaces, in src/runtime/TenzoEngine.cpp of the reference: compute_logits' int8 branch
// (:1634-1638, :1661-1719), the greedy branch of sample_top_k_top_p (:1745-1755),
// embedding_lookup's int8 branch (:1299-1315) and pack_ternary_weights_raw (:1842-1884).
//
// The LM head is a pure HBM scan (vocab x hidden int8 read once per token): a warp takes one
// vocabulary row at a time with coalesced 128-bit loads, the quantised activation sits in shared
// memory, dp4a accumulates in int32 (exact), and the fp32 logit is (float)acc * (s_x * scale_v)
// with the product of scales formed first, as the reference does (:1717).
#include "common.cuh"
#include "../../include/tenzo_kernels.h"

namespace tz {

constexpr int kLmThreads = 256;
constexpr int kLmWarps = kLmThreads / 32;
constexpr int kLmCtas = 148 * 4;

struct LmBest { float val; int idx; };

__device__ __forceinline__ bool better(float v, int i, float bv, int bi) {
    // greedy argmax keeps the first maximum (:1749 strict '>'): larger value, or same value at a lower index
    return v > bv || (v == bv && i < bi);
}

__global__ void __launch_bounds__(kLmThreads) lm_head_kernel(
    const float* __restrict__ x, const float* __restrict__ norm_w, int do_norm, float eps,
    const int8_t* __restrict__ w, const float* __restrict__ row_scales, int vocab, int hidden, int x_stride,
    float* logits, int32_t* acc_out, LmBest* cta_best, int use_pdl) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float* s_y = reinterpret_cast<float*>(smem_raw);                  // [hidden]
    float* s_f = s_y + hidden;                                        // [32]
    LmBest* s_best = reinterpret_cast<LmBest*>(s_f + 32);             // [kLmWarps]
    int8_t* s_x8 = reinterpret_cast<int8_t*>(s_best + kLmWarps);      // [hidden rounded up to 16]

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, seq = blockIdx.y;
    const int total_warps = gridDim.x * kLmWarps;
    const int gw = blockIdx.x * kLmWarps + warp;
    const int nvec = hidden >> 4;                                     // 16-byte pieces per row
    const bool vec_ok = (hidden & 15) == 0;

    if (use_pdl) pdl_wait();

    // ---- prologue: final RMSNorm + absmax(127) quantiser (:1638, :1666-1678) -------------------
    const float* xs = x + (size_t)seq * x_stride;
    for (int i = tid; i < hidden; i += kLmThreads) s_y[i] = __ldcg(xs + i);
    float m = 0.0f;
    if (do_norm) {
        __syncthreads();
        const float ss = sumsq_reference_order(s_y, hidden, s_f);
        const float inv_rms = rms_inv(ss, hidden, eps);
        for (int i = tid; i < hidden; i += kLmThreads) {
            const float y = rms_apply(s_y[i], inv_rms, norm_w, i);
            s_y[i] = y;
            m = fmaxf(m, fabsf(y));
        }
    } else {
        for (int i = tid; i < hidden; i += kLmThreads) m = fmaxf(m, fabsf(s_y[i]));
    }
    m = fmaxf(block_max(m, s_f), 1e-8f);
    const float s_x = m / 127.0f;                                     // :1671
    const float inv_s = 1.0f / s_x;                                   // :1672
    for (int i = tid; i < hidden; i += kLmThreads)
        s_x8[i] = (int8_t)(int)fminf(fmaxf(roundf(s_y[i] * inv_s), -128.0f), 127.0f);
    __syncthreads();
    if (use_pdl) pdl_launch_dependents();

    // ---- rows ------------------------------------------------------------------------------------
    float best_v = -INFINITY;
    int best_i = 0x7fffffff;
    const uint4* x4 = reinterpret_cast<const uint4*>(s_x8);
    for (int v = gw; v < vocab; v += total_warps) {
        const int8_t* row = w + (size_t)v * hidden;
        int acc = 0;
        if (vec_ok) {
            for (int p = lane; p < nvec; p += 32) {
                const uint4 wv = ld_stream_u4(row + (size_t)p * 16);
                const uint4 xv = x4[p];
                acc = dp4a_ss(wv.x, xv.x, acc);
                acc = dp4a_ss(wv.y, xv.y, acc);
                acc = dp4a_ss(wv.z, xv.z, acc);
                acc = dp4a_ss(wv.w, xv.w, acc);
            }
        } else {
            for (int i = lane; i < hidden; i += 32) acc += (int)row[i] * (int)s_x8[i];
        }
        acc = warp_sum_i(acc);
        if (lane == 0) {
            const float lg = (float)acc * (s_x * row_scales[v]);      // :1717
            if (logits) logits[(size_t)seq * vocab + v] = lg;
            if (acc_out) acc_out[(size_t)seq * vocab + v] = acc;
            if (better(lg, v, best_v, best_i)) { best_v = lg; best_i = v; }
        }
    }
    if (lane == 0) { s_best[warp].val = best_v; s_best[warp].idx = best_i; }
    __syncthreads();
    if (tid == 0) {
        LmBest b = s_best[0];
        for (int i = 1; i < kLmWarps; ++i)
            if (better(s_best[i].val, s_best[i].idx, b.val, b.idx)) b = s_best[i];
        cta_best[(size_t)seq * gridDim.x + blockIdx.x] = b;
    }
}

__global__ void __launch_bounds__(256) argmax_finish_kernel(const LmBest* cta_best, int n, int* argmax_out) {
    __shared__ LmBest s[256];
    const int seq = blockIdx.x, tid = threadIdx.x;
    LmBest b = {-INFINITY, 0x7fffffff};
    for (int i = tid; i < n; i += 256) {
        const LmBest c = cta_best[(size_t)seq * n + i];
        if (better(c.val, c.idx, b.val, b.idx)) b = c;
    }
    s[tid] = b;
    __syncthreads();
    for (int h = 128; h > 0; h >>= 1) {
        if (tid < h && better(s[tid + h].val, s[tid + h].idx, s[tid].val, s[tid].idx)) s[tid] = s[tid + h];
        __syncthreads();
    }
    if (tid == 0) argmax_out[seq] = s[0].idx;
}

__global__ void embedding_i8_kernel(const int8_t* __restrict__ w, const float* __restrict__ row_scales, int hidden,
                                    const int* __restrict__ tokens, float* x, int x_stride) {
    const int seq = blockIdx.x, tok = tokens[seq];
    const int8_t* row = w + (size_t)tok * hidden;
    const float s = row_scales[tok];
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) x[(size_t)seq * x_stride + i] = (float)row[i] * s;   // :1313
}

__global__ void tl1_pack_rows2bit_kernel(const uint8_t* __restrict__ raw, int N, int K, uint8_t* packed) {
    const long long total = (long long)(N / 64) * (K / 2) * 32;
    for (long long o = blockIdx.x * (long long)blockDim.x + threadIdx.x; o < total; o += (long long)gridDim.x * blockDim.x) {
        const int c = (int)(o & 31);
        const long long gk = o >> 5;
        const int k = (int)(gk % (K / 2));
        const int b = (int)(gk / (K / 2));
        auto code = [&](int r, int col) -> uint32_t {           // :1854-1859, value+1 kept as the 2-bit code
            return (raw[(size_t)(r >> 2) * K + col] >> ((r & 3) * 2)) & 3u;
        };
        const int r0 = b * 64 + c, r1 = r0 + 32;
        const uint32_t lo = code(r0, 2 * k) | (code(r0, 2 * k + 1) << 2);
        const uint32_t hi = code(r1, 2 * k) | (code(r1, 2 * k + 1) << 2);
        packed[o] = (uint8_t)(lo | (hi << 4));
    }
}

}  // namespace tz

extern "C" size_t tenzo_cuda_lm_head_scratch_bytes(int batch) {
    return batch > 0 ? (size_t)batch * tz::kLmCtas * sizeof(tz::LmBest) : 0;
}

extern "C" int tenzo_cuda_lm_head_i8(const float* x, const float* norm_w, int do_norm, float eps,
                                     const int8_t* w, const float* row_scales, int vocab, int hidden,
                                     int batch, int x_stride, float* logits, int32_t* acc_out,
                                     int* argmax_out, void* scratch, int use_pdl, void* stream) {
    using namespace tz;
    if (!x || !w || !row_scales || vocab <= 0 || hidden <= 0 || batch <= 0 || !scratch) return -1;
    if (hidden > 16384) return -5;
    if ((hidden & 15) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) != 0) return -1;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const size_t smem = (size_t)(hidden + 32) * sizeof(float) + kLmWarps * sizeof(LmBest) + (((size_t)hidden + 15) & ~(size_t)15);
    if (smem > 48 * 1024) {
        cudaError_t ea = cudaFuncSetAttribute(lm_head_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
        if (ea != cudaSuccess) return (int)ea;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(kLmCtas, (unsigned)batch, 1);
    cfg.blockDim = dim3(kLmThreads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = use_pdl ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, lm_head_kernel, x, norm_w, do_norm, eps, w, row_scales, vocab, hidden,
                                       x_stride, logits, acc_out, static_cast<LmBest*>(scratch), use_pdl);
    if (e != cudaSuccess) return (int)e;
    if (argmax_out) {
        argmax_finish_kernel<<<batch, 256, 0, st>>>(static_cast<const LmBest*>(scratch), kLmCtas, argmax_out);
        e = cudaGetLastError();
    }
    return e == cudaSuccess ? 0 : (int)e;
}

// ---- allocation-free variant ------------------------------------------------------------------
// The per-CTA argmax candidates (kLmCtas x 8 bytes per sequence) normally live in scratch the caller
// allocates. Some hosts may not allocate at all once they are running - a serving loop that has
// handed every byte of device memory to its KV-cache pool, or a plugin slot where the embedding
// application forbids cudaMalloc after start-up - so this variant keeps that scratch in a fixed
// device array that is part of the library image. It costs kLmStaticMaxBatch * kLmCtas * 8 bytes
// (151,552) on every GPU that loads the library, until the process exits.
namespace tz {
constexpr int kLmStaticMaxBatch = 32;
static __device__ __align__(256) unsigned char g_lm_static_scratch[kLmStaticMaxBatch * kLmCtas * sizeof(LmBest)];

// In host code the array's name is only a handle for the runtime, not a device address, so the
// address is looked up once per device (with that device current) and cached.
static void* lm_static_scratch_address(cudaError_t* err) {
    static void* per_device[64] = {nullptr};
    int dev = 0;
    *err = cudaGetDevice(&dev);
    if (*err != cudaSuccess) return nullptr;
    if (dev < 0 || dev >= 64) { *err = cudaErrorInvalidDevice; return nullptr; }
    if (!per_device[dev]) {
        void* p = nullptr;
        *err = cudaGetSymbolAddress(&p, g_lm_static_scratch);
        if (*err != cudaSuccess) return nullptr;
        per_device[dev] = p;
    }
    return per_device[dev];
}
}  // namespace tz

extern "C" int tenzo_cuda_lm_head_i8_static(const float* x, const float* norm_w, int do_norm, float eps,
                                            const int8_t* w, const float* row_scales, int vocab, int hidden,
                                            int batch, int x_stride, float* logits, int32_t* acc_out,
                                            int* argmax_out, int use_pdl, void* stream) {
    if (batch > tz::kLmStaticMaxBatch) return -5;   // beyond the built-in scratch: use tenzo_cuda_lm_head_i8
    if (batch <= 0) return -1;
    cudaError_t e = cudaSuccess;
    void* scratch = tz::lm_static_scratch_address(&e);
    if (!scratch) return (int)e;
    return tenzo_cuda_lm_head_i8(x, norm_w, do_norm, eps, w, row_scales, vocab, hidden, batch, x_stride, logits,
                                 acc_out, argmax_out, scratch, use_pdl, stream);
}

extern "C" int tenzo_cuda_lm_head_static_max_batch(void) { return tz::kLmStaticMaxBatch; }

extern "C" int tenzo_cuda_embedding_i8(const int8_t* w, const float* row_scales, int hidden, const int* tokens,
                                       int batch, float* x, int x_stride, void* stream) {
    if (!w || !row_scales || !tokens || !x || hidden <= 0 || batch <= 0) return -1;
    tz::embedding_i8_kernel<<<batch, 256, 0, static_cast<cudaStream_t>(stream)>>>(w, row_scales, hidden, tokens, x, x_stride);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : (int)e;
}

extern "C" int tenzo_cuda_tl1_pack_rows2bit(const uint8_t* raw, int N, int K, uint8_t* packed, void* stream) {
    if (!raw || !packed || N <= 0 || K <= 0 || (N % 64) || (K & 1)) return -1;
    tz::tl1_pack_rows2bit_kernel<<<148 * 8, 256, 0, static_cast<cudaStream_t>(stream)>>>(raw, N, K, packed);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : (int)e;
}
