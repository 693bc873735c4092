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
#include "lm_head.cuh"
#include "../../include/tenzo_kernels.h"

namespace tz {

constexpr int kLmThreads = 256;
constexpr int kLmWarps = kLmThreads / 32;
constexpr int kLmCtas = 148 * 4;
constexpr int kLmInFlight = 5;        // 16-byte loads per lane issued back to back


// Sum of squares in the reference's order (see common.cuh) computed by ONE warp over a vector in
// shared memory: lanes 0-7 run the eight chains, the lane sums are then added left to right.
__device__ __forceinline__ float warp_sumsq_reference_order(const float* x, int dim, int lane) {
    const int n8 = dim & ~7;
    float s = 0.0f;
    if (lane < 8) {
        int i = lane;
        for (; i + 8 * 15 < n8; i += 8 * 16) {
            float v[16];
#pragma unroll
            for (int u = 0; u < 16; ++u) v[u] = x[i + 8 * u];
#pragma unroll
            for (int u = 0; u < 16; ++u) v[u] = __fmul_rn(v[u], v[u]);
#pragma unroll
            for (int u = 0; u < 16; ++u) s = __fadd_rn(s, v[u]);
        }
        for (; i < n8; i += 8) s = __fadd_rn(s, __fmul_rn(x[i], x[i]));
    }
    float t = __shfl_sync(0xffffffffu, s, 0);
#pragma unroll
    for (int j = 1; j < 8; ++j) t = __fadd_rn(t, __shfl_sync(0xffffffffu, s, j));
    for (int i = n8; i < dim; ++i) t = __fadd_rn(t, __fmul_rn(x[i], x[i]));
    return t;
}

// NS sequences per CTA (1 or 8). With 8, warp n prepares sequence n (norm, quantise) and every
// vocabulary row read from HBM is used for all eight sequences.
template <int NS>
__global__ void __launch_bounds__(kLmThreads, NS == 1 ? 4 : 0) lm_head_kernel(
    const float* __restrict__ x, const float* __restrict__ norm_w, int do_norm, float eps,
    const int8_t* __restrict__ w, const float* __restrict__ row_scales, int vocab, int hidden, int x_stride, int batch,
    float* logits, int32_t* acc_out, LmBest* cta_best, int use_pdl) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int hpad = (hidden + 15) & ~15;
    float* s_y = reinterpret_cast<float*>(smem_raw);                  // [NS][hidden]
    float* s_sx = s_y + (size_t)NS * hidden;                          // [NS] activation scales (+ pad to 8 floats)
    LmBest* s_best = reinterpret_cast<LmBest*>(s_sx + 8);             // [kLmWarps][NS]
    int8_t* s_x8 = reinterpret_cast<int8_t*>(s_best + kLmWarps * NS); // [NS][hpad]
    s_x8 = reinterpret_cast<int8_t*>((reinterpret_cast<uintptr_t>(s_x8) + 15) & ~uintptr_t(15));

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, seq0 = blockIdx.y * NS;
    const int total_warps = gridDim.x * kLmWarps;
    const int gw = blockIdx.x * kLmWarps + warp;
    const int nvec = hidden >> 4;                                     // 16-byte pieces per row
    const bool vec_ok = (hidden & 15) == 0;

    if (use_pdl) pdl_wait();

    // ---- prologue: final RMSNorm + absmax(127) quantiser (:1638, :1666-1678), one warp per sequence
    for (int n = warp; n < NS; n += kLmWarps) {
        float* y = s_y + (size_t)n * hidden;
        int8_t* x8 = s_x8 + (size_t)n * hpad;
        if (seq0 + n >= batch) {
            for (int i = lane; i < hpad; i += 32) x8[i] = 0;
            if (lane == 0) s_sx[n] = 0.0f;
            continue;
        }
        const float* xs = x + (size_t)(seq0 + n) * x_stride;
        for (int i = lane; i < hidden; i += 32) y[i] = __ldcg(xs + i);
        __syncwarp();
        float m = 0.0f;
        if (do_norm) {
            const float ss = warp_sumsq_reference_order(y, hidden, lane);
            const float inv_rms = rms_inv(ss, hidden, eps);
            for (int i = lane; i < hidden; i += 32) {
                const float v = rms_apply(y[i], inv_rms, norm_w, i);
                y[i] = v;
                m = fmaxf(m, fabsf(v));
            }
        } else {
            for (int i = lane; i < hidden; i += 32) m = fmaxf(m, fabsf(y[i]));
        }
        m = fmaxf(warp_max(m), 1e-8f);
        const float sx = m / 127.0f;                                  // :1671
        const float inv_s = 1.0f / sx;                                // :1672
        for (int i = lane; i < hpad; i += 32)
            x8[i] = i < hidden ? (int8_t)(int)fminf(fmaxf(roundf(y[i] * inv_s), -128.0f), 127.0f) : (int8_t)0;
        if (lane == 0) s_sx[n] = sx;
    }
    __syncthreads();
    if (use_pdl) pdl_launch_dependents();

    // ---- rows: lane n keeps the running best of sequence n ---------------------------------------
    float best_v = -INFINITY;
    int best_i = 0x7fffffff;
    const float my_sx = lane < NS ? s_sx[lane] : 0.0f;
    for (int v = gw; v < vocab; v += total_warps) {
        const int8_t* row = w + (size_t)v * hidden;
        int acc[NS];
#pragma unroll
        for (int n = 0; n < NS; ++n) acc[n] = 0;
        if (vec_ok) {
            if constexpr (NS == 1) {
                // every load of a row leaves before the first is used (kLmInFlight x 512 bytes per warp: a 2560-byte row
                // is five): with one 16-byte load per lane in flight the kernel moved 3.9 TB/s, bound by latency, not by HBM
                for (int p0 = lane; p0 < nvec; p0 += 32 * kLmInFlight) {
                    uint4 wv[kLmInFlight];
#pragma unroll
                    for (int u = 0; u < kLmInFlight; ++u) {
                        const int p = p0 + 32 * u;
                        wv[u] = p < nvec ? ld_stream_u4(row + (size_t)p * 16) : make_uint4(0u, 0u, 0u, 0u);
                    }
#pragma unroll
                    for (int u = 0; u < kLmInFlight; ++u) {
                        const int p = p0 + 32 * u;
                        if (p < nvec) {
                            const uint4 xv = reinterpret_cast<const uint4*>(s_x8)[p];
                            acc[0] = dp4a_ss(wv[u].x, xv.x, acc[0]);
                            acc[0] = dp4a_ss(wv[u].y, xv.y, acc[0]);
                            acc[0] = dp4a_ss(wv[u].z, xv.z, acc[0]);
                            acc[0] = dp4a_ss(wv[u].w, xv.w, acc[0]);
                        }
                    }
                }
            } else {                                  // eight sequences per row: 32 dp4a per load
                for (int p = lane; p < nvec; p += 32) {
                    const uint4 wv = ld_stream_u4(row + (size_t)p * 16);
#pragma unroll
                    for (int n = 0; n < NS; ++n) {
                        const uint4 xv = reinterpret_cast<const uint4*>(s_x8 + (size_t)n * hpad)[p];
                        acc[n] = dp4a_ss(wv.x, xv.x, acc[n]);
                        acc[n] = dp4a_ss(wv.y, xv.y, acc[n]);
                        acc[n] = dp4a_ss(wv.z, xv.z, acc[n]);
                        acc[n] = dp4a_ss(wv.w, xv.w, acc[n]);
                    }
                }
            }
        } else {
            for (int i = lane; i < hidden; i += 32) {
                const int wi = (int)row[i];
#pragma unroll
                for (int n = 0; n < NS; ++n) acc[n] += wi * (int)s_x8[(size_t)n * hpad + i];
            }
        }
        int mine = 0;
#pragma unroll
        for (int n = 0; n < NS; ++n) {
            const int t = warp_sum_i(acc[n]);
            if (lane == n) mine = t;
        }
        if (lane < NS && seq0 + lane < batch) {
            const float lg = (float)mine * (my_sx * row_scales[v]);   // :1717
            if (logits) logits[(size_t)(seq0 + lane) * vocab + v] = lg;
            if (acc_out) acc_out[(size_t)(seq0 + lane) * vocab + v] = mine;
            if (better(lg, v, best_v, best_i)) { best_v = lg; best_i = v; }
            if (v == 0 && lg != lg) { best_v = INFINITY; best_i = 0; }   // a NaN at index 0 is never displaced (strict '>', :1747-1753)
        }
    }
    if (lane < NS) { s_best[warp * NS + lane].val = best_v; s_best[warp * NS + lane].idx = best_i; }
    __syncthreads();
    if (tid < NS && seq0 + tid < batch) {
        LmBest b = s_best[tid];
        for (int i = 1; i < kLmWarps; ++i)
            if (better(s_best[i * NS + tid].val, s_best[i * NS + tid].idx, b.val, b.idx)) b = s_best[i * NS + tid];
        cta_best[(size_t)(seq0 + tid) * gridDim.x + blockIdx.x] = b;
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
    // nothing compared greater (every logit NaN or -inf): the reference's scan stays at index 0 (:1746)
    if (tid == 0) argmax_out[seq] = s[0].idx == 0x7fffffff ? 0 : s[0].idx;
}

// vocab > 0: ids outside [0, vocab) are read as row 0 instead of reaching past the table.
__global__ void embedding_i8_kernel(const int8_t* __restrict__ w, const float* __restrict__ row_scales, int hidden,
                                    const int* __restrict__ tokens, float* x, int x_stride, int vocab) {
    const int seq = blockIdx.x;
    int tok = tokens[seq];
    if (vocab > 0 && (tok < 0 || tok >= vocab)) tok = 0;
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

namespace tz {
// tensor-core path for 16 or more sequences (lm_head_umma.cu)
bool lm_head_umma_applicable(int vocab, int hidden, int batch, const int8_t* w, const float* logits);
int launch_lm_head_umma(const int8_t* q8, const float* sx, const int8_t* w, const float* row_scales, int vocab, int hidden, int batch,
                        float* logits, int32_t* acc_out, LmBest* cand, int use_pdl, cudaStream_t st);
int lm_head_umma_take_timeouts();
}

// Per sequence: argmax candidates for up to kLmuMaxTiles vocabulary tiles (covers the kLmCtas candidates of the
// warp-per-row kernel), the quantised activation vector (hidden <= 16384) and its scale.
extern "C" size_t tenzo_cuda_lm_head_scratch_bytes(int batch) {
    return batch > 0 ? (size_t)batch * (tz::kLmuMaxTiles * sizeof(tz::LmBest) + 16384 + 16) + 64 : 0;
}

extern "C" int tenzo_cuda_lm_head_take_timeouts(void) { return tz::lm_head_umma_take_timeouts(); }

static int lm_head_launch(const float* x, const float* norm_w, int do_norm, float eps,
                          const int8_t* w, const float* row_scales, int vocab, int hidden,
                          int batch, int x_stride, float* logits, int32_t* acc_out,
                          int* argmax_out, void* scratch, int use_pdl, void* stream, bool allow_batched, bool allow_umma) {
    using namespace tz;
    if (!x || !w || !row_scales || vocab <= 0 || hidden <= 0 || batch <= 0 || !scratch) return -1;
    if (hidden > 16384) return -5;
    if ((hidden & 15) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) != 0) return -1;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (allow_umma && lm_head_umma_applicable(vocab, hidden, batch, w, logits)) {
        const int n_tiles = (vocab + 127) / 128;
        LmBest* cand = static_cast<LmBest*>(scratch);
        int8_t* q8 = reinterpret_cast<int8_t*>(static_cast<unsigned char*>(scratch) + (((size_t)batch * n_tiles * sizeof(LmBest) + 15) & ~(size_t)15));
        float* sx = reinterpret_cast<float*>(q8 + (size_t)batch * hidden);
        int rc = tenzo_cuda_rmsnorm_quant(x, norm_w, do_norm, eps, hidden, 127, batch, x_stride, nullptr, q8, sx, stream);
        if (rc) return rc;
        rc = launch_lm_head_umma(q8, sx, w, row_scales, vocab, hidden, batch, logits, acc_out, argmax_out ? cand : nullptr, use_pdl, st);
        if (rc) return rc;
        if (argmax_out) {
            argmax_finish_kernel<<<batch, 256, 0, st>>>(cand, n_tiles, argmax_out);
            if (cudaGetLastError() != cudaSuccess) return (int)cudaErrorLaunchFailure;
        }
        return 0;
    }
    const size_t hpad = ((size_t)hidden + 15) & ~(size_t)15;
    auto smem_for = [&](int ns) { return (size_t)ns * hidden * sizeof(float) + 8 * sizeof(float) + (size_t)kLmWarps * ns * sizeof(LmBest) + ns * hpad + 16; };
    const bool eight = allow_batched && batch > 1 && smem_for(8) <= 200 * 1024;   // eight sequences share each row read
    const size_t smem = smem_for(eight ? 8 : 1);
    if (smem > 48 * 1024) {
        cudaError_t ea = eight ? cudaFuncSetAttribute(lm_head_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
                               : cudaFuncSetAttribute(lm_head_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (ea != cudaSuccess) return (int)ea;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(kLmCtas, (unsigned)(eight ? (batch + 7) / 8 : batch), 1);
    cfg.blockDim = dim3(kLmThreads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = use_pdl ? 1 : 0;
    cudaError_t e = eight ? cudaLaunchKernelEx(&cfg, lm_head_kernel<8>, x, norm_w, do_norm, eps, w, row_scales, vocab, hidden, x_stride,
                                               batch, logits, acc_out, static_cast<LmBest*>(scratch), use_pdl)
                          : cudaLaunchKernelEx(&cfg, lm_head_kernel<1>, x, norm_w, do_norm, eps, w, row_scales, vocab, hidden, x_stride,
                                               batch, logits, acc_out, static_cast<LmBest*>(scratch), use_pdl);
    if (e != cudaSuccess) return (int)e;
    if (argmax_out) {
        argmax_finish_kernel<<<batch, 256, 0, st>>>(static_cast<const LmBest*>(scratch), kLmCtas, argmax_out);
        e = cudaGetLastError();
    }
    return e == cudaSuccess ? 0 : (int)e;
}

extern "C" int tenzo_cuda_lm_head_i8(const float* x, const float* norm_w, int do_norm, float eps,
                                     const int8_t* w, const float* row_scales, int vocab, int hidden,
                                     int batch, int x_stride, float* logits, int32_t* acc_out,
                                     int* argmax_out, void* scratch, int use_pdl, void* stream) {
    return lm_head_launch(x, norm_w, do_norm, eps, w, row_scales, vocab, hidden, batch, x_stride, logits, acc_out, argmax_out,
                          scratch, use_pdl, stream, true, true);
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
    return lm_head_launch(x, norm_w, do_norm, eps, w, row_scales, vocab, hidden, batch, x_stride, logits,
                          acc_out, argmax_out, scratch, use_pdl, stream, true, false);   // built-in scratch: warp-per-row kernel only
}

extern "C" int tenzo_cuda_lm_head_static_max_batch(void) { return tz::kLmStaticMaxBatch; }

extern "C" int tenzo_cuda_embedding_i8(const int8_t* w, const float* row_scales, int hidden, const int* tokens,
                                       int batch, float* x, int x_stride, int vocab, void* stream) {
    if (!w || !row_scales || !tokens || !x || hidden <= 0 || batch <= 0 || vocab < 0) return -1;
    tz::embedding_i8_kernel<<<batch, 256, 0, static_cast<cudaStream_t>(stream)>>>(w, row_scales, hidden, tokens, x, x_stride, vocab);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : (int)e;
}

extern "C" int tenzo_cuda_tl1_pack_rows2bit(const uint8_t* raw, int N, int K, uint8_t* packed, void* stream) {
    if (!raw || !packed || N <= 0 || K <= 0 || (N % 64) || (K & 1)) return -1;
    tz::tl1_pack_rows2bit_kernel<<<148 * 8, 256, 0, static_cast<cudaStream_t>(stream)>>>(raw, N, K, packed);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : (int)e;
}
