// Sampling after the LM head without moving 128 256 logits to the host.
//
// Replaces, together with Engine::sample_candidates, TenzoEngineImpl::sample_top_k_top_p
// (src/runtime/TenzoEngine.cpp:1722-1807 of the reference) for the non-greedy / penalised cases:
//   1. the repetition penalty is applied to the logits on the device, once per occurrence of a past token
//      (:1735-1743: l > 0 ? l / p : l * p);
//   2. the k-th largest logit v* is found by a three-pass radix select over order-preserving integer keys;
//   3. every (value, index) with value >= v* is written out in ascending index order (at most kMaxCandidates).
// The host then runs the reference's streaming top-k over those candidates only. That gives the same heap as the
// full scan: the heap minimum never decreases, so an element below the final threshold is gone by the end, and an
// element at or above it is only ever rejected or popped while the heap holds nothing smaller than v* - at which
// point the heap of the reduced stream is the same set. Softmax, top-p and the draw stay on the host, as there.
#include "common.cuh"
#include "sampler.h"
#include "../../include/tenzo_kernels.h"

namespace tz {

constexpr int kSelThreads = 1024;

// float -> uint32 with the same order as operator< (and -0 == +0)
__device__ __forceinline__ uint32_t order_key(float f) {
    uint32_t b = __float_as_uint(f);
    if (b == 0x80000000u) b = 0u;
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__global__ void penalty_kernel(float* logits, int vocab, const int* tokens, const int* counts, int n, float penalty) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int t = tokens[i];
    if (t < 0 || t >= vocab) return;
    float l = logits[t];
    for (int c = 0; c < counts[i]; ++c) l = l > 0.0f ? l / penalty : l * penalty;
    logits[t] = l;
}

// One CTA. out_count: number of candidates (all logits >= the k-th largest); if it exceeds kMaxCandidates nothing
// else is written. out_val/out_idx: the candidates in ascending index order.
__global__ void __launch_bounds__(kSelThreads) select_candidates_kernel(const float* __restrict__ logits, int vocab, int k,
                                                                         int* out_count, float* out_val, int* out_idx) {
    __shared__ unsigned int hist[2048];
    __shared__ unsigned int s_prefix, s_remaining;
    __shared__ unsigned int s_scan[kSelThreads / 32];
    const int tid = threadIdx.x;
    uint32_t prefix = 0, prefix_mask = 0;
    unsigned int remaining = (unsigned int)k;               // rank (from the top) still to locate inside the current prefix
    const int shifts[3] = {21, 10, 0}, bits[3] = {11, 11, 10};
    for (int pass = 0; pass < 3; ++pass) {
        const int nb = 1 << bits[pass];
        for (int i = tid; i < nb; i += kSelThreads) hist[i] = 0;
        __syncthreads();
        for (int i = tid; i < vocab; i += kSelThreads) {
            const uint32_t key = order_key(logits[i]);
            if ((key & prefix_mask) == prefix) atomicAdd(&hist[(key >> shifts[pass]) & (nb - 1)], 1u);
        }
        __syncthreads();
        if (tid == 0) {                                     // walk the bins from the top until `remaining` is covered
            unsigned int acc = 0;
            int b = nb - 1;
            for (; b > 0; --b) {
                if (acc + hist[b] >= remaining) break;
                acc += hist[b];
            }
            s_prefix = (uint32_t)b;
            s_remaining = remaining - acc;
        }
        __syncthreads();
        prefix |= s_prefix << shifts[pass];
        prefix_mask |= (uint32_t)(nb - 1) << shifts[pass];
        remaining = s_remaining;
        __syncthreads();
    }
    const uint32_t threshold = prefix;                      // key of the k-th largest logit
    // candidates in ascending index order: contiguous slice per thread, block scan of the counts
    const int per = (vocab + kSelThreads - 1) / kSelThreads;
    const int i0 = tid * per, i1 = min(vocab, i0 + per);
    unsigned int mine = 0;
    for (int i = i0; i < i1; ++i) mine += order_key(logits[i]) >= threshold ? 1u : 0u;
    unsigned int incl = mine;
    const int lane = tid & 31, warp = tid >> 5;
    for (int o = 1; o < 32; o <<= 1) {
        const unsigned int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
    }
    if (lane == 31) s_scan[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        unsigned int w = lane < kSelThreads / 32 ? s_scan[lane] : 0u, wi = w;
        for (int o = 1; o < 32; o <<= 1) {
            const unsigned int v = __shfl_up_sync(0xffffffffu, wi, o);
            if (lane >= o) wi += v;
        }
        if (lane < kSelThreads / 32) s_scan[lane] = wi - w;  // exclusive warp offsets
        if (lane == 31) s_remaining = wi;                    // total
    }
    __syncthreads();
    const unsigned int total = s_remaining;
    if (tid == 0) *out_count = (int)total;
    if (total > (unsigned int)kMaxCandidates) return;
    unsigned int pos = s_scan[warp] + incl - mine;
    for (int i = i0; i < i1; ++i) {
        const float l = logits[i];
        if (order_key(l) >= threshold) {
            out_val[pos] = l;
            out_idx[pos] = i;
            ++pos;
        }
    }
}

cudaError_t launch_penalty(float* logits, int vocab, const int* tokens, const int* counts, int n, float penalty, cudaStream_t st) {
    if (n <= 0) return cudaSuccess;
    penalty_kernel<<<(n + 127) / 128, 128, 0, st>>>(logits, vocab, tokens, counts, n, penalty);
    return cudaGetLastError();
}

cudaError_t launch_select_candidates(const float* logits, int vocab, int k, int* out_count, float* out_val, int* out_idx, cudaStream_t st) {
    select_candidates_kernel<<<1, kSelThreads, 0, st>>>(logits, vocab, k, out_count, out_val, out_idx);
    return cudaGetLastError();
}

}  // namespace tz

extern "C" int tenzo_cuda_repetition_penalty(float* logits, int vocab, const int* tokens, const int* counts, int n, float penalty, void* stream) {
    if (!logits || vocab <= 0 || n < 0 || (n > 0 && (!tokens || !counts))) return -1;
    const cudaError_t e = tz::launch_penalty(logits, vocab, tokens, counts, n, penalty, static_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? 0 : (int)e;
}

extern "C" int tenzo_cuda_topk_candidates(const float* logits, int vocab, int k, int* count, float* values, int* indices, void* stream) {
    if (!logits || !count || !values || !indices || vocab <= 0 || k < 1 || k > vocab) return -1;
    const cudaError_t e = tz::launch_select_candidates(logits, vocab, k, count, values, indices, static_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? 0 : (int)e;
}

extern "C" int tenzo_cuda_topk_max_candidates(void) { return tz::kMaxCandidates; }
