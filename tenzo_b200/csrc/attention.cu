// Fused RoPE + INT8 KV append + GQA decode attention for sm_100a (split along the sequence).
//
// Replaces FusedKVCache::forward_attention_raw in int8_fused mode
// (src/runtime/TenzoEngine.cpp:447-533, :657-694, :823-851, :911-913 of the reference).
//
// Work decomposition: one CTA per (sequence, kv head, 256-key chunk). The CTA rotates the group's
// query heads into shared memory, the CTA that owns slot `pos` rotates/quantises/stores the new
// key and value, then every CTA computes scores for its chunk for all query heads that share the
// kv head (K and V bytes are read from HBM once per kv head, not once per query head), a local
// softmax, and the weighted V sum. A second kernel merges the per-chunk (max, sum, vector)
// partials. K/V stay int8 in memory and are widened in registers against their per-token,
// per-head fp32 scales exactly as the reference does: dot * (s_k * 1/sqrt(d)), p * s_v.
//
// Integer results (the appended int8 rows and their scales) are bit-identical to the reference
// given the same q/k/v; the fp32 output differs only by summation order and expf rounding.
#include "common.cuh"
#include "../../include/tenzo_kernels.h"

namespace tz {

constexpr int kAttnThreads = 128;
constexpr int kChunk = 256;          // keys per CTA
constexpr int kHd = 128;             // head_dim (the reference hard-wires 16 x 8 lanes, :833-850)
constexpr int kKRow = 144;           // padded smem row: 16-byte aligned and bank-conflict free

struct AttnLaunch {
    tenzo_attention_args a;
    int n_splits;
    float* part_o;                   // [batch][n_q][n_splits][128]
    float* part_ml;                  // [batch][n_q][n_splits][2]
};

// signed byte -> float without I2F: place (b ^ 0x80) in the mantissa of 2^23, subtract 2^23+128.
__device__ __forceinline__ float s8_to_f(uint32_t word_xor80, int byte) {
    const uint32_t sel = 0x7540u | (uint32_t)byte;
    return __uint_as_float(prmt(word_xor80, 0x4B000000u, sel)) - 8388736.0f;
}

template <int G>
__global__ void __launch_bounds__(kAttnThreads) attn_chunk_kernel(const AttnLaunch L) {
    const tenzo_attention_args& a = L.a;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float* s_q = reinterpret_cast<float*>(smem_raw);              // [G][128]
    float* s_p = s_q + G * kHd;                                   // [G][kChunk]
    float* s_new = s_p + G * kChunk;                              // [2][128] rotated k, v of the new token
    float* s_red = s_new + 2 * kHd;                               // [32]
    unsigned char* s_k = reinterpret_cast<unsigned char*>(s_red + 32);   // [kChunk][kKRow]; later [4][G][128] floats

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int split = blockIdx.x, kvh = blockIdx.y, seq = blockIdx.z;

    if (a.use_pdl) pdl_wait();
    const int pos = a.pos[seq];
    const int T = pos + 1;
    const int t0 = split * kChunk;
    if (t0 >= T) return;
    const int t1 = min(T, t0 + kChunk), nkeys = t1 - t0;

    const size_t row_base = ((size_t)a.layer * a.n_kv + kvh) * a.max_seq;   // :509-510
    int8_t* ck = a.cache_k + (size_t)seq * a.seq_stride_kv + row_base * kHd;
    int8_t* cv = a.cache_v + (size_t)seq * a.seq_stride_kv + row_base * kHd;
    float* sk = a.scale_k + (size_t)seq * a.seq_stride_sc + row_base;
    float* sv = a.scale_v + (size_t)seq * a.seq_stride_sc + row_base;

    // ---- RoPE on the group's query heads (half-split pairs i, i+64; :471-478) ------------------
    const float* cs = a.rope_cos ? a.rope_cos + (size_t)pos * (kHd / 2) : nullptr;
    const float* sn = a.rope_sin ? a.rope_sin + (size_t)pos * (kHd / 2) : nullptr;
    for (int idx = tid; idx < G * (kHd / 2); idx += kAttnThreads) {
        const int g = idx / (kHd / 2), i = idx % (kHd / 2);
        const float* qh = a.q + (size_t)seq * a.q_stride + (size_t)(kvh * G + g) * kHd;
        const float x0 = __ldcg(qh + i), x1 = __ldcg(qh + i + kHd / 2);
        float r0 = x0, r1 = x1;
        if (cs) {
            const float c = cs[i], s = sn[i];
            r0 = __fmaf_rn(x0, c, -(x1 * s));      // fmsub(x0, c, x1*s)
            r1 = __fmaf_rn(x0, s, x1 * c);         // fmadd(x0, s, x1*c)
        }
        s_q[g * kHd + i] = r0;
        s_q[g * kHd + i + kHd / 2] = r1;
    }

    // ---- the CTA that owns slot `pos` appends the new token (:508-533) -------------------------
    if (a.append && pos >= t0 && pos < t1) {
        if (tid < kHd / 2) {
            const float* kh = a.k + (size_t)seq * a.kv_stride + (size_t)kvh * kHd;
            const float x0 = __ldcg(kh + tid), x1 = __ldcg(kh + tid + kHd / 2);
            float r0 = x0, r1 = x1;
            if (cs) {
                const float c = cs[tid], s = sn[tid];
                r0 = __fmaf_rn(x0, c, -(x1 * s));
                r1 = __fmaf_rn(x0, s, x1 * c);
            }
            s_new[tid] = r0;
            s_new[tid + kHd / 2] = r1;
        } else {
            const float* vh = a.v + (size_t)seq * a.kv_stride + (size_t)kvh * kHd;
            const int i = tid - kHd / 2;
            s_new[kHd + i] = __ldcg(vh + i);
            s_new[kHd + i + kHd / 2] = __ldcg(vh + i + kHd / 2);
        }
        __syncthreads();
        if (warp < 2) {                              // warp 0: key row, warp 1: value row
            const float* src = s_new + warp * kHd;
            float amax = 1e-8f;
#pragma unroll
            for (int j = 0; j < 4; ++j) amax = fmaxf(amax, fabsf(src[lane * 4 + j]));
            amax = warp_max(amax);
            const float s = amax / 127.0f;           // :522
            const float inv = 1.0f / s;              // :527
            uint32_t packed = 0;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float qf = fminf(fmaxf(roundf(src[lane * 4 + j] * inv), -128.0f), 127.0f);   // :530
                packed |= ((uint32_t)(uint8_t)(int8_t)(int)qf) << (8 * j);
            }
            int8_t* dst = (warp == 0 ? ck : cv) + (size_t)pos * kHd;
            reinterpret_cast<uint32_t*>(dst)[lane] = packed;
            if (lane == 0) (warp == 0 ? sk : sv)[pos] = s;
        }
    }
    __syncthreads();   // new row and s_q visible to the whole CTA

    // ---- stage the K chunk in shared memory (coalesced 128-bit loads) --------------------------
    for (int idx = tid; idx < nkeys * 8; idx += kAttnThreads) {
        const int r = idx >> 3, c = idx & 7;
        const uint4 v = ld_cg_u4(ck + (size_t)(t0 + r) * kHd + c * 16);
        *reinterpret_cast<uint4*>(s_k + r * kKRow + c * 16) = v;
    }
    __syncthreads();

    // ---- scores: one key per thread, eight FMA lanes per head in the reference's order (:682-691)
    const float sm_scale = 1.0f / sqrtf((float)kHd);   // :660
    for (int kl = tid; kl < nkeys; kl += kAttnThreads) {
        float acc[G][8];
#pragma unroll
        for (int g = 0; g < G; ++g)
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[g][j] = 0.0f;
        const unsigned char* krow = s_k + kl * kKRow;
#pragma unroll 2
        for (int d = 0; d < kHd; d += 16) {
            const uint4 kw = *reinterpret_cast<const uint4*>(krow + d);
            const uint32_t w[4] = {kw.x ^ 0x80808080u, kw.y ^ 0x80808080u, kw.z ^ 0x80808080u, kw.w ^ 0x80808080u};
            float kf[16];
#pragma unroll
            for (int e = 0; e < 16; ++e) kf[e] = s8_to_f(w[e >> 2], e & 3);
#pragma unroll
            for (int g = 0; g < G; ++g) {
                const float4* q4 = reinterpret_cast<const float4*>(s_q + g * kHd + d);
                const float4 qa = q4[0], qb = q4[1], qc = q4[2], qd = q4[3];
                const float qv[16] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w,
                                      qc.x, qc.y, qc.z, qc.w, qd.x, qd.y, qd.z, qd.w};
#pragma unroll
                for (int e = 0; e < 16; ++e) acc[g][e & 7] = __fmaf_rn(qv[e], kf[e], acc[g][e & 7]);
            }
        }
        const float ks = __ldcg(sk + t0 + kl) * sm_scale;
#pragma unroll
        for (int g = 0; g < G; ++g) {
            const float dot = (acc[g][0] + acc[g][1] + acc[g][2] + acc[g][3] + acc[g][4] + acc[g][5] + acc[g][6] + acc[g][7]) * ks;
            s_p[g * kChunk + kl] = dot;
        }
    }
    __syncthreads();

    // ---- chunk-local softmax numerators; fold the V scale into the weight (:826, :844) ----------
    for (int g = warp; g < G; g += kAttnThreads / 32) {
        float mx = -1e30f;
        for (int kl = lane; kl < nkeys; kl += 32) mx = fmaxf(mx, s_p[g * kChunk + kl]);
        mx = warp_max(mx);
        float sum = 0.0f;
        for (int kl = lane; kl < nkeys; kl += 32) {
            const float e = expf(s_p[g * kChunk + kl] - mx);
            sum += e;
            s_p[g * kChunk + kl] = e * __ldcg(sv + t0 + kl);
        }
        sum = warp_sum(sum);
        if (lane == 0) {
            const size_t slot = ((size_t)seq * a.n_q + kvh * G + g) * L.n_splits + split;
            L.part_ml[slot * 2] = mx;
            L.part_ml[slot * 2 + 1] = sum;
        }
    }
    __syncthreads();

    // ---- weighted V sum: lane owns 4 dims, warps take keys round-robin (:842-851) ---------------
    float o[G][4];
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
        for (int j = 0; j < 4; ++j) o[g][j] = 0.0f;
    for (int kl = warp; kl < nkeys; kl += kAttnThreads / 32) {
        const uint32_t vw = __ldcg(reinterpret_cast<const uint32_t*>(cv + (size_t)(t0 + kl) * kHd) + lane) ^ 0x80808080u;
        float vf[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) vf[j] = s8_to_f(vw, j);
#pragma unroll
        for (int g = 0; g < G; ++g) {
            const float wgt = s_p[g * kChunk + kl];
#pragma unroll
            for (int j = 0; j < 4; ++j) o[g][j] = __fmaf_rn(vf[j], wgt, o[g][j]);
        }
    }
    float* s_o = reinterpret_cast<float*>(s_k);     // K staging is dead; reuse as [4][G][128]
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
        for (int j = 0; j < 4; ++j) s_o[(warp * G + g) * kHd + lane * 4 + j] = o[g][j];
    __syncthreads();
    for (int idx = tid; idx < G * kHd; idx += kAttnThreads) {
        const int g = idx / kHd, d = idx % kHd;
        float t = 0.0f;
#pragma unroll
        for (int w = 0; w < kAttnThreads / 32; ++w) t += s_o[(w * G + g) * kHd + d];
        const size_t slot = ((size_t)seq * a.n_q + kvh * G + g) * L.n_splits + split;
        L.part_o[slot * kHd + d] = t;
    }
}

// Merge the per-chunk partials: out = sum_i o_i * exp(m_i - M) / sum_i l_i * exp(m_i - M).
__global__ void __launch_bounds__(kHd) attn_merge_kernel(const AttnLaunch L) {
    const tenzo_attention_args& a = L.a;
    const int qh = blockIdx.x, seq = blockIdx.y, d = threadIdx.x;
    const int T = a.pos[seq] + 1;
    const int active = min((T + kChunk - 1) / kChunk, L.n_splits);
    const size_t base = ((size_t)seq * a.n_q + qh) * L.n_splits;
    float M = -1e30f;
    for (int i = 0; i < active; ++i) M = fmaxf(M, L.part_ml[(base + i) * 2]);
    float num = 0.0f, den = 0.0f;
    for (int i = 0; i < active; ++i) {
        const float w = expf(L.part_ml[(base + i) * 2] - M);
        den += L.part_ml[(base + i) * 2 + 1] * w;
        num += L.part_o[(base + i) * kHd + d] * w;
    }
    a.out[(size_t)seq * a.n_q * kHd + (size_t)qh * kHd + d] = num * (1.0f / den);   // :829-830
}

template <int G>
static cudaError_t launch_attn(const AttnLaunch& L, cudaStream_t st) {
    const size_t smem = (size_t)(G * kHd + G * kChunk + 2 * kHd + 32) * sizeof(float) +
                        (size_t)max(kChunk * kKRow, 4 * G * kHd * (int)sizeof(float));
    cudaError_t e = cudaFuncSetAttribute(attn_chunk_kernel<G>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)L.n_splits, (unsigned)L.a.n_kv, (unsigned)L.a.batch);
    cfg.blockDim = dim3(kAttnThreads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = L.a.use_pdl ? 1 : 0;
    e = cudaLaunchKernelEx(&cfg, attn_chunk_kernel<G>, L);
    if (e != cudaSuccess) return e;
    attn_merge_kernel<<<dim3((unsigned)L.a.n_q, (unsigned)L.a.batch), kHd, 0, st>>>(L);
    return cudaGetLastError();
}

}  // namespace tz

extern "C" size_t tenzo_cuda_attention_scratch_bytes(int batch, int n_q, int max_len) {
    if (batch <= 0 || n_q <= 0 || max_len <= 0) return 0;
    const size_t splits = (size_t)(max_len + tz::kChunk - 1) / tz::kChunk;
    return (size_t)batch * n_q * splits * (tz::kHd + 2) * sizeof(float);
}

extern "C" int tenzo_cuda_attention_int8(const tenzo_attention_args* args, void* stream) {
    using namespace tz;
    if (!args) return -1;
    const tenzo_attention_args& a = *args;
    if (!a.q || !a.out || !a.cache_k || !a.cache_v || !a.scale_k || !a.scale_v || !a.pos || !a.scratch) return -1;
    if (a.append && (!a.k || !a.v)) return -1;
    if (a.head_dim != kHd) return -5;
    if (a.n_q <= 0 || a.n_kv <= 0 || a.n_q % a.n_kv || a.batch <= 0 || a.max_len <= 0 || a.max_len > a.max_seq) return -1;
    if ((a.rope_cos == nullptr) != (a.rope_sin == nullptr)) return -1;
    AttnLaunch L;
    L.a = a;
    if (L.a.q_stride <= 0) L.a.q_stride = a.n_q * kHd;
    if (L.a.kv_stride <= 0) L.a.kv_stride = a.n_kv * kHd;
    L.n_splits = (a.max_len + kChunk - 1) / kChunk;
    L.part_o = static_cast<float*>(a.scratch);
    L.part_ml = L.part_o + (size_t)a.batch * a.n_q * L.n_splits * kHd;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    cudaError_t e;
    switch (a.n_q / a.n_kv) {
        case 1: e = launch_attn<1>(L, st); break;
        case 2: e = launch_attn<2>(L, st); break;
        case 4: e = launch_attn<4>(L, st); break;
        case 8: e = launch_attn<8>(L, st); break;
        default: return -5;
    }
    return e == cudaSuccess ? 0 : (int)e;
}
