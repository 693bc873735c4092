// INT8 KV-cache GQA decode attention, tolerance mode: the same function as attention.cu (RoPE, INT8 append, softmax(QK)V
// with per-token, per-head scales; FusedKVCache::forward_attention_raw, src/runtime/TenzoEngine.cpp:447-533, :657-694,
// :823-851 of the reference) evaluated in whatever order the hardware likes, for callers that accept the 1e-3 relative
// agreement the floating-point outputs are specified to (attention.cu reproduces the reference's rounding bit for bit and
// pays for it with sequential sums over the keys).
//
//   * The keys of a (sequence, kv head) are split over several CTAs and, inside a CTA, over four warps that never
//     synchronise with one another: each warp streams its own 32-key blocks (K tile, V tile, scales) through a private
//     three-stage ring filled by TMA (2-D tiles with the 128-byte swizzle, no multicast) and keeps a running
//     (max, sum, output) triple per query head - the usual online softmax. Partial triples are merged by log-sum-exp,
//     first across the warps of a CTA, then across CTAs by a second small kernel.
//   * Both products run on the tensor cores as fp16 MMAs with fp32 accumulation (mma.sync.m16n8k16). INT8 K and V are
//     exact in fp16; bytes become halves with one PRMT and one HSUB2 per pair (0x64xx is 1024 + x in fp16). The rotated
//     query enters as two fp16 parts (hi + lo, two MMAs per step), the weights p_t * s_v[t] are rounded to fp16 after the
//     exponential (scaled by 2^10 so that small weights stay normal numbers): a relative error of 2^-11 per weight that
//     averages out over the keys.
//   * Q.K^T: A = the query heads of the kv head (rows 0..G-1 of 16), B = keys straight from the swizzled tile (a lane's
//     32-bit word is two k-pairs; the k order inside a 16-wide step is permuted identically in A). P.V: the score
//     accumulators are already in A-fragment layout; B comes from ldmatrix.trans over the INT8 tile read as 16-bit
//     elements, which hands each lane two keys x two adjacent dims that one PRMT regroups into (key pair, even dim) and
//     (key pair, odd dim) - so even and odd dims go to separate 8-wide column tiles, undone at the final store.
//   * exp is ex2.approx on scores pre-multiplied by log2(e).
// The new token's K/V row is rotated, quantised and stored by a small kernel in front (same arithmetic and bits as the
// exact path, so the cache contents do not depend on the mode).
#include <cuda.h>
#include <cuda_fp16.h>

#include <cstring>
#include <utility>

#include "attn_common.cuh"
#include "common.cuh"
#include "../../include/tenzo_kernels.h"

namespace tz {

constexpr int kFaWarps = 4;
constexpr int kFaThreads = kFaWarps * 32;
constexpr int kFaBlk = 32;                      // keys per warp step
constexpr int kFaStages = 3;
constexpr int kFaTile = kFaBlk * kHd;           // 4096 bytes
constexpr float kFaPScale = 1024.0f;            // weights are scaled by 2^10 before they are rounded to fp16

struct FaLaunch {
    tenzo_attention_args a;
    int n_splits, split_keys, group;
    float* part_o;       // [batch][n_kv][n_splits][G][128] un-normalised outputs (scaled by kFaPScale)
    float* part_ml;      // [batch][n_kv][n_splits][G][2]   running maximum (log2 domain) and sum
};

__device__ int g_fa_timeouts = 0;

__device__ __forceinline__ void fa_tma_tile(void* dst, const CUtensorMap* map, int row0, int seq, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                 ::"r"(smem_addr(dst)), "l"(map), "r"(0), "r"(row0), "r"(seq), "r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ float fa_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t fa_pack_h2(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
}
// two signed bytes of `w_xor80` (already XORed with 0x80808080), picked by `sel`, as two exact halves
__device__ __forceinline__ uint32_t fa_bytes_to_h2(uint32_t w_xor80, uint32_t sel) {
    const uint32_t biased = prmt(w_xor80, 0x64646464u, sel);     // 0x64xx = 1024 + xx
    uint32_t r;
    asm("sub.f16x2 %0, %1, %2;" : "=r"(r) : "r"(biased), "r"(0x64806480u));   // - (1024 + 128)
    return r;
}
__device__ __forceinline__ void fa_mma_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// New token's K (rotated) and V rows: quantise and store at pos[seq] (:459-533), one warp per (sequence, kv head, K|V).
__global__ void __launch_bounds__(64) fa_append_kernel(const tenzo_attention_args a) {
    const int seq = blockIdx.x, kvh = blockIdx.y, is_v = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (a.use_pdl) {                         // resident while the previous kernel drains; nothing is touched before it has completed
        pdl_launch_dependents();
        pdl_wait();
    }
    const int pos = a.pos[seq];
    if (pos < 0 || pos >= a.max_seq) return;
    const float* src = (is_v ? a.v : a.k) + (size_t)seq * a.kv_stride + (size_t)kvh * kHd;
    float x[4];
    if (is_v || !a.rope_cos) {
#pragma unroll
        for (int j = 0; j < 4; ++j) x[j] = __ldcg(src + lane * 4 + j);
    } else {
        const float* cs = a.rope_cos + (size_t)pos * 64;
        const float* sn = a.rope_sin + (size_t)pos * 64;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int e = lane * 4 + j, i = e & 63;
            const float x0 = __ldcg(src + i), x1 = __ldcg(src + i + 64), c = cs[i], sg = sn[i];
            x[j] = e < 64 ? __fmaf_rn(x0, c, -(x1 * sg)) : __fmaf_rn(x0, sg, x1 * c);      // :475-476
        }
    }
    float amax = 1e-8f;
#pragma unroll
    for (int j = 0; j < 4; ++j) amax = fmaxf(amax, fabsf(x[j]));
    amax = warp_max(amax);
    const float sc = amax / 127.0f;           // :522
    const float inv = 1.0f / sc;              // :527
    uint32_t packed = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float qf = fminf(fmaxf(roundf(x[j] * inv), -128.0f), 127.0f);   // :530
        packed |= ((uint32_t)(uint8_t)(int8_t)(int)qf) << (8 * j);
    }
    const size_t row = (size_t)seq * a.seq_stride_sc + ((size_t)a.layer * a.n_kv + kvh) * a.max_seq + pos;
    const size_t byte0 = (size_t)seq * a.seq_stride_kv + (((size_t)a.layer * a.n_kv + kvh) * a.max_seq + pos) * kHd;
    reinterpret_cast<uint32_t*>((is_v ? a.cache_v : a.cache_k) + byte0)[lane] = packed;
    if (lane == 0) (is_v ? a.scale_v : a.scale_k)[row] = sc;
}

template <int G>
__global__ void __launch_bounds__(kFaThreads, 2) attn_fast_kernel(const FaLaunch L, const __grid_constant__ CUtensorMap kmap,
                                                                   const __grid_constant__ CUtensorMap vmap) {
    const tenzo_attention_args& a = L.a;
    extern __shared__ __align__(1024) unsigned char fa_smem[];
    // [warp][stage][K tile 4096 | V tile 4096] | scales [warp][stage][2][32] floats | q [G][128] floats | barriers
    const uint32_t base_off = ((smem_addr(fa_smem) + 1023u) & ~1023u) - smem_addr(fa_smem);
    unsigned char* s_tiles = fa_smem + base_off;
    float* s_scales = reinterpret_cast<float*>(s_tiles + kFaWarps * kFaStages * 2 * kFaTile);
    float* s_q = s_scales + kFaWarps * kFaStages * 64;
    uint64_t* s_bar = reinterpret_cast<uint64_t*>(s_q + 8 * kHd);            // [warp][stage]

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t4 = lane & 3;
    const int split = blockIdx.x, kvh = blockIdx.y, seq = blockIdx.z;
    if (a.use_pdl) {
        pdl_launch_dependents();
        pdl_wait();
    }
    const int pos = a.pos[seq];
    const int T = pos + 1;
    const int c_begin = split * L.split_keys, c_end = min(T, c_begin + L.split_keys);
    const size_t item = ((size_t)seq * a.n_kv + kvh) * L.n_splits + split;
    float* po = L.part_o + item * G * kHd;
    float* pml = L.part_ml + item * G * 2;
    if (pos < 0 || pos >= a.max_len || c_begin >= c_end) {                   // nothing here: a neutral partial
        if (tid < G) { pml[tid * 2] = -INFINITY; pml[tid * 2 + 1] = 0.0f; }
        for (int i = tid; i < G * kHd; i += kFaThreads) po[i] = 0.0f;
        if (pos < 0 || pos >= a.max_len) atomicExch(&g_fa_timeouts, 2);
        return;
    }
    const int row_base = (int)(((size_t)a.layer * a.n_kv + kvh) * a.max_seq);
    const float* sk = a.scale_k + (size_t)seq * a.seq_stride_sc + row_base;
    const float* sv = a.scale_v + (size_t)seq * a.seq_stride_sc + row_base;
    const int n_blocks = (c_end - c_begin + kFaBlk - 1) / kFaBlk;
    const int my_blocks = warp < n_blocks ? (n_blocks - warp + kFaWarps - 1) / kFaWarps : 0;
    unsigned char* my_tiles = s_tiles + (size_t)warp * kFaStages * 2 * kFaTile;
    float* my_scales = s_scales + warp * kFaStages * 64;
    uint64_t* my_bar = s_bar + warp * kFaStages;

    auto issue = [&](int k) {                 // this warp's k-th block into stage k % kFaStages (lane 0 only)
        const int st = k % kFaStages;
        const int t0 = c_begin + (warp + k * kFaWarps) * kFaBlk;
        const int ns = min(kFaBlk, a.max_seq - t0);                            // scale entries that exist
        mbar_expect_tx(&my_bar[st], 2u * kFaTile + 2u * (unsigned)ns * 4u);
        fa_tma_tile(my_tiles + (size_t)st * 2 * kFaTile, &kmap, row_base + t0, seq, &my_bar[st]);
        fa_tma_tile(my_tiles + (size_t)st * 2 * kFaTile + kFaTile, &vmap, row_base + t0, seq, &my_bar[st]);
        bulk_g2s(my_scales + st * 64, sk + t0, (unsigned)ns * 4u, &my_bar[st]);
        bulk_g2s(my_scales + st * 64 + 32, sv + t0, (unsigned)ns * 4u, &my_bar[st]);
    };
    if (lane == 0) {
        for (int s = 0; s < kFaStages; ++s) mbar_init(&my_bar[s], 1);
        mbar_init_fence();
        for (int k = 0; k < kFaStages && k < my_blocks; ++k) issue(k);
    }

    // ---- query heads of this kv head: rotate (:459-480), round to fp16, keep as A fragments ------------------------
    {
        const float* cs = a.rope_cos ? a.rope_cos + (size_t)pos * (kHd / 2) : nullptr;
        const float* sn = a.rope_sin ? a.rope_sin + (size_t)pos * (kHd / 2) : nullptr;
        for (int idx = tid; idx < G * (kHd / 2); idx += kFaThreads) {
            const int h = idx / (kHd / 2), i = idx % (kHd / 2);
            const float* qh = a.q + (size_t)seq * a.q_stride + (size_t)(kvh * G + h) * kHd;
            float r0, r1;
            rope_pair(__ldcg(qh + i), __ldcg(qh + i + kHd / 2), cs, sn, i, r0, r1);
            s_q[h * kHd + i] = r0;
            s_q[h * kHd + i + kHd / 2] = r1;
        }
    }
    __syncthreads();
    // q = hi + lo with both parts in fp16: the product with the (exact) keys is then accurate to about 2^-22 of |q||k|,
    // where a single rounding of q to fp16 (2^-11) would put most of the tolerance budget into the scores
    uint32_t qa[8][2], ql[8][2];
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
        qa[ks][0] = qa[ks][1] = ql[ks][0] = ql[ks][1] = 0u;
        if (g < G) {
            const float4 v = *reinterpret_cast<const float4*>(s_q + g * kHd + ks * 16 + t4 * 4);
            qa[ks][0] = fa_pack_h2(v.x, v.y);        // k = 2*t4, 2*t4+1      <-> dims 16ks + 4t4 + {0,1}
            qa[ks][1] = fa_pack_h2(v.z, v.w);        // k = 2*t4+8, 2*t4+9    <-> dims 16ks + 4t4 + {2,3}
            const float2 h0 = __half22float2(*reinterpret_cast<const __half2*>(&qa[ks][0]));
            const float2 h1 = __half22float2(*reinterpret_cast<const __half2*>(&qa[ks][1]));
            ql[ks][0] = fa_pack_h2(v.x - h0.x, v.y - h0.y);
            ql[ks][1] = fa_pack_h2(v.z - h1.x, v.w - h1.y);
        }
    }

    const float sm_l2e = (1.0f / sqrtf((float)kHd)) * 1.4426950408889634f;   // softmax scale (:660) times log2(e)
    float m_run = -INFINITY, l_run = 0.0f;       // row g (query head g); l is this lane's share until the end
    float acc[8][2][4];                          // [16-byte dim chunk][even | odd dim][mma C regs]; rows g+8 stay zero
#pragma unroll
    for (int c = 0; c < 8; ++c)
#pragma unroll
        for (int e = 0; e < 2; ++e)
#pragma unroll
            for (int r = 0; r < 4; ++r) acc[c][e][r] = 0.0f;
    bool timed_out = false;

    for (int k = 0; k < my_blocks; ++k) {
        const int st = k % kFaStages;
        const int t0 = c_begin + (warp + k * kFaWarps) * kFaBlk;
        if (lane == 0 && !mbar_wait_bounded(&my_bar[st], (unsigned)(k / kFaStages) & 1u)) timed_out = true;
        __syncwarp();
        const unsigned char* kt = my_tiles + (size_t)st * 2 * kFaTile;
        const unsigned char* vt = kt + kFaTile;
        const float* sc_k = my_scales + st * 64;
        const float* sc_v = sc_k + 32;

        // ---- S = Q K^T: rows = query heads, columns = the block's 32 keys (four 8-key tiles) ------------------------
        float s[4][4];
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
            for (int r = 0; r < 4; ++r) s[nt][r] = 0.0f;
            const unsigned char* krow = kt + (size_t)(nt * 8 + g) * kHd + t4 * 4;     // key 8nt+g: its row & 7 is g
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                const uint32_t w = *reinterpret_cast<const uint32_t*>(krow + ((ks ^ g) << 4)) ^ 0x80808080u;
                const uint32_t b0 = fa_bytes_to_h2(w, 0x5140u), b1 = fa_bytes_to_h2(w, 0x7362u);
                fa_mma_f16(s[nt], qa[ks][0], 0u, qa[ks][1], 0u, b0, b1);
                fa_mma_f16(s[nt], ql[ks][0], 0u, ql[ks][1], 0u, b0, b1);
            }
        }
        // ---- online softmax for row g; this lane holds keys 8nt + 2t4 + {0,1} --------------------------------------
        float p[4][2], mx = -INFINITY;
        float vsc[4][2];
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
            const float2 ksc = *reinterpret_cast<const float2*>(sc_k + nt * 8 + t4 * 2);
            const float2 vs2 = *reinterpret_cast<const float2*>(sc_v + nt * 8 + t4 * 2);
            const int key = t0 + nt * 8 + t4 * 2;
            const bool in0 = key < c_end, in1 = key + 1 < c_end;
            p[nt][0] = in0 ? s[nt][0] * (ksc.x * sm_l2e) : -INFINITY;
            p[nt][1] = in1 ? s[nt][1] * (ksc.y * sm_l2e) : -INFINITY;
            vsc[nt][0] = in0 ? vs2.x * kFaPScale : 0.0f;
            vsc[nt][1] = in1 ? vs2.y * kFaPScale : 0.0f;
            mx = fmaxf(mx, fmaxf(p[nt][0], p[nt][1]));
        }
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m_run, mx);
        const float m_use = m_new == -INFINITY ? 0.0f : m_new;
        const float alpha = fa_ex2(m_run - m_use);                   // 0 when nothing was seen before
        m_run = m_new;
        float psum = 0.0f;
        uint32_t pa[2][2];
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
            const float e0 = fa_ex2(p[nt][0] - m_use), e1 = fa_ex2(p[nt][1] - m_use);
            psum += e0 + e1;
            pa[nt >> 1][nt & 1] = fa_pack_h2(e0 * vsc[nt][0], e1 * vsc[nt][1]);   // p_t * s_v[t] (:844), scaled
        }
        l_run = l_run * alpha + psum;
#pragma unroll
        for (int c = 0; c < 8; ++c)
#pragma unroll
            for (int e = 0; e < 2; ++e) { acc[c][e][0] *= alpha; acc[c][e][1] *= alpha; }

        // ---- O += P V: k = keys (two steps of 16), n = dims; B by ldmatrix.trans over the INT8 tile -----------------
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            // lane i addresses one 16-byte row of matrix i / 8: keys 16j + 8*(m & 1) + (i & 7), chunk c + (m >> 1)
            const int mi = lane >> 3, key = 16 * j + 8 * (mi & 1) + (lane & 7);
            const uint32_t row_addr = smem_addr(vt) + (uint32_t)key * kHd;
#pragma unroll
            for (int c = 0; c < 8; c += 2) {
                const uint32_t addr = row_addr + ((uint32_t)((c + (mi >> 1)) ^ (key & 7)) << 4);
                uint32_t r0, r1, r2, r3;
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                             : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr) : "memory");
                r0 ^= 0x80808080u; r1 ^= 0x80808080u; r2 ^= 0x80808080u; r3 ^= 0x80808080u;
                // r0: keys 16j+{2t4,2t4+1}, r1: keys 16j+8+{2t4,2t4+1}; bytes (dim 2g, dim 2g+1) of each key
                fa_mma_f16(acc[c][0], pa[j][0], 0u, pa[j][1], 0u, fa_bytes_to_h2(r0, 0x6240u), fa_bytes_to_h2(r1, 0x6240u));
                fa_mma_f16(acc[c][1], pa[j][0], 0u, pa[j][1], 0u, fa_bytes_to_h2(r0, 0x7351u), fa_bytes_to_h2(r1, 0x7351u));
                fa_mma_f16(acc[c + 1][0], pa[j][0], 0u, pa[j][1], 0u, fa_bytes_to_h2(r2, 0x6240u), fa_bytes_to_h2(r3, 0x6240u));
                fa_mma_f16(acc[c + 1][1], pa[j][0], 0u, pa[j][1], 0u, fa_bytes_to_h2(r2, 0x7351u), fa_bytes_to_h2(r3, 0x7351u));
            }
        }
        __syncwarp();                                                // every lane is done with the stage
        if (lane == 0 && k + kFaStages < my_blocks) issue(k + kFaStages);
    }
    if (timed_out) atomicExch(&g_fa_timeouts, 1);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);

    // ---- merge the four warps (log-sum-exp), then hand the CTA's partial on ---------------------------------------
    __syncthreads();                                                 // all rings are idle: reuse them
    float* w_o = reinterpret_cast<float*>(s_tiles);                  // [warp][G][128]
    float* w_ml = w_o + kFaWarps * G * kHd;                          // [warp][G][2]
    if (g < G) {
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            // this lane's columns of chunk c: dims 16c + 4t4 + {0 (even tile, col 2t4), 2 (even, col 2t4+1), 1, 3 (odd tile)}
            float4 v = make_float4(acc[c][0][0], acc[c][1][0], acc[c][0][1], acc[c][1][1]);
            *reinterpret_cast<float4*>(w_o + ((size_t)warp * G + g) * kHd + c * 16 + t4 * 4) = v;
        }
        if (t4 == 0) { w_ml[(warp * G + g) * 2] = m_run; w_ml[(warp * G + g) * 2 + 1] = l_run; }
    }
    __syncthreads();
    for (int idx = tid; idx < G * kHd; idx += kFaThreads) {
        const int h = idx / kHd;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < kFaWarps; ++w) m = fmaxf(m, w_ml[(w * G + h) * 2]);
        const float m_use = m == -INFINITY ? 0.0f : m;
        float o = 0.0f, l = 0.0f;
#pragma unroll
        for (int w = 0; w < kFaWarps; ++w) {
            const float f = fa_ex2(w_ml[(w * G + h) * 2] - m_use);
            o += w_o[((size_t)w * G + h) * kHd + (idx % kHd)] * f;
            l += w_ml[(w * G + h) * 2 + 1] * f;
        }
        if (L.n_splits == 1) {
            a.out[(size_t)seq * a.n_q * kHd + (size_t)(kvh * G + h) * kHd + (idx % kHd)] = o / (l * kFaPScale);   // p_t / sum (:830)
        } else {
            po[idx] = o;
            if ((idx % kHd) == 0) { pml[h * 2] = m; pml[h * 2 + 1] = l; }
        }
    }
}

// Merge the splits of every (sequence, query head): one thread per output element.
__global__ void __launch_bounds__(128) attn_fast_merge_kernel(const FaLaunch L) {
    const tenzo_attention_args& a = L.a;
    const int G = L.group;
    const int kvh = blockIdx.x, seq = blockIdx.y;
    if (a.use_pdl) {
        pdl_launch_dependents();
        pdl_wait();
    }
    const size_t item0 = ((size_t)seq * a.n_kv + kvh) * L.n_splits;
    // One thread per four adjacent dims of a head; the splits' (max, sum) pairs and partial rows are fetched eight splits
    // at a time with every load in flight (a loop of dependent loads made this kernel ten L2 latencies long).
    constexpr int kBatch = 8;
    for (int idx4 = threadIdx.x; idx4 < G * kHd / 4; idx4 += blockDim.x) {
        const int h = idx4 / (kHd / 4);
        const float2* ml = reinterpret_cast<const float2*>(L.part_ml) + item0 * G + h;          // split s at ml[s * G]
        const float4* po = reinterpret_cast<const float4*>(L.part_o) + item0 * G * (kHd / 4) + idx4;   // split s at po[s * G * kHd / 4]
        float m = -INFINITY;
        for (int s0 = 0; s0 < L.n_splits; s0 += kBatch) {
            float2 v[kBatch];
#pragma unroll
            for (int u = 0; u < kBatch; ++u) v[u] = s0 + u < L.n_splits ? __ldcg(ml + (size_t)(s0 + u) * G) : make_float2(-INFINITY, 0.0f);
#pragma unroll
            for (int u = 0; u < kBatch; ++u) m = fmaxf(m, v[u].x);
        }
        const float m_use = m == -INFINITY ? 0.0f : m;
        float4 o = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        float l = 0.0f;
        for (int s0 = 0; s0 < L.n_splits; s0 += kBatch) {
            float2 v[kBatch];
            float4 p[kBatch];
#pragma unroll
            for (int u = 0; u < kBatch; ++u) {
                const bool in = s0 + u < L.n_splits;
                v[u] = in ? __ldcg(ml + (size_t)(s0 + u) * G) : make_float2(-INFINITY, 0.0f);
                p[u] = in ? __ldcg(po + (size_t)(s0 + u) * G * (kHd / 4)) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            }
#pragma unroll
            for (int u = 0; u < kBatch; ++u) {               // in split order, as the scalar form summed them
                if (s0 + u < L.n_splits) {
                    const float f = fa_ex2(v[u].x - m_use);
                    o.x += p[u].x * f; o.y += p[u].y * f; o.z += p[u].z * f; o.w += p[u].w * f;
                    l += v[u].y * f;
                }
            }
        }
        const float den = l * kFaPScale;
        float4 r = make_float4(o.x / den, o.y / den, o.z / den, o.w / den);
        reinterpret_cast<float4*>(a.out + (size_t)seq * a.n_q * kHd + (size_t)(kvh * G) * kHd)[idx4] = r;
    }
}

static int fa_tensor_map(const tenzo_attention_args& a, const int8_t* base, CUtensorMap* out) {
    typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                 const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static EncodeFn encode = nullptr;
    if (!encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn)
            return -4;
        encode = reinterpret_cast<EncodeFn>(fn);
    }
    // rows reachable from the layers up to this one; tiles that run past them are zero-filled and their keys masked
    const cuuint64_t rows = (cuuint64_t)(a.layer + 1) * a.n_kv * a.max_seq;
    const cuuint64_t dims[3] = {(cuuint64_t)kHd, rows, (cuuint64_t)a.batch};
    const cuuint64_t strides[2] = {(cuuint64_t)kHd, (cuuint64_t)(a.batch > 1 ? a.seq_stride_kv : (size_t)rows * kHd)};
    const cuuint32_t box[3] = {(cuuint32_t)kHd, (cuuint32_t)kFaBlk, 1u};
    const cuuint32_t estr[3] = {1u, 1u, 1u};
    const CUresult r = encode(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<int8_t*>(base), dims, strides, box, estr,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : -4;
}

static size_t fa_smem_bytes() {
    return 1024 + (size_t)kFaWarps * kFaStages * 2 * kFaTile + (size_t)kFaWarps * kFaStages * 64 * 4 + 8 * kHd * 4 + kFaWarps * kFaStages * 8 + 64;
}

// Keys per CTA: enough CTAs for about three waves of two per SM, at least 1024 keys each (a CTA's fixed cost - barriers,
// query rotation, the first tiles' latency - is worth some 500 keys of streaming; measured at 32 x 4160: 93 us with 384
// keys per CTA, 73 us with 1024) unless that leaves SMs without a CTA, then down to 256; a multiple of the 128 keys
// the four warps take per round.
static void fa_pick_split(int batch, int n_kv, int max_len, int* n_splits, int* split_keys) {
    const long long items = (long long)batch * n_kv;
    long long want = (3LL * 2 * 148 + items - 1) / items;
    long long most = (max_len + 1023) / 1024;
    if (items * most < 2 * 148) most = (max_len + 255) / 256;
    if (want > most) want = most;
    if (want < 1) want = 1;
    int keys = (int)((max_len + want - 1) / want);
    keys = (keys + 127) / 128 * 128;
    *split_keys = keys;
    *n_splits = (max_len + keys - 1) / keys;
}

// Launch with (or without) the programmatic-serialisation attribute: the kernel may become resident while its
// predecessor drains, and waits for it (griddepcontrol.wait) before its first global access.
template <typename... KArgs, typename... Args>
static cudaError_t fa_launch_ex(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, bool pdl, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

template <int G>
static int fa_launch(const FaLaunch& L, const CUtensorMap& km, const CUtensorMap& vm, cudaStream_t st) {
    const size_t smem = fa_smem_bytes();
    cudaError_t e = cudaFuncSetAttribute(attn_fast_kernel<G>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    e = fa_launch_ex(attn_fast_kernel<G>, dim3((unsigned)L.n_splits, (unsigned)L.a.n_kv, (unsigned)L.a.batch), dim3(kFaThreads), smem, st, L.a.use_pdl != 0, L, km, vm);
    return e == cudaSuccess ? 0 : (int)e;
}

bool attn_fast_applicable(const tenzo_attention_args& a) {
    if (a.block_table) return false;
    const int group = a.n_q / a.n_kv;
    if (group != 1 && group != 2 && group != 4 && group != 8) return false;
    if ((reinterpret_cast<uintptr_t>(a.cache_k) & 15) || (reinterpret_cast<uintptr_t>(a.cache_v) & 15)) return false;
    if ((reinterpret_cast<uintptr_t>(a.scale_k) & 15) || (reinterpret_cast<uintptr_t>(a.scale_v) & 15)) return false;
    if (reinterpret_cast<uintptr_t>(a.out) & 15) return false;                    // the merge writes 16 bytes at a time
    if (a.max_seq % 4 || a.seq_stride_sc % 4 || a.seq_stride_kv % 16) return false;
    return true;
}

int attn_fast_run(const tenzo_attention_args& a, cudaStream_t st) {
    FaLaunch L;
    L.a = a;
    if (L.a.q_stride <= 0) L.a.q_stride = a.n_q * kHd;
    if (L.a.kv_stride <= 0) L.a.kv_stride = a.n_kv * kHd;
    L.group = a.n_q / a.n_kv;
    fa_pick_split(a.batch, a.n_kv, a.max_len, &L.n_splits, &L.split_keys);
    if (a.split_keys > 0) {
        L.split_keys = (a.split_keys + 127) / 128 * 128;
        L.n_splits = (a.max_len + L.split_keys - 1) / L.split_keys;
    }
    const size_t items = (size_t)a.batch * a.n_kv * L.n_splits;
    const size_t need = items * L.group * (kHd + 2) * sizeof(float);
    if (L.n_splits > 1 && (!a.workspace || a.workspace_bytes < need || (reinterpret_cast<uintptr_t>(a.workspace) & 15))) return -1;
    L.part_o = static_cast<float*>(a.workspace);
    L.part_ml = L.part_o + items * L.group * kHd;
    if (a.append) {
        if (fa_launch_ex(fa_append_kernel, dim3((unsigned)a.batch, (unsigned)a.n_kv), dim3(64), 0, st, a.use_pdl != 0, L.a) != cudaSuccess) return (int)cudaErrorLaunchFailure;
    }
    CUtensorMap km, vm;
    std::memset(&km, 0, sizeof km);
    std::memset(&vm, 0, sizeof vm);
    if (int rc = fa_tensor_map(a, a.cache_k, &km)) return rc;
    if (int rc = fa_tensor_map(a, a.cache_v, &vm)) return rc;
    int rc;
    switch (L.group) {
        case 1: rc = fa_launch<1>(L, km, vm, st); break;
        case 2: rc = fa_launch<2>(L, km, vm, st); break;
        case 4: rc = fa_launch<4>(L, km, vm, st); break;
        default: rc = fa_launch<8>(L, km, vm, st); break;
    }
    if (rc) return rc;
    if (L.n_splits > 1) {
        if (fa_launch_ex(attn_fast_merge_kernel, dim3((unsigned)a.n_kv, (unsigned)a.batch), dim3(128), 0, st, a.use_pdl != 0, L) != cudaSuccess) return (int)cudaErrorLaunchFailure;
    }
    return 0;
}

int attn_fast_take_timeouts() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_fa_timeouts, sizeof v) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(g_fa_timeouts, &zero, sizeof zero);
    return v;
}

}  // namespace tz

extern "C" size_t tenzo_cuda_attention_workspace_bytes(int batch, int n_q, int n_kv, int max_len) {
    if (batch <= 0 || n_q <= 0 || n_kv <= 0 || n_q % n_kv || max_len <= 0) return 0;
    // the finest split the launcher may choose (or a caller may force): 128 keys per CTA
    const size_t splits = ((size_t)max_len + 127) / 128;
    return (size_t)batch * n_kv * splits * (size_t)(n_q / n_kv) * (tz::kHd + 2) * sizeof(float) + 64;
}
