// Fused RoPE + INT8 KV append + GQA decode attention for sm_100a, bit-identical to the reference.
//
// Replaces FusedKVCache::forward_attention_raw in int8_fused mode
// (src/runtime/TenzoEngine.cpp:447-533, :657-694, :823-851, :911-913 of the reference).
//
// Why the arithmetic order is fixed. The attention output feeds an RMSNorm and a +-31 quantiser,
// and with untrained (random) ternary weights a one-ulp difference grows by roughly 1.6x per
// layer, so "close" is not good enough: every fp32 operation here is done in the reference's order.
//   scores   eight FMA lanes over d (lane = d mod 8), lanes added left to right, times (s_k/sqrt(d))
//   softmax  max over t; e_t = expf(score_t - max) with glibc's bits; sum_t e_t left to right;
//            p_t = e_t * (1/sum)
//   output   acc_d = fma(float(V[t][d]), p_t * s_v[t], acc_d) for t = 0..T-1 in order
// The sums over t are therefore sequential chains; parallelism comes from everything else: keys
// are scored one per thread, exponentials are evaluated in parallel, each of the 128 output dims
// has its own chain, and CTAs cover (sequence, group of query heads).
//
// One CTA handles `GH` query heads that share a kv head, so K and V bytes are fetched once for
// all of them. With few sequences GH drops (down to 1) to put more CTAs on the machine; every CTA
// then re-derives the new token's quantised K/V row itself (same arithmetic, same bits) and only
// the CTA holding the group's first head stores it to the cache.
//
// Two instantiations: per-lane global loads of the key rows (few items, lowest latency: single-sequence
// decode) and K tiles brought in by TMA with the 128-byte swizzle, two keys per lane (64 or more
// (sequence, kv head) items). A third one follows the reference's other int8 cache, kv_mode "paged_int8"
// (PagedKVCache::forward_attention_raw, :242-445): 16-token blocks behind a block table, and its own arithmetic
// (two sets of eight FMA lanes, (dot * s_k) * scale, 1 / (sum + 1e-8), weights under 1e-7 dropped), again bit for bit.
// What bounds both long phases is the shared-memory return path, not HBM
// or arithmetic: the query vector is re-read (broadcast LDS.128) for every key or key pair while
// scoring, and every value warp re-reads the weights of its keys.
#include <cuda.h>

#include <cstring>

#include "attn_common.cuh"
#include "common.cuh"
#include "../../include/tenzo_kernels.h"

namespace tz {

constexpr int kAttnThreads = 512;
constexpr int kTileThreads = 384;    // block size of the variant whose scoring warps read K through TMA tiles
constexpr int kTileKeys = 64;        // keys per tile: two per lane
constexpr int kTileBytes = kTileKeys * 128;
constexpr int kMaxTileWarps = kTileThreads / 32;
constexpr int kScoreSmemBytes = 144 * 1024;  // per-CTA budget for the score vectors [T][GH] (whole CTA stays under 227 KB)

struct AttnLaunch {
    tenzo_attention_args a;
    int gh;                          // query heads per CTA
    int n_tile_warps;                // TMA-tile variant: warps that score (each owns a two-stage ring of 8 KB tiles)
};

template <int GH>
struct AttnSmem {
    // floats: s_q[GH*128] | s_new[256] | s_red[16*GH] | s_stat[2*GH+2]; then 16-byte aligned: s_new8[256 B] |
    // mbarriers[2 for V + 2 per tile warp] | V double buffer [2][kChunk*128 B] | scores [GH][padded T] floats.
    // TMA-tile variant: the V double buffer is the start of a 1024-byte-aligned region that first holds the scoring
    // warps' K-tile rings (n_tile_warps x 2 x 8 KB) and is handed to the V chunks once scoring is over.
    static constexpr int n_float = GH * kHd + 2 * kHd + 16 * GH + 2 * GH + 2;
    static constexpr int new8_off = (n_float * 4 + 15) & ~15;
    static constexpr int bar_off = new8_off + 2 * kHd;
    static constexpr int v_off = bar_off + 16 + 16 * kMaxTileWarps;
    static constexpr int sc_off = v_off + 2 * kChunk * kHd;
    static __host__ __device__ int padded(int max_len) { return (max_len + 3) & ~3; }
    static size_t bytes(int max_len) { return (size_t)sc_off + (size_t)padded(max_len) * GH * sizeof(float); }
    static __host__ __device__ int ring_bytes(int n_warps) { const int r = n_warps * 2 * kTileBytes; return r > 2 * kChunk * kHd ? r : 2 * kChunk * kHd; }
    static size_t bytes_tiled(int max_len, int n_warps) { return (size_t)v_off + 1024 + ring_bytes(n_warps) + (size_t)padded(max_len) * GH * sizeof(float); }
    // block pools: the sequence's block table is staged behind the scores
    static __host__ __device__ int table_bytes(int max_len) { return (((max_len + 15) >> 4) * 4 + 15) & ~15; }
    static int tile_warps_that_fit(int max_len, bool paged = false) {
        const long long room = 227LL * 1024 - ((long long)v_off + 1024 + (long long)padded(max_len) * GH * 4) - (paged ? table_bytes(max_len) : 0);
        const long long n = room / (2 * kTileBytes);
        return (int)(n > kMaxTileWarps ? kMaxTileWarps : n);
    }
};

// One 64-row x 128-byte box of the K cache (rows row0.. of sequence `seq`) into shared memory at `dst`
// (1024-byte aligned; rows land 128 bytes apart with their 16-byte chunks XORed by row & 7).
__device__ __forceinline__ void tma_load_k_tile(void* dst, const CUtensorMap* map, int row0, int seq, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                 ::"r"(smem_addr(dst)), "l"(map), "r"(0), "r"(row0), "r"(seq), "r"(smem_addr(bar)) : "memory");
}

// Block pools: the 16 rows x 128 bytes of one (block, layer, kv head) slice, rows row0.. of the pool seen as one long
// 2-D byte matrix; four of them make a 64-key tile with the same swizzled layout as above.
__device__ __forceinline__ void tma_load_k_rows(void* dst, const CUtensorMap* map, int row0, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(smem_addr(dst)), "l"(map), "r"(0), "r"(row0), "r"(smem_addr(bar)) : "memory");
}

__device__ int g_attn_timeouts = 0;   // 1: a bounded wait on a V-chunk copy gave up; 2: a position outside [0, max_len) was refused

#ifdef TZ_ATTN_TRACE
__device__ unsigned long long g_attn_phase[8];
#define TZ_PH(i) do { if (threadIdx.x == 0) { const long long now_ = clock64(); atomicAdd(&g_attn_phase[i], (unsigned long long)(now_ - ph_t_)); ph_t_ = now_; } } while (0)
#define TZ_PH_DECL long long ph_t_ = clock64()
#else
#define TZ_PH(i) do {} while (0)
#define TZ_PH_DECL do {} while (0)
#endif

// TILED = false: 512 threads, every thread scores keys it loads itself from global memory (lowest latency; few items).
// TILED = true:  384 threads; the first n_tile_warps warps score two keys per lane from K tiles that TMA brings into
//                per-warp rings with the 128-byte swizzle. Direct per-lane loads of 128-byte rows cost 32 data-pipe
//                wavefronts per instruction, and the query vector is then re-read once per key; a tile costs four
//                wavefronts per 16-byte column and each query load serves two keys. Same arithmetic, same bits.
// PAGED (with TILED = false): the caches are the reference's block pools [block][n_layers][kv_head][16][128] (scales
//                [..][16]) and key t of a sequence lives in block block_table[t / 16], slot t % 16; the arithmetic is that of
//                PagedKVCache::forward_attention_raw, which differs from the contiguous cache's in four places (marked below).
template <int GH, bool TILED, bool PAGED>
__global__ void __launch_bounds__(TILED ? kTileThreads : kAttnThreads) attn_kernel(const AttnLaunch L, const __grid_constant__ CUtensorMap kmap) {
    constexpr int NT = TILED ? kTileThreads : kAttnThreads;
    const tenzo_attention_args& a = L.a;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    using Lay = AttnSmem<GH>;
    float* s_q = reinterpret_cast<float*>(smem_raw);                     // [GH][128] rotated queries
    float* s_new = s_q + GH * kHd;                                       // [2][128] rotated k, v of the new token
    float* s_red = s_new + 2 * kHd;                                      // [16][GH] per-warp maxima
    float* s_stat = s_red + 16 * GH;                                     // [GH] max, [GH] 1/sum, [2] new-row scales
    int8_t* s_new8 = reinterpret_cast<int8_t*>(smem_raw + Lay::new8_off);   // [2][128] quantised new k, v
    uint64_t* s_bar = reinterpret_cast<uint64_t*>(smem_raw + Lay::bar_off); // [2] one per V buffer
    uint64_t* s_kbar = s_bar + 2;                                        // [n_tile_warps][2] one per K-tile stage
    const uint32_t ring_off = TILED ? ((smem_addr(smem_raw) + (uint32_t)Lay::v_off + 1023u) & ~1023u) - smem_addr(smem_raw) : (uint32_t)Lay::v_off;
    unsigned char* s_v = smem_raw + ring_off;                            // [2][kChunk][128] V rows as in memory (TILED: K rings first)
    float* s_sc = reinterpret_cast<float*>(smem_raw + (TILED ? ring_off + (uint32_t)Lay::ring_bytes(L.n_tile_warps) : (uint32_t)Lay::sc_off));   // [GH][tp]

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int tp = Lay::padded(a.max_len);
    const int G = a.n_q / a.n_kv;
    const int head0 = blockIdx.x * GH, kvh = head0 / G, seq = blockIdx.y;
    const bool stores_new_row = (head0 % G) == 0;

    // Few items, contiguous cache (single-sequence decode, where a layer's attention is 6 us of dependent latencies): the
    // position, the rotation coefficients, the rows of earlier keys and the first value chunks are inputs that no kernel
    // of the same step writes before this one, so they are requested BEFORE waiting for the producer of q / k / v and
    // their round trips overlap the producer's tail. (Callers that launch with use_pdl directly behind a kernel that
    // writes the position, the tables or cache rows below it must not: include/tenzo_kernels.h says so.)
    constexpr bool kEarly = !TILED && !PAGED;
    if (!kEarly && a.use_pdl) pdl_wait();
    TZ_PH_DECL;
    const int pos = __ldcg(a.pos + seq);
    // max_len sizes the score vectors and the staged block table: a position outside [0, max_len) would write past
    // them, so the CTA flags it (the host reads the flag like a give-up) and leaves without touching memory.
    if (pos < 0 || pos >= a.max_len) {
        if (tid == 0) atomicExch(&g_attn_timeouts, 2);
        return;
    }
    const int T = pos + 1;
    const int n_chunks = (T + kChunk - 1) / kChunk;

    const size_t row_base = PAGED ? 0 : ((size_t)a.layer * a.n_kv + kvh) * a.max_seq;   // :509-510
    int8_t* ck = a.cache_k + (PAGED ? (size_t)0 : (size_t)seq * a.seq_stride_kv + row_base * kHd);
    int8_t* cv = a.cache_v + (PAGED ? (size_t)0 : (size_t)seq * a.seq_stride_kv + row_base * kHd);
    float* sk = a.scale_k + (PAGED ? (size_t)0 : (size_t)seq * a.seq_stride_sc + row_base);
    float* sv = a.scale_v + (PAGED ? (size_t)0 : (size_t)seq * a.seq_stride_sc + row_base);
    // row of key t relative to ck / cv / sk / sv: t itself in the contiguous cache, (block, layer, kv head, slot) in the pools (:322-323)
    // The sequence's table entries are staged in shared memory (behind the scores): a lookup per key from global memory
    // would put an L2 round trip in front of every address. rowi_g reads the table in global memory and serves only the
    // value copies that leave before the staging is complete.
    const int* tbl = PAGED ? a.block_table + (size_t)seq * a.table_stride : nullptr;
    int* s_tbl = reinterpret_cast<int*>(s_sc + (size_t)GH * tp);
    if constexpr (PAGED)
        for (int i = tid; i <= (pos >> 4); i += NT) s_tbl[i] = __ldg(tbl + i);
    auto rowi_g = [&](int t) -> size_t {
        if constexpr (PAGED) return (((size_t)__ldg(tbl + (t >> 4)) * a.n_layers + a.layer) * a.n_kv + kvh) * 16 + (size_t)(t & 15);
        else return (size_t)t;
    };
    auto rowi = [&](int t) -> size_t {              // valid after the first block-wide barrier
        if constexpr (PAGED) return (((size_t)s_tbl[t >> 4] * a.n_layers + a.layer) * a.n_kv + kvh) * 16 + (size_t)(t & 15);
        else return (size_t)t;
    };
    const float* cs = a.rope_cos ? a.rope_cos + (size_t)pos * (kHd / 2) : nullptr;
    const float* sn = a.rope_sin ? a.rope_sin + (size_t)pos * (kHd / 2) : nullptr;

    // ---- few items (latency matters): this thread's first key row, its scale and its first value scale are requested
    //      now, so the loads fly while the queries are rotated and the new row is quantised -------------------------
    uint4 pre_row[8];
    float pre_ks = 0.0f, pre_vs = 0.0f;
    bool pre_ok = false, pre_vs_ok = false;
    if constexpr (!TILED && !PAGED) {
        if (tid < T && !(a.append && tid == pos)) {
#pragma unroll
            const size_t r = rowi(tid);
            for (int c = 0; c < 8; ++c) pre_row[c] = ld_cg_u4(reinterpret_cast<const uint4*>(ck + r * kHd) + c);
            pre_ks = __ldcg(sk + r);
            pre_vs = __ldcg(sv + r);                     // first element of the weights pass: head 0, key tid
            pre_ok = pre_vs_ok = true;
        }
    }

    // ---- V chunks travel by bulk copy into a double buffer; the first two leave now and overlap the
    //      whole scoring phase. (Rows are contiguous in the cache, so a chunk is one copy.) -------------
    auto issue_v = [&](int c, bool table_staged) {
        const int t0 = c * kChunk, nk = min(kChunk, T - t0);
        mbar_expect_tx(&s_bar[c & 1], (unsigned)nk * kHd);
        if constexpr (PAGED) {                 // a chunk is eight blocks of 16 rows, each contiguous in the pool
            for (int t = t0; t < t0 + nk; t += 16) {
                const int n = min(16, t0 + nk - t);
                const size_t r = table_staged ? rowi(t) : rowi_g(t);
                bulk_g2s(s_v + (size_t)(c & 1) * kChunk * kHd + (size_t)(t - t0) * kHd, cv + r * kHd, (unsigned)n * kHd, &s_bar[c & 1]);
            }
        } else {
            bulk_g2s(s_v + (size_t)(c & 1) * kChunk * kHd, cv + (size_t)t0 * kHd, (unsigned)nk * kHd, &s_bar[c & 1]);
        }
    };
    if (tid == 0) {
        mbar_init(&s_bar[0], 1);
        mbar_init(&s_bar[1], 1);
        if (TILED)
            for (int i = 0; i < 2 * L.n_tile_warps; ++i) mbar_init(&s_kbar[i], 1);
        mbar_init_fence();
        if (!TILED) {                          // TILED: the buffers hold K tiles first; the V chunks leave after scoring
            issue_v(0, false);
            if (n_chunks > 1) issue_v(1, false);
        }
    }

    // rotation coefficients of this thread's pair index (the query loop below and the key row use i = tid mod 64)
    float pre_c = 1.0f, pre_s = 0.0f;
    if (kEarly && cs && tid < (GH > 1 ? GH : 1) * (kHd / 2)) {
        pre_c = __ldg(cs + (tid & (kHd / 2 - 1)));
        pre_s = __ldg(sn + (tid & (kHd / 2 - 1)));
    }
    if (kEarly && a.use_pdl) pdl_wait();

    // ---- RoPE on this CTA's query heads (pairs i, i+64; :459-480) ---------------------------------
    for (int idx = tid; idx < GH * (kHd / 2); idx += NT) {
        const int g = idx / (kHd / 2), i = idx % (kHd / 2);
        const float* qh = a.q + (size_t)seq * a.q_stride + (size_t)(head0 + g) * kHd;
        float r0, r1;
        if constexpr (kEarly) rope_rotate(__ldcg(qh + i), __ldcg(qh + i + kHd / 2), cs != nullptr, pre_c, pre_s, r0, r1);   // NT > GH * 64: idx == tid
        else rope_pair(__ldcg(qh + i), __ldcg(qh + i + kHd / 2), cs, sn, i, r0, r1);
        s_q[g * kHd + i] = r0;
        s_q[g * kHd + i + kHd / 2] = r1;
    }

    // ---- the new token's K/V row: rotate, quantise (:483-533); one CTA per kv head stores it -------
    if (a.append) {
        if (tid < kHd / 2) {
            const float* kh = a.k + (size_t)seq * a.kv_stride + (size_t)kvh * kHd;
            float r0, r1;
            if constexpr (kEarly) rope_rotate(__ldcg(kh + tid), __ldcg(kh + tid + kHd / 2), cs != nullptr, pre_c, pre_s, r0, r1);
            else rope_pair(__ldcg(kh + tid), __ldcg(kh + tid + kHd / 2), cs, sn, tid, r0, r1);
            s_new[tid] = r0;
            s_new[tid + kHd / 2] = r1;
        } else if (tid < kHd) {
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
            reinterpret_cast<uint32_t*>(s_new8 + warp * kHd)[lane] = packed;
            if (lane == 0) s_stat[2 * GH + warp] = s;
            if (stores_new_row) {
                const size_t r = rowi(pos);
                int8_t* dst = (warp == 0 ? ck : cv) + r * kHd;
                reinterpret_cast<uint32_t*>(dst)[lane] = packed;
                if (lane == 0) (warp == 0 ? sk : sv)[r] = s;
            }
        }
    }
    __syncthreads();
    if (a.use_pdl) pdl_launch_dependents();
    TZ_PH(0);

    // ---- scores (:678-694): one key per thread straight from the cache (a row is 128 contiguous
    //      bytes), the next key's row requested before the current one is used; all GH heads, the
    //      reference's eight FMA lanes ------------------------------------------------------------------
    const float sm_scale = 1.0f / sqrtf((float)kHd);   // :660
    float tmax[GH];
#pragma unroll
    for (int g = 0; g < GH; ++g) tmax[g] = -1e30f;     // :670
    bool timed_out = false;
    if constexpr (TILED) {
        // warp w takes tiles w, w + n_tile_warps, ...; lane l scores rows l and l + 32 of a tile (same row & 7)
        const int n_sc = L.n_tile_warps;
        if (warp < n_sc) {
            const int n_tiles = (T + kTileKeys - 1) / kTileKeys;
            const int my_tiles = warp < n_tiles ? (n_tiles - warp + n_sc - 1) / n_sc : 0;
            unsigned char* ring = s_v + (size_t)warp * 2 * kTileBytes;
            uint64_t* kbar = s_kbar + 2 * warp;
            auto issue_tile = [&](int k) {
                if constexpr (PAGED) {                       // up to four 16-key blocks, each wherever the table says
                    const int tt0 = (warp + k * n_sc) * kTileKeys;
                    const int nb = min(kTileKeys / 16, (T - tt0 + 15) >> 4);
                    mbar_expect_tx(&kbar[k & 1], (unsigned)nb * 16 * kHd);
                    for (int i = 0; i < nb; ++i)
                        tma_load_k_rows(ring + (size_t)(k & 1) * kTileBytes + (size_t)i * 16 * kHd, &kmap, (int)rowi(tt0 + 16 * i), &kbar[k & 1]);
                } else {
                    mbar_expect_tx(&kbar[k & 1], (unsigned)kTileBytes);
                    tma_load_k_tile(ring + (size_t)(k & 1) * kTileBytes, &kmap, (int)row_base + (warp + k * n_sc) * kTileKeys, seq, &kbar[k & 1]);
                }
            };
            if (lane == 0) {
                if (my_tiles > 0) issue_tile(0);
                if (my_tiles > 1) issue_tile(1);
            }
            for (int k = 0; k < my_tiles; ++k) {
                const int t0 = (warp + k * n_sc) * kTileKeys;
                const unsigned char* tile = ring + (size_t)(k & 1) * kTileBytes;
                if (lane == 0 && !mbar_wait_bounded(&kbar[k & 1], (unsigned)(k >> 1) & 1u)) timed_out = true;
                __syncwarp();
                const int tA = t0 + lane, tB = tA + 32;
                const bool newA = a.append && tA == pos, newB = a.append && tB == pos;
                const unsigned char* rowA = newA ? reinterpret_cast<const unsigned char*>(s_new8) : tile + lane * kHd;
                const unsigned char* rowB = newB ? reinterpret_cast<const unsigned char*>(s_new8) : tile + (lane + 32) * kHd;
                const uint32_t xa = newA ? 0u : (uint32_t)(lane & 7), xb = newB ? 0u : (uint32_t)(lane & 7);
                if constexpr (PAGED) {
                    // the paged cache's dot product and score (differences 1 and 2 below), two keys per lane, one head
                    // at a time: 2 x 16 accumulators live; the maxima are taken from the stored scores afterwards
                    float ksc2[2];
#pragma unroll
                    for (int s2 = 0; s2 < 2; ++s2) {
                        const int t = s2 ? tB : tA;
                        ksc2[s2] = t < T ? ((a.append && t == pos) ? s_stat[2 * GH] : __ldcg(sk + rowi(t))) : 0.0f;
                    }
#pragma unroll 1
                    for (int g = 0; g < GH; ++g) {
                        float acc[2][16];
#pragma unroll
                        for (int e = 0; e < 16; ++e) acc[0][e] = acc[1][e] = 0.0f;
#pragma unroll
                        for (int c = 0; c < 8; ++c) {
                            const uint4 ka = *reinterpret_cast<const uint4*>(rowA + (((uint32_t)c ^ xa) << 4));
                            const uint4 kb = *reinterpret_cast<const uint4*>(rowB + (((uint32_t)c ^ xb) << 4));
                            const uint32_t wa[4] = {ka.x ^ 0x80808080u, ka.y ^ 0x80808080u, ka.z ^ 0x80808080u, ka.w ^ 0x80808080u};
                            const uint32_t wb[4] = {kb.x ^ 0x80808080u, kb.y ^ 0x80808080u, kb.z ^ 0x80808080u, kb.w ^ 0x80808080u};
                            const float4* q4 = reinterpret_cast<const float4*>(s_q + g * kHd + c * 16);
                            const float4 qa = q4[0], qb = q4[1], qc = q4[2], qd = q4[3];
                            const float qv[16] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w,
                                                  qc.x, qc.y, qc.z, qc.w, qd.x, qd.y, qd.z, qd.w};
#pragma unroll
                            for (int e = 0; e < 16; ++e) {
                                acc[0][e] = __fmaf_rn(qv[e], s8_to_f(wa[e >> 2], e & 3), acc[0][e]);
                                acc[1][e] = __fmaf_rn(qv[e], s8_to_f(wb[e >> 2], e & 3), acc[1][e]);
                            }
                        }
#pragma unroll
                        for (int s2 = 0; s2 < 2; ++s2) {
                            const int t = s2 ? tB : tA;
                            if (t < T) {
                                float dot = 0.0f;
#pragma unroll
                                for (int j = 0; j < 8; ++j) dot = __fadd_rn(dot, __fadd_rn(acc[s2][j], acc[s2][j + 8]));
                                s_sc[(size_t)g * tp + t] = __fmul_rn(__fmul_rn(dot, ksc2[s2]), sm_scale);
                            }
                        }
                    }
                    __syncwarp();                             // every lane has read the tile: the stage can be refilled
                    if (lane == 0 && k + 2 < my_tiles) issue_tile(k + 2);
                    continue;
                }
                float acc[2][GH][8];
#pragma unroll
                for (int s2 = 0; s2 < 2; ++s2)
#pragma unroll
                    for (int g = 0; g < GH; ++g)
#pragma unroll
                        for (int j = 0; j < 8; ++j) acc[s2][g][j] = 0.0f;
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    const uint4 ka = *reinterpret_cast<const uint4*>(rowA + (((uint32_t)c ^ xa) << 4));
                    const uint4 kb = *reinterpret_cast<const uint4*>(rowB + (((uint32_t)c ^ xb) << 4));
                    const uint32_t wa[4] = {ka.x ^ 0x80808080u, ka.y ^ 0x80808080u, ka.z ^ 0x80808080u, ka.w ^ 0x80808080u};
                    const uint32_t wb[4] = {kb.x ^ 0x80808080u, kb.y ^ 0x80808080u, kb.z ^ 0x80808080u, kb.w ^ 0x80808080u};
                    float kfa[16], kfb[16];
#pragma unroll
                    for (int e = 0; e < 16; ++e) {
                        kfa[e] = s8_to_f(wa[e >> 2], e & 3);
                        kfb[e] = s8_to_f(wb[e >> 2], e & 3);
                    }
#pragma unroll
                    for (int g = 0; g < GH; ++g) {
                        const float4* q4 = reinterpret_cast<const float4*>(s_q + g * kHd + c * 16);
                        const float4 qa = q4[0], qb = q4[1], qc = q4[2], qd = q4[3];
                        const float qv[16] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w,
                                              qc.x, qc.y, qc.z, qc.w, qd.x, qd.y, qd.z, qd.w};
#pragma unroll
                        for (int e = 0; e < 16; ++e) {
                            acc[0][g][e & 7] = __fmaf_rn(qv[e], kfa[e], acc[0][g][e & 7]);
                            acc[1][g][e & 7] = __fmaf_rn(qv[e], kfb[e], acc[1][g][e & 7]);
                        }
                    }
                }
                __syncwarp();                                 // every lane has read the tile: the stage can be refilled
                if (lane == 0 && k + 2 < my_tiles) issue_tile(k + 2);
#pragma unroll
                for (int s2 = 0; s2 < 2; ++s2) {
                    const int t = s2 ? tB : tA;
                    if (t < T) {
                        const float ksc = (a.append && t == pos) ? s_stat[2 * GH] : __ldcg(sk + t);
                        const float ks = ksc * sm_scale;
#pragma unroll
                        for (int g = 0; g < GH; ++g) {
                            const float* ac = acc[s2][g];
                            const float dot = (ac[0] + ac[1] + ac[2] + ac[3] + ac[4] + ac[5] + ac[6] + ac[7]) * ks;   // :691
                            s_sc[(size_t)g * tp + t] = dot;
                            tmax[g] = fmaxf(tmax[g], dot);
                        }
                    }
                }
            }
        }
    } else if constexpr (PAGED) {
        // One key per thread through the block table. Where the arithmetic departs from the contiguous cache's:
        // difference 1 (:371-386): sixteen accumulators - element e of every 16 has its own chain - then lane j =
        //   acc[j] + acc[j + 8], and the eight lanes are added left to right starting from 0.0f;
        // difference 2 (:388): score = (dot * s_k) * (1/sqrt(d)).
        // One head at a time, so that sixteen accumulators are live, not 16 x GH.
        for (int t = tid; t < T; t += NT) {
            const bool is_new = a.append && t == pos;
            const size_t r = is_new ? 0 : rowi(t);
            const uint4* src = is_new ? reinterpret_cast<const uint4*>(s_new8) : reinterpret_cast<const uint4*>(ck + r * kHd);
            uint4 cur[8];
#pragma unroll
            for (int c = 0; c < 8; ++c) cur[c] = is_new ? src[c] : ld_cg_u4(src + c);
            const float ksc = is_new ? s_stat[2 * GH] : __ldcg(sk + r);
#pragma unroll 1
            for (int g = 0; g < GH; ++g) {             // not unrolled: the byte-to-float conversions are redone per head instead of kept live
                float acc[16];
#pragma unroll
                for (int e = 0; e < 16; ++e) acc[e] = 0.0f;
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    const uint32_t w[4] = {cur[c].x ^ 0x80808080u, cur[c].y ^ 0x80808080u, cur[c].z ^ 0x80808080u, cur[c].w ^ 0x80808080u};
                    const float4* q4 = reinterpret_cast<const float4*>(s_q + g * kHd + c * 16);
                    const float4 qa = q4[0], qb = q4[1], qc = q4[2], qd = q4[3];
                    const float qv[16] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w,
                                          qc.x, qc.y, qc.z, qc.w, qd.x, qd.y, qd.z, qd.w};
#pragma unroll
                    for (int e = 0; e < 16; ++e) acc[e] = __fmaf_rn(qv[e], s8_to_f(w[e >> 2], e & 3), acc[e]);
                }
                float dot = 0.0f;
#pragma unroll
                for (int j = 0; j < 8; ++j) dot = __fadd_rn(dot, __fadd_rn(acc[j], acc[j + 8]));
                const float score = __fmul_rn(__fmul_rn(dot, ksc), sm_scale);
                s_sc[(size_t)g * tp + t] = score;
                tmax[g] = fmaxf(tmax[g], score);
            }
        }
    } else {
        auto load_row = [&](int t, uint4 (&r)[8]) {
            const bool is_new = a.append && t == pos;
            const uint4* src = is_new ? reinterpret_cast<const uint4*>(s_new8) : reinterpret_cast<const uint4*>(ck + rowi(t) * kHd);
    #pragma unroll
            for (int c = 0; c < 8; ++c) r[c] = is_new ? src[c] : ld_cg_u4(src + c);
        };
        uint4 cur[8], nxt[8];
        if (tid < T) {
            if (pre_ok) {
    #pragma unroll
                for (int c = 0; c < 8; ++c) cur[c] = pre_row[c];
            } else {
                load_row(tid, cur);
            }
        }
        for (int t = tid; t < T; t += NT) {
            const bool more = t + NT < T;
            if (more) load_row(t + NT, nxt);
            const float ksc = (a.append && t == pos) ? s_stat[2 * GH] : ((pre_ok && t == tid) ? pre_ks : __ldcg(sk + rowi(t)));
            {
                float acc[GH][8];
    #pragma unroll
                for (int g = 0; g < GH; ++g)
    #pragma unroll
                    for (int j = 0; j < 8; ++j) acc[g][j] = 0.0f;
    #pragma unroll
                for (int c = 0; c < 8; ++c) {
                    const uint32_t w[4] = {cur[c].x ^ 0x80808080u, cur[c].y ^ 0x80808080u, cur[c].z ^ 0x80808080u, cur[c].w ^ 0x80808080u};
                    float kf[16];
    #pragma unroll
                    for (int e = 0; e < 16; ++e) kf[e] = s8_to_f(w[e >> 2], e & 3);
    #pragma unroll
                    for (int g = 0; g < GH; ++g) {
                        const float4* q4 = reinterpret_cast<const float4*>(s_q + g * kHd + c * 16);
                        const float4 qa = q4[0], qb = q4[1], qc = q4[2], qd = q4[3];
                        const float qv[16] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w,
                                              qc.x, qc.y, qc.z, qc.w, qd.x, qd.y, qd.z, qd.w};
    #pragma unroll
                        for (int e = 0; e < 16; ++e) acc[g][e & 7] = __fmaf_rn(qv[e], kf[e], acc[g][e & 7]);
                    }
                }
                const float ks = ksc * sm_scale;
    #pragma unroll
                for (int g = 0; g < GH; ++g) {
                    const float dot = (acc[g][0] + acc[g][1] + acc[g][2] + acc[g][3] + acc[g][4] + acc[g][5] + acc[g][6] + acc[g][7]) * ks;   // :691
                    s_sc[(size_t)g * tp + t] = dot;
                    tmax[g] = fmaxf(tmax[g], dot);
                }
            }
            if (more) {
    #pragma unroll
                for (int c = 0; c < 8; ++c) cur[c] = nxt[c];
            }
        }
    }
    if constexpr (TILED && PAGED) {               // maxima from the stored scores (the scoring loop keeps no per-head registers)
        __syncthreads();
#pragma unroll
        for (int g = 0; g < GH; ++g)
            for (int t = tid; t < T; t += NT) tmax[g] = fmaxf(tmax[g], s_sc[(size_t)g * tp + t]);
    }
#pragma unroll
    for (int g = 0; g < GH; ++g) {
        const float m = warp_max(tmax[g]);
        if (lane == 0) s_red[warp * GH + g] = m;
    }
    __syncthreads();
    if (tid < GH) {
        float m = s_red[tid];
        for (int w = 1; w < NT / 32; ++w) m = fmaxf(m, s_red[w * GH + tid]);
        s_stat[tid] = m;
    }
    __syncthreads();
    TZ_PH(1);

    // ---- e_t = expf(score - max), in parallel (:826) -----------------------------------------------
    if (TILED && tid == 0) {                   // scoring is over: the ring region now takes the V chunks
        issue_v(0, true);
        if (n_chunks > 1) issue_v(1, true);
    }
    exp_in_place<GH>(s_sc, T, tp, s_stat, tid, NT);
    __syncthreads();
    TZ_PH(2);
    // ---- sum_t e_t, left to right, one thread per head (:824-829) ----------------------------------
    if (tid < GH) {
        const float sum = sequential_sum(s_sc + (size_t)tid * tp, T);
        s_stat[GH + tid] = PAGED ? 1.0f / __fadd_rn(sum, 1e-8f) : 1.0f / sum;       // difference 3 (:400)
    }
    __syncthreads();
    TZ_PH(3);
    // ---- weights p_t * s_v[t] (:830, :844) ------------------------------------------------------------
    {
        float inv_sum[GH];
#pragma unroll
        for (int g = 0; g < GH; ++g) inv_sum[g] = s_stat[GH + g];
#pragma unroll 4
        for (int t = tid; t < T; t += NT) {          // one value scale per key serves all the heads
            const float vs = (a.append && t == pos) ? s_stat[2 * GH + 1] : ((pre_vs_ok && t == tid) ? pre_vs : __ldcg(sv + rowi(t)));
#pragma unroll
            for (int g = 0; g < GH; ++g) {
                float* row = s_sc + (size_t)g * tp;
                const float p = row[t] * inv_sum[g];
                // difference 4 (:416): keys whose weight is under 1e-7 are skipped; a zero weight leaves every sum as it was
                row[t] = (PAGED && p < 1e-7f) ? 0.0f : p * vs;
            }
        }
    }
    __syncthreads();
    TZ_PH(4);

    // ---- output: thread d owns dim d of every head and walks t in order (:842-851) ------------------
    float o[GH];
#pragma unroll
    for (int g = 0; g < GH; ++g) o[g] = 0.0f;
    for (int c = 0; c < n_chunks; ++c) {
        const int t0 = c * kChunk, nkeys = min(kChunk, T - t0);
        unsigned char* vb = s_v + (size_t)(c & 1) * kChunk * kHd;
        if (lane == 0 && !mbar_wait_bounded(&s_bar[c & 1], (unsigned)(c >> 1) & 1u)) timed_out = true;
        __syncwarp();
        if (a.append && pos >= t0 && pos < t0 + nkeys) {        // the new token's row is not in the cache copy: patch it in
            __syncthreads();                                     // every warp has seen the copy complete
            if (tid < 8) reinterpret_cast<uint4*>(vb + (size_t)(pos - t0) * kHd)[tid] = reinterpret_cast<const uint4*>(s_new8 + kHd)[tid];
            __syncthreads();
        }
        if (tid < kHd) value_sum_chunk<GH>(vb + tid, s_sc + t0, tp, nkeys, o);
        __syncthreads();                                         // buffer free again
        if (tid == 0 && c + 2 < n_chunks) issue_v(c + 2, true);
    }
    if (timed_out) atomicExch(&g_attn_timeouts, 1);
    if (tid < kHd) {
#pragma unroll
        for (int g = 0; g < GH; ++g) a.out[(size_t)seq * a.n_q * kHd + (size_t)(head0 + g) * kHd + tid] = o[g];
    }
    TZ_PH(5);
}

// The K cache as a 3-D byte tensor {128, rows per sequence, sequences} for the scoring warps' tile loads.
// Block pools (paged): a 2-D byte matrix {128, every row of the pool}, read in boxes of one block slice (16 rows).
static int make_k_tensor_map(const tenzo_attention_args& a, CUtensorMap* out, bool paged) {
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
    if (paged) {
        const cuuint64_t rows = (cuuint64_t)a.n_pool_blocks * a.n_layers * a.n_kv * 16;
        const cuuint64_t dims[2] = {(cuuint64_t)kHd, rows};
        const cuuint64_t strides[1] = {(cuuint64_t)kHd};
        const cuuint32_t box[2] = {(cuuint32_t)kHd, 16u};
        const cuuint32_t estr[2] = {1u, 1u};
        const CUresult r = encode(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, a.cache_k, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        return r == CUDA_SUCCESS ? 0 : -4;
    }
    // rows reachable from the layers up to this one; tiles that run past them are zero-filled and their keys are never used
    const cuuint64_t rows = (cuuint64_t)(a.layer + 1) * a.n_kv * a.max_seq;
    const cuuint64_t dims[3] = {(cuuint64_t)kHd, rows, (cuuint64_t)a.batch};
    const cuuint64_t strides[2] = {(cuuint64_t)kHd, (cuuint64_t)a.seq_stride_kv};
    const cuuint32_t box[3] = {(cuuint32_t)kHd, (cuuint32_t)kTileKeys, 1u};
    const cuuint32_t estr[3] = {1u, 1u, 1u};
    const CUresult r = encode(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, a.cache_k, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : -4;
}

template <int GH, bool TILED, bool PAGED = false>
static int launch_attn(const AttnLaunch& L, cudaStream_t st) {
    CUtensorMap kmap;
    std::memset(&kmap, 0, sizeof kmap);
    if (TILED)
        if (int rc = make_k_tensor_map(L.a, &kmap, PAGED)) return rc;
    const size_t smem = (TILED ? AttnSmem<GH>::bytes_tiled(L.a.max_len, L.n_tile_warps) : AttnSmem<GH>::bytes(L.a.max_len)) +
                        (PAGED ? AttnSmem<GH>::table_bytes(L.a.max_len) : 0);
    cudaError_t e = cudaFuncSetAttribute(attn_kernel<GH, TILED, PAGED>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(L.a.n_q / GH), (unsigned)L.a.batch, 1);
    cfg.blockDim = dim3(TILED ? kTileThreads : kAttnThreads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = L.a.use_pdl ? 1 : 0;
    e = cudaLaunchKernelEx(&cfg, attn_kernel<GH, TILED, PAGED>, L, kmap);
    return e == cudaSuccess ? 0 : (int)e;
}

template <int GH>
static int tile_warps_for(int max_len, bool paged = false) { return AttnSmem<GH>::tile_warps_that_fit(max_len, paged); }

// Query heads per CTA: as many as share a kv head, halved while that leaves SMs idle or the score
// vectors [max_len][GH] would not fit in shared memory.
static int pick_heads_per_cta(int batch, int n_q, int group, int max_len) {
    // As many heads as share the kv head (K and V bytes are then fetched once for all of them), fewer
    // when that would leave SMs idle or the score vectors would not fit in shared memory.
    int gh = group;
    while (gh > 1 && ((long long)batch * (n_q / gh) < 148 || (size_t)gh * max_len * sizeof(float) > (size_t)kScoreSmemBytes)) gh >>= 1;
    return gh;
}

}  // namespace tz

#ifdef TZ_ATTN_TRACE
extern "C" __attribute__((visibility("default"))) int tenzo_cuda_attention_trace(unsigned long long* out8, int reset) {
    unsigned long long z[8] = {0};
    if (cudaMemcpyFromSymbol(out8, tz::g_attn_phase, sizeof z) != cudaSuccess) return -1;
    if (reset) cudaMemcpyToSymbol(tz::g_attn_phase, z, sizeof z);
    return 0;
}
#endif

namespace tz {
// tolerance mode (attention_fast.cu)
bool attn_fast_applicable(const tenzo_attention_args& a);
int attn_fast_run(const tenzo_attention_args& a, cudaStream_t st);
int attn_fast_take_timeouts();
}

extern "C" int tenzo_cuda_attention_take_timeouts(void) {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, tz::g_attn_timeouts, sizeof v) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(tz::g_attn_timeouts, &zero, sizeof zero);
    const int f = tz::attn_fast_take_timeouts();
    if (f < 0) return -1;
    return v > f ? v : f;
}

extern "C" int tenzo_cuda_attention_heads_per_cta(int batch, int n_q, int n_kv, int max_len) {
    if (batch <= 0 || n_q <= 0 || n_kv <= 0 || n_q % n_kv || max_len <= 0) return 0;
    return tz::pick_heads_per_cta(batch, n_q, n_q / n_kv, max_len);
}

extern "C" int tenzo_cuda_attention_int8(const tenzo_attention_args* args, void* stream) {
    using namespace tz;
    if (!args) return -1;
    const tenzo_attention_args& a = *args;
    if (!a.q || !a.out || !a.cache_k || !a.cache_v || !a.scale_k || !a.scale_v || !a.pos) return -1;
    if (a.append && (!a.k || !a.v)) return -1;
    if (a.head_dim != kHd) return -5;
    if (a.block_table && (a.n_layers <= 0 || a.layer < 0 || a.layer >= a.n_layers || a.table_stride < 0 || a.n_pool_blocks < 0)) return -1;
    if (a.n_q <= 0 || a.n_kv <= 0 || a.n_q % a.n_kv || a.batch <= 0 || a.max_len <= 0 || a.max_len > a.max_seq) return -1;
    if ((a.rope_cos == nullptr) != (a.rope_sin == nullptr)) return -1;
    const int group = a.n_q / a.n_kv;
    if (group != 1 && group != 2 && group != 4 && group != 8) return -5;
    if (a.mode == 1) return attn_fast_applicable(a) ? attn_fast_run(a, static_cast<cudaStream_t>(stream)) : -5;
    if (a.mode != 0) return -1;
    if ((size_t)a.max_len * sizeof(float) > (size_t)kScoreSmemBytes) return -5;   // one head's scores must fit on chip
    AttnLaunch L;
    L.a = a;
    if (L.a.q_stride <= 0) L.a.q_stride = a.n_q * kHd;
    if (L.a.kv_stride <= 0) L.a.kv_stride = a.n_kv * kHd;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    L.gh = pick_heads_per_cta(a.batch, a.n_q, group, a.max_len);
    if (a.heads_per_cta == 1 || a.heads_per_cta == 2 || a.heads_per_cta == 4 || a.heads_per_cta == 8)
        if (a.heads_per_cta <= group && (size_t)a.heads_per_cta * a.max_len * sizeof(float) <= (size_t)kScoreSmemBytes) L.gh = a.heads_per_cta;
    if (a.block_table) {
        // block pools: K through TMA tiles of four blocks when there are many (sequence, kv head) items and the pool
        // size is known (the tensor map needs it); per-lane loads through the block table otherwise
        int ptw = 0;
        switch (L.gh) {
            case 1: ptw = tile_warps_for<1>(a.max_len, true); break;
            case 2: ptw = tile_warps_for<2>(a.max_len, true); break;
            case 4: ptw = tile_warps_for<4>(a.max_len, true); break;
            default: break;
        }
        const long long pool_rows = (long long)a.n_pool_blocks * a.n_layers * a.n_kv * 16;
        const bool ptiled = a.tiles != 2 && ptw >= 4 && (a.tiles == 1 || a.batch * a.n_kv >= 64) && a.n_pool_blocks > 0 &&
                            pool_rows < (1LL << 31) && (reinterpret_cast<uintptr_t>(a.cache_k) & 15) == 0;
        if (a.tiles == 1 && !ptiled) return -5;
        if (ptiled) {
            L.n_tile_warps = ptw;
            switch (L.gh) {
                case 1: return launch_attn<1, true, true>(L, st);
                case 2: return launch_attn<2, true, true>(L, st);
                default: return launch_attn<4, true, true>(L, st);
            }
        }
        L.n_tile_warps = 0;
        switch (L.gh) {
            case 1: return launch_attn<1, false, true>(L, st);
            case 2: return launch_attn<2, false, true>(L, st);
            case 4: return launch_attn<4, false, true>(L, st);
            default: return launch_attn<8, false, true>(L, st);
        }
    }
    // Many (sequence, kv head) items: K through TMA tiles, two keys per lane. Few items (single-sequence decode): direct loads.
    int tw = 0;
    switch (L.gh) {
        case 1: tw = tile_warps_for<1>(a.max_len); break;
        case 2: tw = tile_warps_for<2>(a.max_len); break;
        case 4: tw = tile_warps_for<4>(a.max_len); break;
        default: tw = 0; break;          // eight heads per CTA need more registers than the tiled variant has
    }
    const bool tiled = a.tiles != 2 && tw >= 4 && (a.tiles == 1 || a.batch * a.n_kv >= 64) && a.seq_stride_kv % 16 == 0 &&
                       (reinterpret_cast<uintptr_t>(a.cache_k) & 15) == 0;
    if (a.tiles == 1 && !tiled) return -5;
    L.n_tile_warps = tiled ? tw : 0;
    if (tiled) {
        switch (L.gh) {
            case 1: return launch_attn<1, true>(L, st);
            case 2: return launch_attn<2, true>(L, st);
            default: return launch_attn<4, true>(L, st);
        }
    }
    switch (L.gh) {
        case 1: return launch_attn<1, false>(L, st);
        case 2: return launch_attn<2, false>(L, st);
        case 4: return launch_attn<4, false>(L, st);
        default: return launch_attn<8, false>(L, st);
    }
}
