// Batched TL1 bitlinear on the 5th-generation tensor cores (tcgen05.mma kind::i8, accumulators in
// tensor memory) for sm_100a. Used by tenzo_cuda_tl1_gemv when there are at least 16 sequences.
//
// Replaces, for many sequences at once, the same reference code as tl1_gemv.cu
// (src/runtime/TenzoEngine.cpp:22-166 and the call shapes :1547-1628 of the reference): integer
// accumulators are exact, so the result is bit-identical to the one-sequence path.
//
//   D[128 weight rows][N sequences] (int32, TMEM) += A[128][K] (u8 codes 0,1,2) * B[K][N] (s8 activations)
//   sum_k w*a = sum_k code*a - sum_k a          (w = code - 1; the per-sequence sum comes from the quantiser)
//
// One CTA per 128-row tile (two 64-row TL1 blocks; for the GLU epilogue the gate block and its up
// block, so the activation is applied inside the CTA). K is walked in 128-byte chunks; per chunk
//   warp 0 (one lane)   bulk-copies the packed 2-bit weights eight chunks at a time (2 x 16 KB; issuing a copy
//                       costs a few hundred cycles, so few large ones) into a two-group ring (64 KB in flight
//                       per CTA covers HBM latency) and TMA-loads the activation tile
//                       [N][128 B] into a 3- or 4-stage ring with the 128-byte swizzle the tensor core expects;
//   warps 2-5 / 6-9     (alternate chunks) expand the 2-bit codes to bytes and write the A tile [128][128 B] in the same
//                       swizzled K-major layout (a 4x4 byte transpose per 4 column pairs with PRMT, then
//                       mask/shift/interleave), fence it to the async proxy and arrive;
//   warp 1 (one lane)   issues four tcgen05.mma (K = 32 each) and commits them to the stage's "empty"
//                       barrier, which is what lets the producer refill the stage.
// After the last chunk a final commit signals the epilogue (warps 2-5: one TMEM lane = one weight
// row per thread, tcgen05.ld 16 sequences at a time, scale / residual / ReLU^2*GLU, coalesced stores).
// Few row tiles (the out, down and q|k|v projections have 20 to 30) would leave most SMs idle, so K is then split
// across the 2, 4 or 8 CTAs of a thread-block cluster: each accumulates its share of the chunks in its own tensor
// memory and parks its int32 partial tile in shared memory; after a hardware cluster barrier every CTA takes the
// 16-sequence column blocks b = rank, rank + ksplit, ..., adds its peers' partials for them through distributed
// shared memory (integer sums: order-free, exact), runs the epilogue on them and stores them (a reduce-scatter:
// the epilogue work is spread over the cluster instead of queueing on one leader).
// Every mbarrier wait is bounded; a wait that gives up sets g_umma_timeouts, the roles fall through
// to the end and the TMEM allocation is released on every path.
#include <cooperative_groups.h>

#include <cstdlib>

#include "umma.cuh"
#include "../../include/tenzo_kernels.h"

namespace cg = cooperative_groups;

namespace tz {

constexpr int kUmmaThreads = 320;              // warp 0 producer, warp 1 MMA, warps 2-5 and 6-9 expand alternate chunks
constexpr int kMaxStages = 4;                  // A/B tile stages (3 when the activation tile is 32 KB)
constexpr int kPGroup = 8;                     // chunks of packed weights per bulk copy (16 KB per row block)
constexpr int kPGroups = 2;                    // such groups in the ring: up to 64 KB of packed weights in flight
constexpr int kKc = 128;                       // bytes of K per stage (one swizzle atom row)
constexpr int kTileRows = 128;
constexpr int kABytes = kTileRows * kKc;       // 16 KB
constexpr int kPBytes = 2 * (kKc / 2) * 32;    // packed weights of one chunk, two row blocks: 4 KB
constexpr int kMaxN = 256;

struct UmmaLaunch {
    tenzo_tl1_gemv_args a;
    const float* inv;        // [batch] m/31
    const int* sum_a;        // [batch] sum_k a_k
    int units;               // tiles along the rows
    int n_box;               // sequences per CTA, padded to a multiple of 16 (<= 256)
    int tmem_cols;           // power of two >= max(32, n_box)
    int n_stages;            // A/B tile stages
    int ksplit;              // CTAs of a cluster that share one tile's K range (1 = no cluster)
};

__device__ int g_umma_timeouts = 0;


__device__ __forceinline__ float umma_seg_scale(const tenzo_tl1_gemv_args& a, int block) {
    return block < a.seg_end[0] ? a.seg_scale[0] : (block < a.seg_end[1] ? a.seg_scale[1] : a.seg_scale[2]);
}

struct UmmaSmem {
    // [1024-aligned] stages x { A 16 KB | B n_box*128 } | packed ring kPGroups x 2 blocks x 16 KB | barriers | tmem slot | GLU exchange [16][64] floats | inv[256] | sum_a[256]
    static __host__ __device__ int stage_bytes(int n_box) { return kABytes + n_box * kKc; }
    static __host__ __device__ int stages_for(int n_box) { return n_box > 128 ? 3 : kMaxStages; }
    static constexpr int n_bars = 3 * kMaxStages + 2 * kPGroups + 1;
    static __host__ __device__ size_t bytes(int n_box) {
        return 1024 + (size_t)stages_for(n_box) * stage_bytes(n_box) + (size_t)kPGroups * kPGroup * kPBytes + ((8 * n_bars + 15) & ~15) + 16 + 16 * 64 * 4 + 2 * kMaxN * 4;
    }
};

__global__ void __launch_bounds__(kUmmaThreads, 1) tl1_umma_kernel(const UmmaLaunch L, const __grid_constant__ CUtensorMap amap,
                                                                   const __grid_constant__ CUtensorMap omap,
                                                                   const __grid_constant__ CUtensorMap omap16) {
    const tenzo_tl1_gemv_args& a = L.a;
    extern __shared__ unsigned char smem_raw[];
    const uint32_t base_off = ((smem_addr(smem_raw) + 1023u) & ~1023u) - smem_addr(smem_raw);
    unsigned char* stages = smem_raw + base_off;
    const int stage_bytes = UmmaSmem::stage_bytes(L.n_box), S = L.n_stages;
    unsigned char* pring = stages + (size_t)S * stage_bytes;                  // [kPGroups][2 row blocks][kPGroup chunks][64][32] packed weights
    uint64_t* bars = reinterpret_cast<uint64_t*>(pring + (size_t)kPGroups * kPGroup * kPBytes);
    uint64_t* bar_raw = bars;                          // [S] activation tile has landed
    uint64_t* bar_ready = bars + kMaxStages;           // [S] A tile expanded (one arrival per expanding warp)
    uint64_t* bar_empty = bars + 2 * kMaxStages;       // [S] the stage's MMAs have completed
    uint64_t* bar_p = bars + 3 * kMaxStages;           // [kPGroups] packed weights have landed
    uint64_t* bar_pfree = bar_p + kPGroups;            // [kPGroups] packed weights consumed (one arrival per expanding warp per chunk)
    uint64_t* bar_accum = bar_pfree + kPGroups;        // all MMAs have completed
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(reinterpret_cast<unsigned char*>(bars) + ((8 * UmmaSmem::n_bars + 15) & ~15));   // 16-byte aligned
    float* s_glu = reinterpret_cast<float*>(tmem_slot + 4);   // [16][64]
    float* s_inv = s_glu + 16 * 64;                           // [kMaxN] m/31 of this CTA's sequences
    int* s_sum = reinterpret_cast<int*>(s_inv + kMaxN);       // [kMaxN] sum_k a_k

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const bool glu = a.epilogue == TENZO_EPI_RELU2_GLU;
    const int tile = blockIdx.x, seq0 = blockIdx.y * kMaxN;
    const int blk0 = glu ? tile : 2 * tile;
    const int blk1 = glu ? tile + L.units : (2 * tile + 1 < a.n_blocks ? 2 * tile + 1 : -1);
    const int ksplit = L.ksplit;
    const int split = ksplit > 1 ? (int)cg::this_cluster().block_rank() : 0;      // cluster = the CTAs with this tile's blockIdx.z = 0..ksplit-1
    const int all_chunks = a.K / kKc;
    const int c_begin = split * all_chunks / ksplit;                                // this CTA's chunks of K: never empty (all_chunks >= ksplit)
    const int n_chunks = (split + 1) * all_chunks / ksplit - c_begin;
    const int N = L.n_box;

    if (tid == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(&bar_raw[s], 1);
            mbar_init(&bar_ready[s], 4);
            mbar_init(&bar_empty[s], 1);
        }
        for (int s = 0; s < kPGroups; ++s) {
            mbar_init(&bar_p[s], 1);
            mbar_init(&bar_pfree[s], 4 * kPGroup);
        }
        mbar_init(bar_accum, 1);
        mbar_init_fence();
    }
    l2_prefetch_slice(a.prefetch, a.prefetch_bytes);       // the next kernel's weights
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(tmem_slot)), "r"(L.tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);
    if (a.use_pdl) {
        pdl_wait();
        pdl_launch_dependents();
    }
    bool timed_out = false, epi_ok = false;
    for (int i = tid; i < N; i += kUmmaThreads) {              // per-sequence epilogue operands (read after the final barrier)
        const int seq = seq0 + i;
        s_inv[i] = seq < a.batch ? __ldcg(L.inv + seq) : 0.0f;
        s_sum[i] = seq < a.batch ? __ldcg(L.sum_a + seq) : 0;
    }
    __syncthreads();

    if (warp == 0) {
        // ---- producer -----------------------------------------------------------------------------
        if (lane == 0) {
            const size_t blk_bytes = (size_t)(a.K / 2) * 32;
            int gp = 0;                                   // next group of packed chunks to request
            const int n_groups = (n_chunks + kPGroup - 1) / kPGroup;
            for (int j = 0; j < n_chunks && !timed_out; ++j) {
                for (; gp < n_groups && gp <= j / kPGroup + 1; ++gp) {
                    const int slot = gp % kPGroups, guse = gp / kPGroups;
                    if (guse > 0 && !mbar_test(&bar_pfree[slot], (unsigned)(guse - 1) & 1u)) {
                        if (gp > j / kPGroup) break;               // the group after the current one: do not hold up the activation tiles
                        if (!mbar_spin_bounded(&bar_pfree[slot], (unsigned)(guse - 1) & 1u)) { timed_out = true; break; }
                    }
                    const int chunks = min(kPGroup, n_chunks - gp * kPGroup);
                    const unsigned bytes = (unsigned)chunks * (kPBytes / 2);
                    unsigned char* sP = pring + (size_t)slot * kPGroup * kPBytes;
                    mbar_expect_tx(&bar_p[slot], blk1 >= 0 ? 2 * bytes : bytes);
                    const size_t k_off = (size_t)(c_begin + gp * kPGroup) * (kPBytes / 2);
                    bulk_g2s(sP, a.w + (size_t)blk0 * blk_bytes + k_off, bytes, &bar_p[slot]);
                    if (blk1 >= 0) bulk_g2s(sP + kPGroup * (kPBytes / 2), a.w + (size_t)blk1 * blk_bytes + k_off, bytes, &bar_p[slot]);
                }
                if (timed_out) break;
                const int s = j % S, use = j / S;
                if (use > 0 && !mbar_spin_bounded(&bar_empty[s], (unsigned)(use - 1) & 1u)) { timed_out = true; break; }
                mbar_expect_tx(&bar_raw[s], (unsigned)(N * kKc));
                tma_load_2d(stages + (size_t)s * stage_bytes + kABytes, &amap, (c_begin + j) * kKc, seq0, &bar_raw[s]);
            }
        }
    } else if (warp == 1) {
        // ---- MMA issue ------------------------------------------------------------------------------
        if (lane == 0) {
            // c = s32, a = u8, b = s8, both K-major, N at bit 17 (>>3), M at bit 24 (>>4)
            const uint32_t idesc = (2u << 4) | (0u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(kTileRows >> 4) << 24);
            for (int j = 0; j < n_chunks; ++j) {
                const int s = j % S, use = j / S;
                if (!mbar_spin_bounded(&bar_ready[s], (unsigned)use & 1u)) { timed_out = true; break; }
                if (!mbar_spin_bounded(&bar_raw[s], (unsigned)use & 1u)) { timed_out = true; break; }
                tc_fence_after();
                const uint32_t sa = smem_addr(stages + (size_t)s * stage_bytes);
                const uint64_t da = umma_desc_sw128(sa), db = umma_desc_sw128(sa + kABytes);
#pragma unroll
                for (int k4 = 0; k4 < kKc / 32; ++k4)
                    umma_i8(tmem_base, da + (uint64_t)(2 * k4), db + (uint64_t)(2 * k4), idesc, (j > 0 || k4 > 0) ? 1u : 0u);
                umma_commit(&bar_empty[s]);
            }
            umma_commit(bar_accum);
        }
    } else {
        // ---- expand the 2-bit codes into the A tile ---------------------------------------------------
        // lane bits 0-1: kk8 & 3, bit 2: c4 & 1, bits 3-4: c4 >> 1; warp: kk8 >> 2 and the row block. A quarter
        // warp then stores eight different 16-byte chunk positions (no bank conflicts on the A tile).
        const int uw = (warp - 2) & 3, grp = (warp - 2) >> 2;   // two groups of four warps take alternate chunks
        const int kk8 = (lane & 3) | ((uw & 1) << 2), c4 = ((lane >> 2) & 1) | (((lane >> 3) & 3) << 1), blk = uw >> 1;
        int seen_group = -1;
        for (int j = grp; j < n_chunks; j += 2) {
            const int s = j % S, use = j / S, ps = (j / kPGroup) % kPGroups, puse = (j / kPGroup) / kPGroups;
            bool ok = true;
            if (lane == 0 && (j / kPGroup != seen_group)) ok = mbar_spin_bounded(&bar_p[ps], (unsigned)puse & 1u);
            seen_group = j / kPGroup;
            if (lane == 0 && ok) ok = (use == 0 || mbar_spin_bounded(&bar_empty[s], (unsigned)(use - 1) & 1u));
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) { timed_out = true; break; }
            unsigned char* st = stages + (size_t)s * stage_bytes;
            const uint32_t* sP = reinterpret_cast<const uint32_t*>(pring + (size_t)ps * kPGroup * kPBytes + (size_t)blk * kPGroup * (kPBytes / 2) +
                                                                   (size_t)(j % kPGroup) * (kPBytes / 2));
            uint32_t W[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) W[i] = (blk == 1 && blk1 < 0) ? 0u : sP[(8 * kk8 + i) * 8 + c4];
            // 4x4 byte transposes: T[h][jj] = bytes (W[4h+0].jj, W[4h+1].jj, W[4h+2].jj, W[4h+3].jj): column pair 8*kk8+4h.. of byte column 4*c4+jj
            uint32_t T[2][4];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint32_t p0 = prmt(W[4 * h], W[4 * h + 1], 0x5140u), p1 = prmt(W[4 * h + 2], W[4 * h + 3], 0x5140u);
                const uint32_t p2 = prmt(W[4 * h], W[4 * h + 1], 0x7362u), p3 = prmt(W[4 * h + 2], W[4 * h + 3], 0x7362u);
                T[h][0] = prmt(p0, p1, 0x5410u); T[h][1] = prmt(p0, p1, 0x7632u);
                T[h][2] = prmt(p2, p3, 0x5410u); T[h][3] = prmt(p2, p3, 0x7632u);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&bar_pfree[ps]);   // the packed chunk has been consumed into registers
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) {
#pragma unroll
                for (int hi = 0; hi < 2; ++hi) {            // low nibble: row 4*c4+jj, high nibble: row 32+4*c4+jj
                    uint4 o;
                    uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const uint32_t n = T[h][jj] >> (4 * hi);
                        const uint32_t e0 = n & 0x03030303u, e1 = (n >> 2) & 0x03030303u;   // codes of the even / odd columns
                        ow[2 * h] = prmt(e0, e1, 0x5140u);
                        ow[2 * h + 1] = prmt(e0, e1, 0x7362u);
                    }
                    const int row = blk * 64 + hi * 32 + 4 * c4 + jj;
                    *reinterpret_cast<uint4*>(st + row * kKc + ((kk8 ^ (row & 7)) << 4)) = o;
                }
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bar_ready[s]);
        }
        if (grp == 0) {
            // ---- all of this CTA's MMAs have completed; in a cluster it parks its partial tile [N][128] int32 (the
            //      column blocks its peers will reduce) in the stage memory the pipeline no longer needs ------------------
            bool ok = true;
            if (lane == 0) ok = !timed_out && mbar_spin_bounded(bar_accum, 0u);
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) timed_out = true;
            tc_fence_after();
            epi_ok = ok;
            if (ksplit > 1) {
                const int q = warp & 3, row = 32 * q + lane;
                int* s_part = reinterpret_cast<int*>(stages);
                for (int c0 = 0; c0 < N; c0 += 16) {
                    if ((c0 >> 4) % ksplit == split) continue;       // this CTA's own column blocks stay in tensor memory
                    uint32_t r[16];
#pragma unroll
                    for (int i = 0; i < 16; ++i) r[i] = 0u;
                    if (ok) tmem_ld16(tmem_base + ((uint32_t)(32 * q) << 16) + (uint32_t)c0, r);
#pragma unroll
                    for (int i = 0; i < 16; ++i) s_part[(c0 + i) * 128 + row] = (int)r[i];
                }
            }
        }
    }
    if (ksplit > 1) cg::this_cluster().sync();               // every CTA's partial tile is in place
    if (warp >= 2 && warp < 6) {
        // ---- epilogue: TMEM lane = weight row; column blocks split, split + ksplit, ... (all of them without a cluster) ----
        const bool ok = epi_ok;
        const int q = warp & 3;                              // this warp may touch TMEM lanes 32q..32q+31
        const int row = 32 * q + lane, rblk = row >> 6, rr = row & 63;
        const int block = rblk ? blk1 : blk0;
        const float wscale = block >= 0 ? umma_seg_scale(a, block) : 0.0f;
        const int* peer[8];
#pragma unroll
        for (int p = 0; p < 8; ++p)
            peer[p] = (ksplit > 1 && p < ksplit && p != split) ? cg::this_cluster().map_shared_rank(reinterpret_cast<int*>(stages), p) : nullptr;
        // The output columns [sequences][128 rows] (GLU: [..][64]) are assembled in shared memory the pipeline no
        // longer needs - the stage memory, or with a cluster the packed-weight ring, because the stage memory then
        // holds the partial tile the peers are reading - one row per thread, and leave through TMA stores: rows of
        // 512 (256) contiguous bytes per sequence, clipped at the matrix edge by the tensor map.
        float* s_out = reinterpret_cast<float*>(ksplit > 1 ? pring : stages);
        int o0 = 0;                                          // column slot in s_out of the block being processed
        for (int c0 = 16 * split; c0 < N; c0 += 16 * ksplit, o0 += 16) {
            uint32_t r[16];
            if (ok) tmem_ld16(tmem_base + ((uint32_t)(32 * q) << 16) + (uint32_t)c0, r);
#pragma unroll
            for (int p = 0; p < 8; ++p) {
                if (peer[p]) {
#pragma unroll
                    for (int i = 0; i < 16; ++i) r[i] += (uint32_t)peer[p][(c0 + i) * 128 + row];
                }
            }
            int sums[16];
            float invs[16], res[16];
#pragma unroll
            for (int i = 0; i < 16; i += 4) {
                const int4 sv = *reinterpret_cast<const int4*>(s_sum + c0 + i);
                const float4 iv = *reinterpret_cast<const float4*>(s_inv + c0 + i);
                sums[i] = sv.x; sums[i + 1] = sv.y; sums[i + 2] = sv.z; sums[i + 3] = sv.w;
                invs[i] = iv.x; invs[i + 1] = iv.y; invs[i + 2] = iv.z; invs[i + 3] = iv.w;
            }
            if (a.epilogue == TENZO_EPI_RESIDUAL) {
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const int seq = seq0 + c0 + i;
                    res[i] = (seq < a.batch && block >= 0) ? __ldcg(a.resid + (size_t)seq * a.out_stride + block * 64 + rr) : 0.0f;
                }
            }
            float v[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const int accv = (int)r[i] - sums[i];
                r[i] = (uint32_t)accv;
                v[i] = (float)accv * (invs[i] * wscale);      // :1554, :118
            }
            if (a.acc_out && ok && block >= 0) {
#pragma unroll
                for (int i = 0; i < 16; ++i)
                    if (seq0 + c0 + i < a.batch) a.acc_out[(size_t)(seq0 + c0 + i) * a.n_blocks * 64 + block * 64 + rr] = (int)r[i];
            }
            if (glu) {
                if (rblk == 1) {
#pragma unroll
                    for (int i = 0; i < 16; ++i) s_glu[i * 64 + rr] = v[i];
                }
                named_barrier_sync(1, 128);
                if (rblk == 0) {
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const float rl = fmaxf(0.0f, v[i]);
                        s_out[(o0 + i) * 64 + rr] = (rl * rl) * s_glu[i * 64 + rr];   // :1618-1619
                    }
                }
                named_barrier_sync(1, 128);
            } else {
#pragma unroll
                for (int i = 0; i < 16; ++i)
                    s_out[(o0 + i) * 128 + row] = a.epilogue == TENZO_EPI_RESIDUAL ? res[i] + v[i] : v[i];   // :1590
            }
        }
        fence_proxy_async_smem();
        named_barrier_sync(1, 128);
        if (tid == 64 && ok) {
            if (ksplit == 1) {
                asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];"
                             ::"l"(&omap), "r"((glu ? tile : blk0) * 64), "r"(seq0), "r"(smem_addr(s_out)) : "memory");
            } else {                                         // one 16-sequence box per column block of this CTA
                const int row_floats = glu ? 64 : 128;
                int slot = 0;
                for (int c0 = 16 * split; c0 < N; c0 += 16 * ksplit, slot += 16) {
                    if (seq0 + c0 >= a.batch) break;         // nothing but padding from here on
                    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];"
                                 ::"l"(&omap16), "r"((glu ? tile : blk0) * 64), "r"(seq0 + c0), "r"(smem_addr(s_out + slot * row_floats)) : "memory");
                }
            }
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");     // the tile has left shared memory
        }
    }
    if (ksplit > 1) cg::this_cluster().sync();               // every peer has read this CTA's partial tile: it may exit
    if (timed_out) atomicExch(&g_umma_timeouts, 1);
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(L.tmem_cols) : "memory");
    }
}

bool tl1_umma_applicable(const tenzo_tl1_gemv_args& a) {
    return a.batch >= 16 && a.K % kKc == 0 && a.K >= kKc && a.out_stride % 4 == 0 && (reinterpret_cast<uintptr_t>(a.out) & 15) == 0;
}

// CTAs of a cluster that split one tile's K range: doubled while the grid still fits the SMs (one CTA per SM) and
// every CTA keeps at least four 128-byte chunks. TENZO_UMMA_KSPLIT = 1, 2, 4 or 8 overrides the choice (measurement aid).
static int pick_umma_ksplit(int ctas, int n_chunks) {
    static int n_sm = 0, forced = -1;
    if (forced < 0) {
        const char* e = std::getenv("TENZO_UMMA_KSPLIT");
        const int v = e ? std::atoi(e) : 0;
        forced = (v == 1 || v == 2 || v == 4 || v == 8) ? v : 0;
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n_sm <= 0) n_sm = 148;
    }
    if (forced) return forced <= n_chunks ? forced : 1;
    int k = 1;
    while (k < 8 && ctas * k * 2 <= n_sm && n_chunks / (k * 2) >= 4) k *= 2;
    return k;
}

// a8 [batch][K] int8 (16-byte aligned), inv [batch], sum_a [batch] already produced on `st`.
int launch_tl1_umma(const tenzo_tl1_gemv_args& a, const int8_t* a8, const float* inv, const int* sum_a, cudaStream_t st) {
    UmmaLaunch L;
    L.a = a;
    L.inv = inv;
    L.sum_a = sum_a;
    const bool glu = a.epilogue == TENZO_EPI_RELU2_GLU;
    L.units = glu ? a.n_blocks / 2 : (a.n_blocks + 1) / 2;
    const int per_cta = a.batch < kMaxN ? a.batch : kMaxN;
    L.n_box = (per_cta + 15) & ~15;
    L.tmem_cols = 32;
    while (L.tmem_cols < L.n_box) L.tmem_cols *= 2;
    L.n_stages = UmmaSmem::stages_for(L.n_box);
    const int seq_tiles = (a.batch + kMaxN - 1) / kMaxN;
    L.ksplit = pick_umma_ksplit(L.units * seq_tiles, a.K / kKc);
    CUtensorMap amap, omap, omap16;
    // activations [batch][K] int8: B-operand tiles {128 bytes of K, n_box sequences}, 128-byte swizzle
    if (int rc = encode_2d(&amap, CU_TENSOR_MAP_DATA_TYPE_UINT8, a8, (uint64_t)a.K, (uint64_t)a.batch, (uint64_t)a.K, kKc, (uint32_t)L.n_box,
                           CU_TENSOR_MAP_SWIZZLE_128B)) return rc;
    // output [batch][n_out] fp32: store tiles {128 (GLU: 64) rows of the weight matrix, n_box sequences}
    const uint64_t n_out = (uint64_t)(glu ? a.n_blocks / 2 : a.n_blocks) * 64;
    if (int rc = encode_2d(&omap, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, a.out, n_out, (uint64_t)a.batch, (uint64_t)a.out_stride * 4, glu ? 64u : 128u,
                           (uint32_t)L.n_box, CU_TENSOR_MAP_SWIZZLE_NONE)) return rc;
    // the same matrix in boxes of 16 sequences, for the column blocks a cluster's CTAs store separately
    if (int rc = encode_2d(&omap16, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, a.out, n_out, (uint64_t)a.batch, (uint64_t)a.out_stride * 4, glu ? 64u : 128u,
                           16u, CU_TENSOR_MAP_SWIZZLE_NONE)) return rc;
    const size_t smem = UmmaSmem::bytes(L.n_box);
    cudaError_t e = cudaFuncSetAttribute(tl1_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)L.units, (unsigned)seq_tiles, (unsigned)L.ksplit);
    cfg.blockDim = dim3(kUmmaThreads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    int n_attr = 0;
    if (L.ksplit > 1) {
        attr[n_attr].id = cudaLaunchAttributeClusterDimension;
        attr[n_attr].val.clusterDim.x = 1;
        attr[n_attr].val.clusterDim.y = 1;
        attr[n_attr].val.clusterDim.z = (unsigned)L.ksplit;
        ++n_attr;
    }
    if (a.use_pdl) {
        attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
        ++n_attr;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n_attr;
    e = cudaLaunchKernelEx(&cfg, tl1_umma_kernel, L, amap, omap, omap16);
    return e == cudaSuccess ? 0 : (int)e;
}


int tl1_umma_take_timeouts() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_umma_timeouts, sizeof v) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(g_umma_timeouts, &zero, sizeof zero);
    return v;
}

}  // namespace tz

extern "C" int tenzo_cuda_tl1_gemm_ksplit(int n_blocks, int K, int batch, int epilogue) {
    if (n_blocks <= 0 || K < tz::kKc || K % tz::kKc || batch < 16) return 0;       // the tensor-core path does not apply
    const int units = epilogue == TENZO_EPI_RELU2_GLU ? n_blocks / 2 : (n_blocks + 1) / 2;
    return tz::pick_umma_ksplit(units * ((batch + tz::kMaxN - 1) / tz::kMaxN), K / tz::kKc);
}
