// Batched TL1 bitlinear on the 5th-generation tensor cores (tcgen05.mma kind::i8, accumulators AND the weight
// operand in tensor memory) for sm_100a. Used by tenzo_cuda_tl1_gemv when there are at least 16 sequences.
//
// Replaces, for many sequences at once, the same reference code as tl1_gemv.cu
// (src/runtime/TenzoEngine.cpp:22-166 and the call shapes :1547-1628 of the reference): integer
// accumulators are exact, so the result is bit-identical to the one-sequence path.
//
//   D[128 weight rows][N sequences] (int32, TMEM) += A[128][K] (u8 codes 0,1,2, TMEM) * B[K][N] (s8 activations, smem)
//   sum_k w*a = sum_k code*a - sum_k a          (w = code - 1; the per-sequence sum comes from the quantiser)
//
// One CTA per 128-row tile (two 64-row TL1 blocks; for the GLU epilogue the gate block and its up block, so the
// activation is applied inside the CTA). K is walked in 128-byte chunks through a ring of 4, 8 or 12 slots (a multiple of
// four: see UmmaSmem::slots_for); 21 warps per CTA:
//   warp 0 (lane 0)     bulk-copies the packed 2-bit weights eight chunks at a time (2 x 16 KB) into a ring of two or
//                       three groups; the first groups are requested by one lane each first thing in the kernel
//                       (weights depend on no earlier kernel); lanes 1-31 fetch the per-sequence scale and sum for
//                       the epilogue;
//   warps 2-17          (four groups of four; group g takes chunks g, g + 4, ..., two per iteration when there are
//                       eight or more slots) expand the 2-bit codes to bytes in registers and write them straight into
//                       the slot's 32 columns of tensor memory (tcgen05.st 16x256b: no shared-memory A tile, no
//                       proxy fence). Lane quarter q of a group takes one nibble half of one row block; a thread's
//                       four TMEM lanes are the four rows of ONE packed word, so a thread loads sixteen words per
//                       chunk and every byte of them is used. The row order inside a quarter is therefore permuted
//                       (TMEM lane l holds row 4*(l&7) + (l>>3)); the epilogue undoes it. The warps of a group
//                       take turns TMA-loading the chunk's activation tile [N][128 B] (128-byte swizzle) into the
//                       slot right after they have seen it free: a dedicated thread doing a poll, an expect_tx and
//                       a TMA issue per chunk was the slowest role of the pipeline (about 800 cycles per chunk);
//   warps 1, 18-20      (lane 0 each) take every fourth chunk: one poll of the slot's barrier (expand arrivals + the
//                       TMA's bytes), four tcgen05.mma (K = 32 each, A from tensor memory), one commit that frees the
//                       slot. A poll costs the issuing thread about 180 cycles, a commit about 80 and the loop
//                       another 270 (measured), more than the MMAs of a chunk take below 256 sequences, so one
//                       issuing thread bounds the loop; four hide it. Integer accumulation is order-free, so the only
//                       ordering needed between them is that chunk 0 (which overwrites) completes first.
// After the last chunk every issuing thread commits to one barrier, which starts the epilogue on all sixteen expand
// warps (the groups on alternate 32-sequence column units; TMEM lane = weight row, tcgen05.ld 16 sequences at a
// time, scale / residual / ReLU^2*GLU, the unit assembled in shared memory and sent off by its own TMA store while
// the next one is computed).
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

constexpr int kExpandGroups = 4;               // groups of four warps that expand alternate chunks (and run the epilogue)
constexpr int kUmmaThreads = 32 * (2 + 4 * kExpandGroups + 3);   // warp 0 producer, warp 1 and the last three MMA issue, the rest expand
constexpr int kMmaThreads = 4;
constexpr int kMaxSlots = 16;                  // ring of chunk slots: as many as tensor memory and shared memory allow (4 at 256 sequences, 12 at 64)
constexpr int kPGroup = 8;                     // chunks of packed weights per bulk copy (16 KB per row block)
constexpr int kMaxPGroups = 3;                 // such groups in the ring (3 up to 64 sequences, else 2): 64 KB of packed weights in flight behind the group in use
constexpr int kKc = 128;                       // bytes of K per chunk (one swizzle atom row)
constexpr int kTileRows = 128;
constexpr int kPBytes = 2 * (kKc / 2) * 32;    // packed weights of one chunk, two row blocks: 4 KB
constexpr int kMaxN = 256;
constexpr int kTmemCols = 512;                 // columns 0..N-1 accumulators, then 32 columns per slot for the A operand
constexpr int kSmemBudget = 216 * 1024;        // activation ring + packed-weight ring

struct UmmaLaunch {
    tenzo_tl1_gemv_args a;
    const float* inv;        // [batch] m/31
    const int* sum_a;        // [batch] sum_k a_k
    int units;               // tiles along the rows
    int n_box;               // sequences per CTA, padded to a multiple of 16 (<= 256)
    int n_slots;             // ring slots (A in tensor memory, activation tile in shared memory)
    int n_pgroups;           // groups of kPGroup chunks in the packed-weight ring
    int ksplit;              // CTAs of a cluster that share one tile's K range (1 = no cluster)
    int store_cols;          // sequences per TMA store of the epilogue (32; 16 with a cluster or up to 64 sequences)
};

__device__ int g_umma_timeouts = 0;

// Optional in-kernel timeline (compile with -DTZ_UMMA_TRACE): CTA-local clock64 stamps per phase, read back through
// tenzo_trace_umma; compiled out of the library build.
#ifdef TZ_UMMA_TRACE
__device__ long long g_umma_trace[160 * 16];
#define UT(i) (g_umma_trace[(blockIdx.x % 160) * 16 + (i)] = clock64())
__device__ long long g_umma_chunks[64 * 8];      // CTA 0: per chunk, when each role reached it
#define UC(j, k) do { if (blockIdx.x == 0 && blockIdx.z == 0 && (j) < 64) g_umma_chunks[(j) * 8 + (k)] = clock64(); } while (0)
#define UTG(i) do { long long t_; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_)); g_umma_trace[(blockIdx.x % 160) * 16 + (i)] = t_; } while (0)
#else
#define UT(i) ((void)0)
#define UC(j, k) ((void)0)
#define UTG(i) ((void)0)
#endif

// Optional self-check (compile with -DTZ_UMMA_CHECK): every shared-memory range handed to a copy engine and every
// tensor-memory column range is checked against the allocation first; a violation is recorded (code, value, limit) and
// the access skipped. Read back through tenzo_check_umma; compiled out of the library build.
#ifdef TZ_UMMA_CHECK
__device__ unsigned long long g_umma_check[4];
__device__ __forceinline__ bool umma_check(bool good, int code, unsigned long long v, unsigned long long lim) {
    if (!good && atomicCAS(&g_umma_check[0], 0ull, (unsigned long long)code) == 0ull) { g_umma_check[1] = v; g_umma_check[2] = lim; g_umma_check[3] = blockIdx.x; }
    return good;
}
#define UCHK(good, code, v, lim) umma_check((good), (code), (unsigned long long)(v), (unsigned long long)(lim))
#else
#define UCHK(good, code, v, lim) true
#endif

__device__ __forceinline__ float umma_seg_scale(const tenzo_tl1_gemv_args& a, int block) {
    return block < a.seg_end[0] ? a.seg_scale[0] : (block < a.seg_end[1] ? a.seg_scale[1] : a.seg_scale[2]);
}

struct UmmaSmem {
    // [1024-aligned] ring n_slots x { B n_box*128 } | packed ring n_pgroups x 2 blocks x 16 KB | barriers | tmem slot | inv[256] | sum_a[256]
    static __host__ __device__ int pgroups_for(int n_box) { return n_box <= 64 ? kMaxPGroups : 2; }
    static __host__ __device__ int tmem_a(int n_box) { return (n_box + 31) & ~31; }          // first column of the A slots
    static __host__ __device__ int slots_for(int n_box) {
        const int by_tmem = (kTmemCols - tmem_a(n_box)) / 32, by_smem = (kSmemBudget - pgroups_for(n_box) * kPGroup * kPBytes) / (n_box * kKc);
        const int r = by_tmem < by_smem ? by_tmem : by_smem;
        // A multiple of four (the expand groups and the issuing threads): slot s then always belongs to group s % 4 and
        // thread s % 4, so every phase of a slot's barriers is seen, in order, by the same waiter. (A parity wait
        // cannot tell phase k from phase k - 2: with five slots a thread that ran ahead of its neighbour took a slot's
        // previous phase for the one it waited for and multiplied a tile that had not arrived.)
        return (r < kMaxSlots ? r : kMaxSlots) & ~3;
    }
    static constexpr int n_bars = 2 * kMaxSlots + 2 * kMaxPGroups + 3;
    static __host__ __device__ size_t bytes(int n_box) {
        return 1024 + (size_t)slots_for(n_box) * n_box * kKc + (size_t)pgroups_for(n_box) * kPGroup * kPBytes + ((8 * n_bars + 15) & ~15) + 16 + 2 * kMaxN * 4;
    }
};

// One 16-sequence block of the epilogue: r = accumulators of TMEM lane m (weight row `row`, `rr` inside its block).
template <int EPI>
__device__ __forceinline__ void umma_epilogue_block(const tenzo_tl1_gemv_args& a, uint32_t (&r)[16], const float* s_inv, const int* s_sum, float wscale,
                                                    int c0, int seq0, int block, int rr, int row, bool up_half, float* s_out_cols, float* s_glu_cols, bool ok) {
    float v[16];
#pragma unroll
    for (int i = 0; i < 16; i += 4) {
        const int4 sv = *reinterpret_cast<const int4*>(s_sum + c0 + i);
        const float4 iv = *reinterpret_cast<const float4*>(s_inv + c0 + i);
        const int s4[4] = {sv.x, sv.y, sv.z, sv.w};
        const float i4[4] = {iv.x, iv.y, iv.z, iv.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int accv = (int)r[i + e] - s4[e];
            r[i + e] = (uint32_t)accv;
            v[i + e] = (float)accv * (i4[e] * wscale);      // :1554, :118
        }
    }
    if (a.acc_out && ok && block >= 0) {
#pragma unroll
        for (int i = 0; i < 16; ++i)
            if (seq0 + c0 + i < a.batch) a.acc_out[(size_t)(seq0 + c0 + i) * a.n_blocks * 64 + block * 64 + rr] = (int)r[i];
    }
    if (EPI == TENZO_EPI_RELU2_GLU) {
        if (up_half) {                                   // the up value, and ReLU(gate)^2: multiplied once both are in place
#pragma unroll
            for (int i = 0; i < 16; ++i) s_glu_cols[i * 64 + rr] = v[i];
        } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const float rl = fmaxf(0.0f, v[i]);
                s_out_cols[i * 64 + rr] = rl * rl;                               // :1618
            }
        }
    } else if (EPI == TENZO_EPI_RESIDUAL) {
        float res[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const int seq = seq0 + c0 + i;
            res[i] = (seq < a.batch && block >= 0) ? __ldcg(a.resid + (size_t)seq * a.out_stride + block * 64 + rr) : 0.0f;
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) s_out_cols[i * 128 + row] = res[i] + v[i];                          // :1590
    } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) s_out_cols[i * 128 + row] = v[i];
    }
}

template <int EPI, bool CLUSTER>
__global__ void __launch_bounds__(kUmmaThreads, 1) tl1_umma_kernel(const UmmaLaunch L, const __grid_constant__ CUtensorMap amap,
                                                                   const __grid_constant__ CUtensorMap omap) {
    const tenzo_tl1_gemv_args& a = L.a;
    extern __shared__ unsigned char smem_raw[];
    const uint32_t base_off = ((smem_addr(smem_raw) + 1023u) & ~1023u) - smem_addr(smem_raw);
    unsigned char* ring = smem_raw + base_off;
    const int N = L.n_box, R = L.n_slots, slot_bytes = N * kKc;
    const int PG = L.n_pgroups;
    unsigned char* pring = ring + (size_t)R * slot_bytes;                       // [PG][2 row blocks][kPGroup chunks][64][32] packed weights
    uint64_t* bars = reinterpret_cast<uint64_t*>(pring + (size_t)PG * kPGroup * kPBytes);
    const uint32_t tmem_a0 = (uint32_t)UmmaSmem::tmem_a(N);
    uint64_t* bar_full = bars;                         // [R] A expanded (one arrival per expanding warp) and the activation tile landed
    uint64_t* bar_empty = bars + kMaxSlots;            // [R] the slot's MMAs have completed
    uint64_t* bar_p = bars + 2 * kMaxSlots;            // [PG] packed weights have landed
    uint64_t* bar_pfree = bar_p + kMaxPGroups;         // [PG] packed weights consumed (one arrival per expanding warp per chunk)
    uint64_t* bar_accum = bar_pfree + kMaxPGroups;        // every issuing thread's MMAs have completed
    uint64_t* bar_first = bar_accum + 1;               // chunk 0 (the one that overwrites the accumulators) has completed
    uint64_t* bar_meta = bar_first + 1;                // per-sequence scale and sum are in shared memory
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(reinterpret_cast<unsigned char*>(bars) + ((8 * UmmaSmem::n_bars + 15) & ~15));   // 16-byte aligned
    float* s_inv = reinterpret_cast<float*>(tmem_slot + 4);   // [kMaxN] m/31 of this CTA's sequences
    int* s_sum = reinterpret_cast<int*>(s_inv + kMaxN);       // [kMaxN] sum_k a_k

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) { UT(0); UTG(10); }
#ifdef TZ_UMMA_CHECK
    uint32_t dyn_bytes;
    asm volatile("mov.u32 %0, %%dynamic_smem_size;" : "=r"(dyn_bytes));
    const unsigned char* smem_end = smem_raw + dyn_bytes;
    UCHK(reinterpret_cast<const unsigned char*>(s_sum + kMaxN) <= smem_end, 7, reinterpret_cast<const unsigned char*>(s_sum + kMaxN) - smem_raw, dyn_bytes);
#endif
    constexpr bool glu = EPI == TENZO_EPI_RELU2_GLU;
    const int tile = blockIdx.x, seq0 = blockIdx.y * kMaxN;
    const int blk0 = glu ? tile : 2 * tile;
    const int blk1 = glu ? tile + L.units : (2 * tile + 1 < a.n_blocks ? 2 * tile + 1 : -1);
    const int ksplit = CLUSTER ? L.ksplit : 1;
    const int split = CLUSTER ? (int)cg::this_cluster().block_rank() : 0;         // cluster = the CTAs with this tile's blockIdx.z = 0..ksplit-1
    const int all_chunks = a.K / kKc;
    const int c_begin = split * all_chunks / ksplit;                                // this CTA's chunks of K: never empty (all_chunks >= ksplit)
    const int n_chunks = (split + 1) * all_chunks / ksplit - c_begin;

    const size_t blk_bytes = (size_t)(a.K / 2) * 32;
    const int n_groups = (n_chunks + kPGroup - 1) / kPGroup;
    auto request_group = [&](int g) {                      // packed weights of chunks kPGroup*g .. kPGroup*g + kPGroup-1, both row blocks
        const int slot = g % PG;
        const int chunks = min(kPGroup, n_chunks - g * kPGroup);
        const unsigned bytes = (unsigned)chunks * (kPBytes / 2);
        unsigned char* sP = pring + (size_t)slot * kPGroup * kPBytes;
        if (!UCHK(sP + 2 * kPGroup * (kPBytes / 2) <= reinterpret_cast<unsigned char*>(bars) && slot < PG && chunks > 0, 1, sP - smem_raw, g)) return;
        mbar_expect_tx(&bar_p[slot], blk1 >= 0 ? 2 * bytes : bytes);
        const size_t k_off = (size_t)(c_begin + g * kPGroup) * (kPBytes / 2);
        bulk_g2s(sP, a.w + (size_t)blk0 * blk_bytes + k_off, bytes, &bar_p[slot]);
        if (blk1 >= 0) bulk_g2s(sP + kPGroup * (kPBytes / 2), a.w + (size_t)blk1 * blk_bytes + k_off, bytes, &bar_p[slot]);
    };
    if (warp == 0 && lane < PG) {
        // The weights depend on no earlier kernel and their latency is the longest in the prologue: ask for the first
        // groups before anything else, one lane per group (an mbarrier operation or a bulk-copy issue costs its thread
        // over a hundred cycles; the other barriers are initialised by another warp meanwhile).
        mbar_init(&bar_p[lane], 1);
        mbar_init_fence();
        if (lane < n_groups) request_group(lane);
        if (lane == 0) UT(2);
    } else if (warp == 2) {
        if (lane < R) {
            mbar_init(&bar_full[lane], 5);             // four expanding warps + the expect_tx of the warp that requests the activation tile
            mbar_init(&bar_empty[lane], 1);
        } else if (lane >= 16 && lane < 16 + kMaxPGroups) {
            mbar_init(&bar_pfree[lane - 16], 4 * kExpandGroups * (R >= 8 ? 1 : 2));   // one arrival per expanding warp per iteration
        } else if (lane == 24) {
            mbar_init(bar_accum, kMmaThreads);
        } else if (lane == 25) {
            mbar_init(bar_first, 1);
        } else if (lane == 26) {
            mbar_init(bar_meta, 1);
        }
        mbar_init_fence();
    } else if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(tmem_slot)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (warp >= 3) l2_prefetch_slice(a.prefetch, a.prefetch_bytes);       // the next kernel's weights
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);
    if (a.use_pdl) pdl_launch_dependents();
    if (tid == 0) UT(1);
    bool timed_out = false, epi_ok = false;
    const int mma_t = warp == 1 ? 0 : warp - (1 + 4 * kExpandGroups);        // issuing thread 0..3: warp 1 and the three warps after the expand warps

    if (warp == 0) {
        if (lane == 0) {
            // ---- producer: the remaining groups of packed weights, each as soon as its ring half is free -------
            for (int gp = PG; gp < n_groups; ++gp) {
                const int slot = gp % PG, guse = gp / PG;
                if (!mbar_spin_bounded(&bar_pfree[slot], (unsigned)(guse - 1) & 1u)) { timed_out = true; break; }
                request_group(gp);
            }
        } else {
            // ---- per-sequence epilogue operands (quantiser outputs) ---------------------------------------
            if (a.use_pdl) pdl_wait();
            for (int i = lane - 1; i < N; i += 31) {
                const int seq = seq0 + i;
                s_inv[i] = seq < a.batch ? __ldcg(L.inv + seq) : 0.0f;
                s_sum[i] = seq < a.batch ? __ldcg(L.sum_a + seq) : 0;
            }
            __syncwarp(0xfffffffeu);
            if (lane == 1) mbar_arrive(bar_meta);
        }
    } else if (warp == 1 || warp >= 2 + 4 * kExpandGroups) {
        // ---- MMA issue: thread t takes chunks t, t + 4, ... ---------------------------------------------------
        if (lane == 0) {
            // c = s32, a = u8, b = s8, both K-major, N at bit 17 (>>3), M at bit 24 (>>4)
            const uint32_t idesc = (2u << 4) | (0u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(kTileRows >> 4) << 24);
            if (mma_t > 0 && mma_t < n_chunks && !mbar_spin_bounded(bar_first, 0u)) timed_out = true;
            for (int j = mma_t; j < n_chunks && !timed_out; j += kMmaThreads) {
                const int s = j % R, use = j / R;
                UC(j, 4);
                if (!mbar_spin_bounded(&bar_full[s], (unsigned)use & 1u)) { timed_out = true; break; }
                tc_fence_after();
                UC(j, 5);
                const uint32_t ta = tmem_base + tmem_a0 + (uint32_t)(32 * s);
                const uint64_t db = umma_desc_sw128(smem_addr(ring + (size_t)s * slot_bytes));
                if (UCHK(tmem_a0 + 32 * s + 32 <= (uint32_t)kTmemCols && s < R && ring + (size_t)(s + 1) * slot_bytes <= pring, 5, s, j))
#pragma unroll
                for (int k4 = 0; k4 < kKc / 32; ++k4)
                    umma_i8_ta(tmem_base, ta + (uint32_t)(8 * k4), db + (uint64_t)(2 * k4), idesc, (j > 0 || k4 > 0) ? 1u : 0u);
                umma_commit(&bar_empty[s]);
                UC(j, 6);
                if (j == 0) umma_commit(bar_first);
            }
            umma_commit(bar_accum);
        }
    } else {
        // ---- expand the 2-bit codes into tensor memory ----------------------------------------------------------
        // Quarter q = warp & 3 owns TMEM lanes 32q..32q+31 = row block q >> 1, nibble half q & 1. Thread 4g + t holds
        // lanes g + 8*jj (jj = 0..3) = rows 4g + jj of the half = the four bytes of packed word g of a column pair, and
        // the columns 8n + 2t, 8n + 2t + 1 = column pairs 16n + 4t .. 16n + 4t + 3. The four words of a (thread, n) are
        // fetched in the order u ^ t so that a warp's request covers 32 banks; the byte permutes that transpose them
        // take the order back (selectors chosen per thread).
        const int q = warp & 3, grp = (warp - 2) >> 2;
        const int blk = q >> 1, hi = q & 1, g = lane >> 2, t = lane & 3;
        const bool have = blk == 0 || blk1 >= 0;
        const uint32_t sel_a = (t & 1) ? 0x1504u : 0x5140u, sel_b = (t & 1) ? 0x3726u : 0x7362u;
        const uint32_t sel_lo = (t & 2) ? 0x1054u : 0x5410u, sel_hi = (t & 2) ? 0x3276u : 0x7632u;
        int woff[4];                                           // word offsets of the four loads inside a 16-column-pair set
#pragma unroll
        for (int u = 0; u < 4; ++u) woff[u] = (4 * t + (u ^ t)) * 8 + g;
        // An iteration costs a warp about two thousand cycles whatever it expands (a poll of a barrier that has long
        // completed is 300 cycles, a tensor-memory store 500 until it has landed), so with eight or more slots it takes
        // two chunks, j and j + 4: one poll for both slots (the same thread issues both chunks' MMAs in order, so the
        // later one's completion implies the earlier one's), one for the weights (both lie in the same group of eight),
        // the two polls on different lanes, one wait for the four stores.
        const int cpi = R >= 8 ? 2 : 1;
        int seen_group = -1;
        for (int it = 0, j0 = grp; j0 < n_chunks; ++it, j0 += kExpandGroups * cpi) {
            const int n_here = (cpi == 2 && j0 + kExpandGroups < n_chunks) ? 2 : 1;
            const int j_last = j0 + kExpandGroups * (n_here - 1);
            const int pg = j0 / kPGroup, ps = pg % PG, puse = pg / PG;
            bool ok = true;
            if (lane == 0 && q == 0) { UC(j0, 0); if (n_here == 2) UC(j0 + kExpandGroups, 0); }
            if (lane == 0) {
                const int s = j_last % R, use = j_last / R;
                ok = use == 0 || mbar_spin_bounded(&bar_empty[s], (unsigned)(use - 1) & 1u);
            } else if (lane == 1 && pg != seen_group) {
                ok = mbar_spin_bounded(&bar_p[ps], (unsigned)puse & 1u);
            }
            seen_group = pg;
            ok = __all_sync(0xffffffffu, ok);
            __syncwarp();                                   // what lanes 0 and 1 acquired is visible to the whole warp
            if (j0 == 0 && tid == 64) UT(6);
            if (!ok) { timed_out = true; break; }
            tc_fence_after();
            if (lane == 0 && q == 0) { UC(j0, 1); if (n_here == 2) UC(j0 + kExpandGroups, 1); }
            // The group's warps take turns requesting the activation tiles. They come from the previous kernel, so in the
            // first iteration the request (and the wait for that kernel) is left until the chunks have been expanded:
            // the weights depend on nothing, and the previous kernel runs about as long as the first round of expansion.
            auto request_tiles = [&]() {
                for (int c = 0; c < n_here; ++c) {
                    const int j = j0 + kExpandGroups * c, s = j % R;
                    if (lane == 0 && ((it * cpi + c) & 3) == q) {
                        if (UCHK(s < R && ring + (size_t)(s + 1) * slot_bytes <= pring, 2, s, j)) {
                            mbar_expect_tx(&bar_full[s], (unsigned)slot_bytes);
                            tma_load_2d(ring + (size_t)s * slot_bytes, &amap, (c_begin + j) * kKc, seq0, &bar_full[s]);
                        }
                    }
                }
            };
            const bool request_last = it == 0 && a.use_pdl;
            if (!request_last) request_tiles();
            for (int c = 0; c < n_here; ++c) {
                const int j = j0 + kExpandGroups * c, s = j % R;
                const uint32_t* sP = reinterpret_cast<const uint32_t*>(pring + (size_t)ps * kPGroup * kPBytes + (size_t)blk * kPGroup * (kPBytes / 2) +
                                                                       (size_t)(j % kPGroup) * (kPBytes / 2));
                uint32_t W[16];
                const bool sp_ok = UCHK(reinterpret_cast<const unsigned char*>(sP) >= pring && reinterpret_cast<const unsigned char*>(sP + 512) <= reinterpret_cast<unsigned char*>(bars), 3,
                                        reinterpret_cast<const unsigned char*>(sP) - smem_raw, j);
#pragma unroll
                for (int n = 0; n < 4; ++n)
#pragma unroll
                    for (int u = 0; u < 4; ++u) W[4 * n + u] = (have && sp_ok) ? sP[n * 128 + woff[u]] : 0u;
                uint32_t lo[16], up[16];                       // registers of the two stores: lanes 0-15 (jj = 0, 1) and 16-31 (jj = 2, 3)
#pragma unroll
                for (int n = 0; n < 4; ++n) {
                    // 4x4 byte transpose: T[jj] = byte jj of the words of column pairs 16n + 4t + 0..3
                    const uint32_t p0 = prmt(W[4 * n], W[4 * n + 1], sel_a), p1 = prmt(W[4 * n + 2], W[4 * n + 3], sel_a);
                    const uint32_t p2 = prmt(W[4 * n], W[4 * n + 1], sel_b), p3 = prmt(W[4 * n + 2], W[4 * n + 3], sel_b);
                    const uint32_t T[4] = {prmt(p0, p1, sel_lo), prmt(p0, p1, sel_hi), prmt(p2, p3, sel_lo), prmt(p2, p3, sel_hi)};
#pragma unroll
                    for (int jj = 0; jj < 4; ++jj) {
                        const uint32_t nb = T[jj] >> (4 * hi);
                        const uint32_t e = nb & 0x03030303u, o = (nb >> 2) & 0x03030303u;    // codes of the even / odd columns
                        uint32_t* dst = (jj < 2 ? lo : up) + 4 * n + 2 * (jj & 1);
                        dst[0] = prmt(e, o, 0x5140u);
                        dst[1] = prmt(e, o, 0x7362u);
                    }
                }
                const uint32_t ta = tmem_base + tmem_a0 + (uint32_t)(32 * s) + ((uint32_t)(32 * q) << 16);
                if (UCHK(tmem_a0 + 32 * s + 32 <= (uint32_t)kTmemCols && (tmem_base & 0xffffu) == 0u, 4, tmem_a0 + 32 * s, tmem_base)) {
                    tmem_st_16x256b_x4(ta, lo);
                    tmem_st_16x256b_x4(ta + (16u << 16), up);
                }
            }
            if (lane == 0 && q == 0) { UC(j0, 2); if (n_here == 2) UC(j0 + kExpandGroups, 2); }
            __syncwarp();
            if (lane == 0) mbar_arrive(&bar_pfree[ps]);       // every lane's packed words have been loaded and used
            if (request_last) {
                if (lane == 0) pdl_wait();
                request_tiles();
            }
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane < n_here) mbar_arrive(&bar_full[(j0 + kExpandGroups * lane) % R]);
            if (lane == 0 && q == 0) { UC(j0, 3); if (n_here == 2) UC(j0 + kExpandGroups, 3); }
        }
        // ---- all of this CTA's MMAs have completed; in a cluster it parks its partial tile [N][128 TMEM lanes] int32
        //      (the column blocks its peers will reduce) in the ring memory the pipeline no longer needs -----------------
        if (a.use_pdl) pdl_wait();                           // the residual rows come from an earlier kernel (long done by now)
        bool ok = true;
        if (lane == 0) ok = !timed_out && mbar_spin_bounded(bar_meta, 0u) && mbar_spin_bounded(bar_accum, 0u);
        ok = __shfl_sync(0xffffffffu, ok, 0);
        __syncwarp();
        if (!ok) timed_out = true;
        tc_fence_after();
        if (tid == 64) UT(7);
        epi_ok = ok;
        if (CLUSTER) {
            const int m = 32 * q + lane;
            int* s_part = reinterpret_cast<int*>(ring);
            for (int c0 = 16 * grp; c0 < N; c0 += 16 * kExpandGroups) {
                if ((c0 >> 4) % ksplit == split) continue;       // this CTA's own column blocks stay in tensor memory
                uint32_t r[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) r[i] = 0u;
                if (ok) tmem_ld16(tmem_base + ((uint32_t)(32 * q) << 16) + (uint32_t)c0, r);
#pragma unroll
                for (int i = 0; i < 16; ++i) s_part[(c0 + i) * 128 + m] = (int)r[i];
            }
        }
    }
    if (CLUSTER) cg::this_cluster().sync();                  // every CTA's partial tile is in place
    if (warp >= 2 && warp < 2 + 4 * kExpandGroups) {
        // ---- epilogue: every group, alternate column units; TMEM lane -> weight row through the quarter's permutation ----
        const bool ok = epi_ok;
        const int q = warp & 3, grp = (warp - 2) >> 2;
        const int m = 32 * q + lane;                         // TMEM lane
        const int rblk = q >> 1, rr = 32 * (q & 1) + 4 * (lane & 7) + (lane >> 3), row = 64 * rblk + rr;
        const int block = rblk ? blk1 : blk0;
        const float wscale = block >= 0 ? umma_seg_scale(a, block) : 0.0f;
        // Output columns [sequences][128 rows] (GLU: [..][64]) are assembled in shared memory the pipeline no longer
        // needs - the rings, which are contiguous; with a cluster behind the partial tile the peers are reading - and
        // leave unit by unit through TMA stores: rows of 512 (256) contiguous bytes per sequence, clipped at the
        // matrix edge by the tensor map. GLU: the up half parks its values and the gate half its ReLU^2 side by side, then
        // the group multiplies them in place. Space: N*512 bytes without a cluster (at least four slots), N*512 plus 512 per
        // own column with one (a rank owns at most every other block), which the two rings hold for every N.
        constexpr int row_floats = glu ? 64 : 128;
        const int SB = L.store_cols >> 4;                    // 16-sequence blocks per store unit: 2, or 1 (a cluster; few sequences)
        float* s_out = reinterpret_cast<float*>(ring + (CLUSTER ? (size_t)N * 512 : 0));            // behind the partial tile [N][128] int32
        float* s_glu = s_out + (size_t)(CLUSTER ? 16 * ((N / 16 + 1) / 2) : N) * 64;                 // behind the GLU output columns (a rank owns at most every other block)
        const int n_blocks16 = N / 16;
        const int own_blocks = CLUSTER ? (n_blocks16 - split + ksplit - 1) / ksplit : n_blocks16;
        const int n_units = (own_blocks + SB - 1) / SB;
        const bool leader = lane == 0 && q == 0;
        const uint32_t t_lane = tmem_base + ((uint32_t)(32 * q) << 16);
#pragma unroll 1
        for (int un = grp; un < n_units; un += kExpandGroups) {
            const int ob0 = un * SB;
            const bool two = SB == 2 && ob0 + 1 < own_blocks;
            const int c0 = 16 * (CLUSTER ? split + ksplit * ob0 : ob0);
            uint32_t r0[16], r1[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) r0[i] = r1[i] = 0u;
            if (ok) {
                tmem_ld16_nowait(t_lane + (uint32_t)c0, r0);
                if (two) tmem_ld16_nowait(t_lane + (uint32_t)(c0 + 16), r1);
                tmem_wait_ld();
            }
            if (CLUSTER) {
                // the peers' partials over distributed shared memory: every load issued before the first is
                // used (ranks beyond the cluster and this CTA's own read its own tile and are masked out)
#pragma unroll
                for (int p = 0; p < 8; ++p) {
                    const bool use_p = p < ksplit && p != split;
                    const int* peer = cg::this_cluster().map_shared_rank(reinterpret_cast<int*>(ring), use_p ? p : split);
                    const uint32_t mask = use_p ? 0xffffffffu : 0u;
#pragma unroll
                    for (int i = 0; i < 16; ++i) r0[i] += mask & (uint32_t)peer[(c0 + i) * 128 + m];
                }
            }
            float* unit_out = s_out + (size_t)16 * ob0 * row_floats;
            float* unit_glu = s_glu + (size_t)16 * ob0 * 64;
            umma_epilogue_block<EPI>(a, r0, s_inv, s_sum, wscale, c0, seq0, block, rr, row, rblk == 1, unit_out, unit_glu, ok);
            if (two)
                umma_epilogue_block<EPI>(a, r1, s_inv, s_sum, wscale, c0 + 16, seq0, block, rr, row, rblk == 1, unit_out + 16 * row_floats,
                                         unit_glu + 16 * 64, ok);
            if (glu) {
                // gate and up halves of the unit are both in shared memory: out = ReLU(gate)^2 * up, four floats at a time
                named_barrier_sync(1 + grp, 128);
                const int n4 = (two ? 32 : 16) * 64 / 4;
                float4* o4 = reinterpret_cast<float4*>(unit_out);
                const float4* g4 = reinterpret_cast<const float4*>(unit_glu);
                for (int i = 32 * q + lane; i < n4; i += 128) {
                    float4 o = o4[i];
                    const float4 u = g4[i];
                    o.x *= u.x; o.y *= u.y; o.z *= u.z; o.w *= u.w;             // :1619
                    o4[i] = o;
                }
            }
            // the unit is complete in shared memory: hand it to the TMA and go on with the next one
            fence_proxy_async_smem();
            named_barrier_sync(1 + grp, 128);
            if (leader && ok && seq0 + c0 < a.batch &&
                UCHK(reinterpret_cast<unsigned char*>(unit_out) + 16 * SB * row_floats * 4 <= reinterpret_cast<unsigned char*>(bars), 6,
                     reinterpret_cast<unsigned char*>(unit_out) - smem_raw, un)) {             // else nothing but padding
                asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];"
                             ::"l"(&omap), "r"((glu ? tile : blk0) * 64), "r"(seq0 + c0), "r"(smem_addr(unit_out)) : "memory");
                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            }
        }
        if (tid == 64) UT(8);
        if (leader) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");     // the tiles have left shared memory
        if (tid == 64) UT(9);
    }
    if (CLUSTER) cg::this_cluster().sync();                  // every peer has read this CTA's partial tile: it may exit
    if (timed_out) atomicExch(&g_umma_timeouts, 1);
    tc_fence_before();
    if (__syncthreads_or(timed_out ? 1 : 0)) {
        // A role gave up: copies it no longer waits for may still be on their way into this CTA's shared memory, and
        // MMAs it issued may still be running. Give them a bounded time (about 100 us; a copy lands within a few) before
        // the memory and the tensor-memory columns go back to the SM.
        const long long t_end = clock64() + 200000;
        while (clock64() < t_end) __nanosleep(1000);
        __syncthreads();
    }
    if (tid == 0) UTG(11);
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
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
    L.n_slots = UmmaSmem::slots_for(L.n_box);
    L.n_pgroups = UmmaSmem::pgroups_for(L.n_box);
    const int seq_tiles = (a.batch + kMaxN - 1) / kMaxN;
    L.ksplit = pick_umma_ksplit(L.units * seq_tiles, a.K / kKc);
    L.store_cols = (L.ksplit > 1 || L.n_box <= 64) ? 16 : 32;      // few sequences: 16 per unit, so that every group gets one
    CUtensorMap amap, omap;
    // activations [batch][K] int8: B-operand tiles {128 bytes of K, n_box sequences}, 128-byte swizzle
    if (int rc = encode_2d(&amap, CU_TENSOR_MAP_DATA_TYPE_UINT8, a8, (uint64_t)a.K, (uint64_t)a.batch, (uint64_t)a.K, kKc, (uint32_t)L.n_box,
                           CU_TENSOR_MAP_SWIZZLE_128B)) return rc;
    // output [batch][n_out] fp32: store units {128 (GLU: 64) rows of the weight matrix, 32 sequences (16: the column
    // blocks a cluster's CTAs store separately)}
    const uint64_t n_out = (uint64_t)(glu ? a.n_blocks / 2 : a.n_blocks) * 64;
    if (int rc = encode_2d(&omap, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, a.out, n_out, (uint64_t)a.batch, (uint64_t)a.out_stride * 4, glu ? 64u : 128u,
                           (uint32_t)L.store_cols, CU_TENSOR_MAP_SWIZZLE_NONE)) return rc;
    const size_t smem = UmmaSmem::bytes(L.n_box);
    using Kernel = void (*)(const UmmaLaunch, const CUtensorMap, const CUtensorMap);
    const bool cl = L.ksplit > 1;
    Kernel kernel = a.epilogue == TENZO_EPI_RELU2_GLU   ? (cl ? tl1_umma_kernel<TENZO_EPI_RELU2_GLU, true> : tl1_umma_kernel<TENZO_EPI_RELU2_GLU, false>)
                    : a.epilogue == TENZO_EPI_RESIDUAL ? (cl ? tl1_umma_kernel<TENZO_EPI_RESIDUAL, true> : tl1_umma_kernel<TENZO_EPI_RESIDUAL, false>)
                                                       : (cl ? tl1_umma_kernel<TENZO_EPI_STORE, true> : tl1_umma_kernel<TENZO_EPI_STORE, false>);
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
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
    e = cudaLaunchKernelEx(&cfg, kernel, L, amap, omap);
    return e == cudaSuccess ? 0 : (int)e;
}


int tl1_umma_take_timeouts() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_umma_timeouts, sizeof v) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(g_umma_timeouts, &zero, sizeof zero);
    return v;
}

}  // namespace tz

#ifdef TZ_UMMA_CHECK
extern "C" __attribute__((visibility("default"))) int tenzo_check_umma(unsigned long long* out) {
    return (int)cudaMemcpyFromSymbol(out, tz::g_umma_check, sizeof(unsigned long long) * 4);
}
#endif
#ifdef TZ_UMMA_TRACE
extern "C" __attribute__((visibility("default"))) int tenzo_trace_umma(long long* out) {
    return (int)cudaMemcpyFromSymbol(out, tz::g_umma_trace, sizeof(long long) * 160 * 16);
}
extern "C" __attribute__((visibility("default"))) int tenzo_trace_umma_chunks(long long* out) {
    return (int)cudaMemcpyFromSymbol(out, tz::g_umma_chunks, sizeof(long long) * 64 * 8);
}
#endif

extern "C" int tenzo_cuda_tl1_gemm_layout(int batch, int* slots, int* weight_groups, size_t* smem_bytes, size_t* epilogue_bytes) {
    if (batch < 16) return -1;
    const int per_cta = batch < tz::kMaxN ? batch : tz::kMaxN, n_box = (per_cta + 15) & ~15;
    if (slots) *slots = tz::UmmaSmem::slots_for(n_box);
    if (weight_groups) *weight_groups = tz::UmmaSmem::pgroups_for(n_box);
    if (smem_bytes) *smem_bytes = tz::UmmaSmem::bytes(n_box);
    // without a cluster: the output columns [n_box][128] fp32 (GLU: [n_box][64] twice); with one: behind the partial tile
    // [n_box][128] int32, the columns of the blocks a rank owns (at most every other 16-sequence block)
    if (epilogue_bytes) *epilogue_bytes = (size_t)n_box * 512 + (size_t)16 * ((n_box / 16 + 1) / 2) * 512;
    return 0;
}

extern "C" int tenzo_cuda_tl1_gemm_ksplit(int n_blocks, int K, int batch, int epilogue) {
    if (n_blocks <= 0 || K < tz::kKc || K % tz::kKc || batch < 16) return 0;       // the tensor-core path does not apply
    const int units = epilogue == TENZO_EPI_RELU2_GLU ? n_blocks / 2 : (n_blocks + 1) / 2;
    return tz::pick_umma_ksplit(units * ((batch + tz::kMaxN - 1) / tz::kMaxN), K / tz::kKc);
}
