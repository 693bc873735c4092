// TL1 ternary GEMV / skinny GEMM for sm_100a on the int8 tensor-core path (mma.sync m16n8k32,
// u8 x s8 -> s32), with the RMSNorm + absmax(31) activation quantiser fused into its prologue at
// batch 1 and the reference's three epilogues (store / residual add / squared-ReLU GLU).
//
// What it replaces in the reference CPU engine (src/runtime/TenzoEngine.cpp): rms_norm_raw
// (:148-166), build_lut (:22-62), compute_single_block (:64-127) and their call sites (:1542-1628).
//
// How the arithmetic is organised on the GPU
//   * The reference looks every 4-bit index up in a 16-entry table of clamp(w0*a0+w1*a1). With
//     |a| <= 31 the clamp can never fire, so the accumulator is the plain integer dot product
//     sum_k w[r][k]*a[k]; any exact integer evaluation gives the same int32.
//   * Weights stay in the reference's layout [N/64][K/2][32 B]. Lane (g = lane>>2, t = lane&3) of a
//     warp reads, for a "set" of 16 column pairs, the four 32-bit words at byte 4g of column pairs
//     16s+4i+t (i = 0..3) from the staged copy (bank-conflict free). A 4x4 byte transpose
//     (8 PRMT) turns them into T[j] = row pair 4g+j at those four column pairs.
//   * A byte of the layout is c0 | c1<<2 | c2<<4 | c3<<6 with codes c = w+1 in {0,1,2}: (c0,c1) =
//     row c at columns (2p,2p+1), (c2,c3) = row c+32. Masking without shifting gives bytes
//     c0, 4c1, 16c2, 64c3 — four ready-made u8 A fragments of mma.m16n8k32:
//        a0 = T&0x03.. (row 4g+j, even cols)    a2 = T&0x0C.. (row 4g+j, odd cols, x4)
//        a1 = T&0x30.. (row 32+4g+j, even, x16) a3 = T&0xC0.. (row 32+4g+j, odd, x64)
//     The B fragment holds the int8 activations of up to 8 sequences, even columns pre-multiplied
//     by 4 (|4a| <= 124), so the low rows accumulate 4*sum(c*a) and the high rows 64*sum(c*a).
//     One LOP3 per fragment register, four MMAs per 512 weight bytes per 8 sequences, and the
//     tensor core does the reduction over k that a dot-product kernel would do with shuffles.
//   * sum(w*a) = sum(c*a) - sum(a); sum(a) per sequence is accumulated while the activations are
//     staged.
//   * K can be split across the CTAs of a thread-block cluster (2, 4 or 8): partials meet in the
//     leader CTA's shared memory through distributed-shared-memory atomicAdd (integer, hence
//     order-free and exact) between hardware cluster barriers; the leader runs the epilogue.
//   * Each CTA brings its weight bytes into shared memory with 1-D bulk asynchronous copies (TMA)
//     completing on mbarriers, issued by one thread as the very first thing the kernel does: tens
//     of kilobytes per SM are in flight from a handful of instructions, which ordinary loads cannot
//     do (the load/store unit's request queue saturates at a fraction of the HBM latency-bandwidth
//     product). Every wait on an mbarrier is bounded; a give-up raises a flag the host can read.
//   * Nothing that does not depend on the previous kernel waits for it: the bulk copies, the norm
//     weights and an L2 prefetch of the NEXT kernel's weights are issued before griddepcontrol.wait.
//   * batch == 1: every CTA normalises and quantises the activation itself (bit-identical to the
//     reference, see common.cuh) and only packs the columns of its own K range.
//     batch > 1: act_quant_kernel (norm_quant.cu) has written packed int8 activations to a
//     workspace; CTAs stage their K range for 8 or 32 sequences and reuse every weight word for all.
#include <cooperative_groups.h>
#include <type_traits>

#include "common.cuh"
#include "attn_common.cuh"
#include "../../include/tenzo_kernels.h"

namespace tz {

namespace cg = cooperative_groups;

#ifndef TZ_FUSED_WARPS
#define TZ_FUSED_WARPS 16
#endif
constexpr int kFusedWarps = TZ_FUSED_WARPS;    // batch 1: one CTA per row block; two fit on an SM so consecutive kernels overlap
constexpr int kBatchedWarps = 16;

struct GemvLaunch {
    tenzo_tl1_gemv_args a;
    int ksplit;      // cluster size along K
    int units;       // CTAs along the row dimension (n_blocks, or n_blocks/2 in GLU mode)
    int nsets;       // ceil(K/2 / 16)
    const uint32_t* act_words;   // batch > 1: [batch][nsets][4][2] packed activations
    const float* act_inv;        // batch > 1: [batch] m/31
};

__device__ __forceinline__ float seg_scale_for(const tenzo_tl1_gemv_args& a, int block) {
    return block < a.seg_end[0] ? a.seg_scale[0] : (block < a.seg_end[1] ? a.seg_scale[1] : a.seg_scale[2]);
}

__device__ __forceinline__ void mma_u8s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t ld_stream_u32(const void* p) {
    uint32_t v;
    asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}

// Optional in-kernel timeline (compile with -DTZ_TRACE): first and last CTA record their SM's cycle counter at
// stage boundaries into g_trace (16 words per record; stamps 0-6 are the stages, 8-12 lie inside the prologue; word 15:
// block index, grid size in the upper half), read and reset by tenzo_trace_gemv(); compiled out of the library build.
#ifdef TZ_TRACE
__device__ unsigned long long g_trace[4096 * 16];
__device__ unsigned int g_trace_n;
#define TZ_TRACE_DECL unsigned long long tr[16] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0}
#define TZ_STAMP(k) do { if (threadIdx.x == 0 && (blockIdx.x == 0 || blockIdx.x == gridDim.x - 1)) tr[k] = (unsigned long long)clock64(); } while (0)
#define TZ_TRACE_FLUSH do { if (threadIdx.x == 0 && (blockIdx.x == 0 || blockIdx.x == gridDim.x - 1)) { \
    const unsigned slot = atomicAdd(&g_trace_n, 1u); \
    if (slot < 4096) { for (int k = 0; k < 15; ++k) g_trace[slot * 16 + k] = tr[k]; \
                       g_trace[slot * 16 + 15] = blockIdx.x | ((unsigned long long)gridDim.x << 32); } } } while (0)
#else
#define TZ_TRACE_DECL do {} while (0)
#define TZ_STAMP(k) do {} while (0)
#define TZ_TRACE_FLUSH do {} while (0)
#endif

#ifndef TZ_GEMV_CHUNKS
#define TZ_GEMV_CHUNKS 1
#endif
// Bulk copies (and mbarriers) per row block. One: a bulk copy costs about the same whatever its size (measured: an SM
// completes roughly one copy per 0.45 us up to 16 KB), so splitting a 40 KB slice into eight pieces to start computing on
// the first cost more than it gained (decode went 820 -> 865 tok/s with one copy).
constexpr int kChunks = TZ_GEMV_CHUNKS;

__device__ int g_tl1_timeouts = 0; // set when a bounded mbarrier wait gave up (the result of that launch is invalid)

// One sequence, 4096 < K <= 8192: a thread owns up to four 16-byte pieces of the input vector and parks their norm weights in
// a private shared-memory slot while it waits (see the prologue): [4][threads] float4.
__host__ __device__ constexpr int own_park_floats(int K) { return (K > 2 * 4 * kFusedWarps * 32 && K <= 4 * 4 * kFusedWarps * 32) ? 4 * kFusedWarps * 32 * 4 : 0; }

template <int NT, bool FUSED>
struct GemvSmem {
    static constexpr int SL = FUSED ? 1 : 8 * NT;                       // sequences per CTA
    // 32-bit words: s_d[128*SL] | s_sa4[SL] | s_inv[SL] | scratch[32] | mbarriers[2*kChunks x 2 words]
    //               | s_b[sets*SL*8] | weights[nb_cta*sets*128] | (fused) x[K]
    static __host__ __device__ int head_words() { return (128 * SL + 2 * SL + 32 + 2 + 4 * kChunks + 3) & ~3; }
    static __host__ __device__ size_t bytes(int sets_per_cta, int K, int nb_cta) {
        return (size_t)(head_words() + sets_per_cta * SL * 8 + nb_cta * sets_per_cta * 128 + (FUSED ? K + 64 + own_park_floats(K) : 0)) * 4;   // x, or its squares in padded chain-major rows (+ parked norm weights)
    }
};

template <int NT, bool FUSED>
__global__ void __launch_bounds__((FUSED ? kFusedWarps : kBatchedWarps) * 32, FUSED ? 2 : 1) tl1_mma_kernel(const GemvLaunch L) {
    constexpr int kGemvWarps = FUSED ? kFusedWarps : kBatchedWarps;
    constexpr int kGemvThreads = kGemvWarps * 32;
    using Lay = GemvSmem<NT, FUSED>;
    constexpr int SL = Lay::SL;
    const tenzo_tl1_gemv_args& a = L.a;
    extern __shared__ __align__(16) uint32_t smem[];
    int* s_d = reinterpret_cast<int*>(smem);                 // [rows_cta][SL] scaled accumulators
    int* s_sa4 = s_d + 128 * SL;                             // [SL] 4 * sum(a) over this CTA's columns
    float* s_inv = reinterpret_cast<float*>(s_sa4 + SL);     // [SL] m/31 per sequence
    float* s_f = s_inv + SL;                                 // [32] reduction scratch
    uint64_t* s_bar = reinterpret_cast<uint64_t*>(smem + ((128 * SL + 2 * SL + 32 + 1) & ~1));   // [2][kChunks]
    uint32_t* s_b = smem + Lay::head_words();                // [sets][SL][4 t][2] packed activations

    TZ_TRACE_DECL;
    TZ_STAMP(0);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t4 = lane & 3;
    const int unit = blockIdx.x / L.ksplit, split = blockIdx.x % L.ksplit, seq0 = blockIdx.y * SL;
    const bool glu = a.epilogue == TENZO_EPI_RELU2_GLU;
    const int nb_cta = glu ? 2 : 1;                 // row blocks handled by this CTA
    const int wb = kGemvWarps / nb_cta;             // warps per row block
    const int my_blk = glu ? (warp & 1) : 0;        // which of the CTA's row blocks this warp feeds
    const int wi = glu ? (warp >> 1) : warp;        // index among the warps of that row block
    const int kh = a.K >> 1;                        // column pairs
    cg::cluster_group cluster = cg::this_cluster();

    // K range of this CTA in sets of 16 column pairs (512 weight bytes per row block per set)
    const int s_begin = (int)(((long long)L.nsets * split) / L.ksplit);
    const int s_end = (int)(((long long)L.nsets * (split + 1)) / L.ksplit);
    const int n_cta_sets = s_end - s_begin;
    const int my_sets = (n_cta_sets - wi + wb - 1) / wb;   // this warp takes sets wi, wi+wb, ... of the range
    uint32_t* s_wt = s_b + n_cta_sets * SL * 8;              // [nb_cta][n_cta_sets][128 words] weights as in memory
    float* s_x = reinterpret_cast<float*>(s_wt + nb_cta * n_cta_sets * 128);   // fused only: x[K]
    const int sets_per_chunk = (n_cta_sets + kChunks - 1) / kChunks;

    // ---- weights: bulk-copy this CTA's slice of each row block into shared memory ----------------
    // They do not depend on the previous kernel, so they are requested before anything else.
    const unsigned range_bytes = (unsigned)(min(s_end * 512, kh * 32) - s_begin * 512);
    if (tid == 0) {
        for (int i = 0; i < nb_cta * kChunks; ++i) mbar_init(&s_bar[i], 1);
        mbar_init_fence();
        for (int bk = 0; bk < nb_cta; ++bk) {
            const int block = bk ? unit + L.units : unit;
            const uint8_t* src = a.w + (size_t)block * kh * 32 + (size_t)s_begin * 512;
            for (int c = 0; c < kChunks; ++c) {
                const unsigned off = (unsigned)c * sets_per_chunk * 512;
                const unsigned bytes = off < range_bytes ? min((unsigned)sets_per_chunk * 512, range_bytes - off) : 0u;
                mbar_expect_tx(&s_bar[bk * kChunks + c], bytes);   // zero bytes completes the phase at once
                if (bytes)
                    bulk_g2s(reinterpret_cast<uint8_t*>(s_wt + bk * n_cta_sets * 128) + off, src + off, bytes, &s_bar[bk * kChunks + c]);
            }
        }
    }
    l2_prefetch_slice(a.prefetch, a.prefetch_bytes);

    const int rows_cta = nb_cta * 64;
    for (int i = tid; i < rows_cta * SL; i += kGemvThreads) s_d[i] = 0;
    for (int i = tid; i < SL; i += kGemvThreads) s_sa4[i] = 0;
    constexpr int kWRegs = 16;                      // norm weights held in registers while waiting (K <= 16*threads)
    float wreg[kWRegs];
    const bool has_w = FUSED && a.do_norm && a.norm_w;
    const bool w_in_regs = has_w && a.K <= kWRegs * kGemvThreads;
    // Prologue form for K a multiple of 32 up to 8192 with 16-byte aligned vectors: every thread OWNS the elements it loads
    // (16-byte pieces f = tid, tid + threads, ...; elements 4f..4f+3) and keeps them in registers from the load to the
    // quantised bytes, which it stores straight into the packed activation words: no shared-memory round trip for the
    // normalised vector and no second pass over it. Up to two pieces per thread (K <= 4096) their norm weights wait in
    // registers too; with up to four, the thread parks the weights in a shared-memory slot of its own before the wait and
    // takes them back after the sum of squares (sixteen more live registers would not fit the 64 that two CTAs per SM
    // leave a thread).
    const int n_pieces = a.K >> 2;
    const bool own_ok = FUSED && (a.K & 31) == 0 &&
                        ((reinterpret_cast<uintptr_t>(a.x + (size_t)seq0 * a.x_stride) | (has_w ? reinterpret_cast<uintptr_t>(a.norm_w) : 0)) & 15) == 0;
    const int own_p = !own_ok ? 0 : n_pieces <= 2 * kGemvThreads ? 2 : n_pieces <= 4 * kGemvThreads ? 4 : 0;
    float4* s_w4 = reinterpret_cast<float4*>(s_x + a.K + 64);          // [4][threads], own_p == 4 only
    if (own_p == 2 && has_w) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int f = tid + j * kGemvThreads;
            const float4 w4 = f < n_pieces ? __ldg(reinterpret_cast<const float4*>(a.norm_w) + f) : make_float4(0.f, 0.f, 0.f, 0.f);
            wreg[4 * j] = w4.x; wreg[4 * j + 1] = w4.y; wreg[4 * j + 2] = w4.z; wreg[4 * j + 3] = w4.w;
        }
    } else if (own_p == 4 && has_w) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int f = tid + j * kGemvThreads;
            if (f < n_pieces) s_w4[j * kGemvThreads + tid] = __ldg(reinterpret_cast<const float4*>(a.norm_w) + f);
        }
    } else if (own_p == 0 && w_in_regs) {
#pragma unroll
        for (int r = 0; r < kWRegs; ++r) {
            const int i = tid + r * kGemvThreads;
            wreg[r] = i < a.K ? __ldg(a.norm_w + i) : 0.0f;   // model constant: no need to wait for the previous kernel
        }
    }
    if (L.ksplit > 1 || !FUSED) __syncthreads();    // batched: the staging loop below adds into s_sa4 from every warp, so the
                                                    // zeroes above must be in place first (one sequence: barriers follow anyway)
    if (L.ksplit > 1) cluster.barrier_arrive();     // "my s_d is zeroed": peers may add into it after their wait

    TZ_STAMP(1);
    if (a.use_pdl) pdl_wait();
    TZ_STAMP(2);
    if (FUSED && a.use_pdl) pdl_launch_dependents();   // one sequence: the next kernel's CTAs may come in and fetch their weights from here on

    float resid_v = 0.0f;                           // batch 1: fetched now so the epilogue does not wait on it
    if (FUSED && a.epilogue == TENZO_EPI_RESIDUAL && split == 0 && tid < 64)
        resid_v = __ldcg(a.resid + (size_t)seq0 * a.out_stride + unit * 64 + tid);

    auto own_prologue = [&](auto pieces_c) {
        constexpr int P = decltype(pieces_c)::value;      // pieces per thread
        // ---- RMSNorm + absmax(31) quantiser, recomputed identically by every CTA; owned elements (see above) --------
        const float4* x4 = reinterpret_cast<const float4*>(a.x + (size_t)seq0 * a.x_stride);
        float xv[4 * P];
#pragma unroll
        for (int j = 0; j < P; ++j) {
            const int f = tid + j * kGemvThreads;
            const float4 v = f < n_pieces ? __ldcg(x4 + f) : make_float4(0.f, 0.f, 0.f, 0.f);
            xv[4 * j] = v.x; xv[4 * j + 1] = v.y; xv[4 * j + 2] = v.z; xv[4 * j + 3] = v.w;
        }
        float m = 0.0f;
        if (a.do_norm) {
            // squares chain-major (element e in row e & 7, column e >> 3) in padded rows, 16-byte aligned and four banks
            // apart: the lane of chain c then reads four of its elements per load
            const int stride = (((a.K >> 3) + 3) & ~3) + 4;
#pragma unroll
            for (int j = 0; j < P; ++j) {
                const int f = tid + j * kGemvThreads;
                if (f < n_pieces) {
                    float* d = s_x + (4 * (f & 1)) * stride + (f >> 1);
#pragma unroll
                    for (int k = 0; k < 4; ++k) d[k * stride] = __fmul_rn(xv[4 * j + k], xv[4 * j + k]);
                }
            }
            __syncthreads();
            TZ_STAMP(8);
            if (tid < 8) {
                // eight elements requested while the previous eight are added (two registers sets of two loads)
                const float4* p = reinterpret_cast<const float4*>(s_x + tid * stride);
                const int n4 = a.K >> 5;                                  // 16-byte pieces per chain
                float sum = 0.0f;
                auto add4 = [&](const float4& v) {
                    sum = __fadd_rn(sum, v.x); sum = __fadd_rn(sum, v.y); sum = __fadd_rn(sum, v.z); sum = __fadd_rn(sum, v.w);
                };
                float4 a0 = p[0], a1 = n4 > 1 ? p[1] : make_float4(0.f, 0.f, 0.f, 0.f), b0, b1;
                int i = 0;
                for (; i + 4 <= n4; i += 4) {
                    b0 = p[i + 2]; b1 = p[i + 3];
                    add4(a0); add4(a1);
                    if (i + 6 <= n4) { a0 = p[i + 4]; a1 = p[i + 5]; } else if (i + 5 <= n4) { a0 = p[i + 4]; }
                    add4(b0); add4(b1);
                }
                for (; i < n4; ++i) add4(p[i]);                           // at most three pieces (read again: rare shapes)
                s_f[tid] = sum;
            }
            __syncthreads();
            float ss = s_f[0];
#pragma unroll
            for (int j = 1; j < 8; ++j) ss = __fadd_rn(ss, s_f[j]);     // the eight lanes left to right (common.cuh)
            TZ_STAMP(9);
            const float inv_rms = rms_inv(ss, a.K, a.eps);
#pragma unroll
            for (int r = 0; r < 4 * P; ++r) {
                float y = xv[r] * inv_rms;                              // x * inv_rms * w, left to right (:158)
                if (has_w) {
                    if constexpr (P == 2) {
                        y = y * wreg[r];
                    } else {                                                // parked before the wait (same thread, same slot)
                        const float* wp = reinterpret_cast<const float*>(s_w4 + (r >> 2) * kGemvThreads + tid);
                        if (tid + (r >> 2) * kGemvThreads < n_pieces) y = y * wp[r & 3];
                    }
                }
                xv[r] = y;
                m = fmaxf(m, fabsf(y));                                 // slots beyond K hold zeros
            }
        } else {
#pragma unroll
            for (int r = 0; r < 4 * P; ++r) m = fmaxf(m, fabsf(xv[r]));
        }
        TZ_STAMP(10);
        m = fmaxf(block_max_nonneg(m, s_f), 1e-6f); // TenzoEngine.cpp:28-32 (m: running maximum of |y| from 0)
        TZ_STAMP(11);
        const float to_q = 31.0f / m;               // :34
        if (tid == 0) s_inv[0] = m / 31.0f;         // :35
        const bool parity_out = a.a_out && blockIdx.x == 0;
        uint8_t* s_b8 = reinterpret_cast<uint8_t*>(s_b);
        int sa = 0;
#pragma unroll
        for (int j = 0; j < P; ++j) {
            const int f = tid + j * kGemvThreads, s = f >> 3, i = (f >> 1) & 3;     // element 4f + k: set, byte of its word
            if (f < n_pieces) {
                const bool mine = s >= s_begin && s < s_end;                        // this CTA's K range
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const int q = (int)roundf(xv[4 * j + k] * to_q);                // :41-42, half away from zero
                    // word (set, column c = 4 (f & 1) + k) holds its elements 8 i + c, i = 0..3; even columns carry the factor 4
                    if (mine) {
                        s_b8[(((s - s_begin) * 8 + 4 * (f & 1) + k) << 2) + i] = (uint8_t)(int8_t)((k & 1) ? q : 4 * q);
                        sa += q;
                    }
                    if (parity_out) a.a_out[(size_t)seq0 * a.K + 4 * f + k] = (int8_t)q;
                }
            }
        }
        sa = warp_sum_i(sa);
        if (lane == 0 && sa) atomicAdd(&s_sa4[0], 4 * sa);
        if (a.inv_out && blockIdx.x == 0 && tid == 0) a.inv_out[seq0] = m / 31.0f;
        TZ_STAMP(12);
    };
    if (own_p == 2) {
        own_prologue(std::integral_constant<int, 2>{});
    } else if (own_p == 4) {
        own_prologue(std::integral_constant<int, 4>{});
    } else if (FUSED) {
        // ---- the same for any other K: x staged in shared memory, two passes over it ----------------
        const float* x = a.x + (size_t)seq0 * a.x_stride;
        const bool vec = ((a.K & 3) == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0);
        if (vec) {
            for (int i = tid; i < (a.K >> 2); i += kGemvThreads)
                reinterpret_cast<float4*>(s_x)[i] = __ldcg(reinterpret_cast<const float4*>(x) + i);
        } else {
            for (int i = tid; i < a.K; i += kGemvThreads) s_x[i] = __ldcg(x + i);
        }
        __syncthreads();
        float m = 0.0f;
        if (a.do_norm) {
            const float ss = sumsq_reference_order(s_x, a.K, s_f);
            const float inv_rms = rms_inv(ss, a.K, a.eps);
            if (w_in_regs) {
#pragma unroll
                for (int r = 0; r < kWRegs; ++r) {
                    const int i = tid + r * kGemvThreads;
                    if (i < a.K) {
                        const float y = s_x[i] * inv_rms * wreg[r];   // x * inv_rms * w, left to right (:158)
                        s_x[i] = y;
                        m = fmaxf(m, fabsf(y));
                    }
                }
            } else {
                for (int i = tid; i < a.K; i += kGemvThreads) {
                    const float y = rms_apply(s_x[i], inv_rms, has_w ? a.norm_w : nullptr, i);
                    s_x[i] = y;
                    m = fmaxf(m, fabsf(y));
                }
            }
        } else {
            for (int i = tid; i < a.K; i += kGemvThreads) m = fmaxf(m, fabsf(s_x[i]));
        }
        m = fmaxf(block_max_nonneg(m, s_f), 1e-6f); // TenzoEngine.cpp:28-32 (m: running maximum of |y| from 0)
        const float to_q = 31.0f / m;               // :34
        if (tid == 0) s_inv[0] = m / 31.0f;         // :35
        // pack only this CTA's columns: one 32-bit fragment word per (set, t, even/odd)
        int sa = 0;
        for (int wd = tid; wd < n_cta_sets * 8; wd += kGemvThreads) {
            const int s = s_begin + (wd >> 3), tt = (wd >> 1) & 3, odd = wd & 1;
            uint32_t word = 0;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int col = 2 * (16 * s + 4 * i + tt) + odd;
                const int q = col < a.K ? (int)roundf(s_x[col] * to_q) : 0;   // :41-42, half away from zero
                sa += q;
                word |= (uint32_t)(uint8_t)(int8_t)(odd ? q : 4 * q) << (8 * i);
            }
            s_b[wd] = word;
        }
        sa = warp_sum_i(sa);
        if (lane == 0 && sa) atomicAdd(&s_sa4[0], 4 * sa);
        if ((a.a_out || a.inv_out) && blockIdx.x == 0) {                      // parity-check outputs
            for (int i = tid; i < a.K; i += kGemvThreads)
                if (a.a_out) a.a_out[(size_t)seq0 * a.K + i] = (int8_t)(int)roundf(s_x[i] * to_q);
            if (a.inv_out && tid == 0) a.inv_out[seq0] = m / 31.0f;
        }
    } else {
        // ---- stage this CTA's K range of the pre-quantised activations of SL sequences -----------
        for (int idx = tid; idx < n_cta_sets * SL * 2; idx += kGemvThreads) {
            const int half = idx & 1, n = (idx >> 1) % SL, sl = (idx >> 1) / SL;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (seq0 + n < a.batch)
                v = __ldcg(reinterpret_cast<const uint4*>(L.act_words + ((size_t)(seq0 + n) * L.nsets + s_begin + sl) * 8) + half);
            reinterpret_cast<uint4*>(s_b + ((size_t)sl * SL + n) * 8)[half] = v;
            int sa4 = dp4a_ss(0x01010101u, v.x, 0);     // even-column words already carry the factor 4
            sa4 = dp4a_ss(0x04040404u, v.y, sa4);
            sa4 = dp4a_ss(0x01010101u, v.z, sa4);
            sa4 = dp4a_ss(0x04040404u, v.w, sa4);
            if (sa4) atomicAdd(&s_sa4[n], sa4);
        }
        for (int n = tid; n < SL; n += kGemvThreads) s_inv[n] = seq0 + n < a.batch ? __ldcg(L.act_inv + seq0 + n) : 0.0f;
    }
    __syncthreads();
    TZ_STAMP(3);
    if (!FUSED && a.use_pdl) pdl_launch_dependents();

    // ---- main loop: weights from shared memory, four MMAs per set per 8 sequences -----------------
    int acc[NT][4][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[nt][j][e] = 0;
    // Per-lane cursors advance by one stride per set: no index arithmetic in the loop. Words past the
    // copied range (ragged K) are stale shared memory, but the activation bytes they meet are zero.
    const uint32_t* wt = s_wt + my_blk * n_cta_sets * 128 + (16 * wi + t4) * 8 + g;      // column pair 16*sl + 4*i + t4, byte 4g
    const uint32_t* bp = s_b + ((size_t)wi * SL + g) * 8 + t4 * 2;                        // B fragment words of sequence g
    const int wt_step = 16 * wb * 8, bp_step = wb * SL * 8;
    int next_wait = 0, chunk = 0;                                                         // first set of the next chunk to wait for
    bool timed_out = false;
    for (int u = 0, sl = wi; u < my_sets; ++u, sl += wb, wt += wt_step, bp += bp_step) {
        while (sl >= next_wait) {
            // one lane polls (operations on one mbarrier serialise); the warp barrier passes the
            // acquired visibility on to the other lanes
            if (lane == 0 && !mbar_wait_bounded(&s_bar[my_blk * kChunks + chunk], 0)) timed_out = true;
            __syncwarp();
            ++chunk;
            next_wait += sets_per_chunk;
        }
        const uint32_t W0 = wt[0], W1 = wt[32], W2 = wt[64], W3 = wt[96];
        // 4x4 byte transpose: T[j] = (W0.j, W1.j, W2.j, W3.j) = row pair 4g+j at this lane's four column pairs
        const uint32_t p0 = prmt(W0, W1, 0x5140u), p1 = prmt(W2, W3, 0x5140u);
        const uint32_t p2 = prmt(W0, W1, 0x7362u), p3 = prmt(W2, W3, 0x7362u);
        const uint32_t T[4] = {prmt(p0, p1, 0x5410u), prmt(p0, p1, 0x7632u), prmt(p2, p3, 0x5410u), prmt(p2, p3, 0x7632u)};
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            uint2 b = make_uint2(0, 0);
            if (nt * 8 + g < SL) b = *reinterpret_cast<const uint2*>(bp + nt * 64);
#pragma unroll
            for (int j = 0; j < 4; ++j)
                mma_u8s8(acc[nt][j], T[j] & 0x03030303u, T[j] & 0x30303030u, T[j] & 0x0C0C0C0Cu, T[j] & 0xC0C0C0C0u, b.x, b.y);
        }
    }
    if (timed_out) atomicExch(&g_tl1_timeouts, 1);
    TZ_STAMP(4);

    // ---- warps of a row block meet in shared memory ---------------------------------------------
    if (my_sets > 0) {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int n = nt * 8 + 2 * t4 + e;          // sequence (column of D) held in c[e] and c[2+e]
                if (n < SL) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        atomicAdd(&s_d[(my_blk * 64 + 4 * g + j) * SL + n], acc[nt][j][e]);            // x4
                        atomicAdd(&s_d[(my_blk * 64 + 32 + 4 * g + j) * SL + n], acc[nt][j][2 + e]);   // x64
                    }
                }
            }
    }
    __syncthreads();

    // ---- split-K meeting point: the cluster leader's shared memory -----------------------------
    if (L.ksplit > 1) {
        cluster.barrier_wait();                     // every peer has zeroed its s_d (arrive above)
        if (split != 0) {
            int* remote = cluster.map_shared_rank(s_d, 0);
            for (int i = tid; i < rows_cta * SL; i += kGemvThreads) {
                const int v = s_d[i];
                if (v) atomicAdd(remote + i, v);
            }
            for (int n = tid; n < SL; n += kGemvThreads) atomicAdd(remote + 128 * SL + n, s_sa4[n]);
        }
        cluster.sync();                             // all remote adds have landed in the leader
        if (split != 0) return;
    }

    TZ_STAMP(5);
    // ---- epilogue -----------------------------------------------------------------------------
    for (int idx = tid; idx < 64 * SL; idx += kGemvThreads) {
        const int r = idx / SL, n = idx % SL, seq = seq0 + n;
        if (seq >= a.batch) continue;
        const int sum_a = s_sa4[n] >> 2;
        const float inv_act = s_inv[n];
        float v[2];
#pragma unroll
        for (int bk = 0; bk < 2; ++bk) {
            if (bk >= nb_cta) break;
            const int blk = bk ? unit + L.units : unit;
            const int raw = s_d[(bk * 64 + r) * SL + n];
            const int accv = (r < 32 ? (raw >> 2) : (raw >> 6)) - sum_a;
            if (a.acc_out) a.acc_out[(size_t)seq * a.n_blocks * 64 + blk * 64 + r] = accv;
            v[bk] = (float)accv * (inv_act * seg_scale_for(a, blk));   // :1554, :118
        }
        const size_t o = (size_t)seq * a.out_stride + unit * 64 + r;
        if (a.epilogue == TENZO_EPI_STORE) {
            a.out[o] = v[0];
        } else if (a.epilogue == TENZO_EPI_RESIDUAL) {
            a.out[o] = (FUSED ? resid_v : __ldcg(a.resid + o)) + v[0];   // :1590
        } else {
            const float rl = fmaxf(0.0f, v[0]);
            a.out[o] = (rl * rl) * v[1];                                 // :1618-1619
        }
    }
    TZ_STAMP(6);
    TZ_TRACE_FLUSH;
}

// Cluster size along K: 1, 2, 4 or 8. Enough CTAs to put one on every SM, few enough sets per warp
// that a warp's loads are all in flight at once, a K range whose packed activations fit in shared
// memory, never more CTAs than sets.
static int pick_ksplit(int n_blocks, int K, int epilogue, int batch) {
    const int nsets = ((K >> 1) + 15) / 16;
    const int nb_cta = epilogue == TENZO_EPI_RELU2_GLU ? 2 : 1;
    const int units = n_blocks / nb_cta;
    int ks = 1;
    if (batch == 1) {
        // one CTA per row block, two resident per SM: weights (512 B per set per row block) + x must fit ~100 KB
        auto bytes = [&](int k) { return (size_t)((nsets + k - 1) / k + 1) * (512 * nb_cta + 32) + (size_t)K * 4 + 2048; };
        while (ks < 8 && ks * 2 <= nsets && (units * ks < 32 || bytes(ks) > 100 * 1024)) ks *= 2;
    } else {
        const int sl = batch <= 8 ? 8 : 32, seq_tiles = (batch + sl - 1) / sl;
        auto bytes = [&](int k) { return (size_t)((nsets + k - 1) / k + 1) * (512 * nb_cta + 32 * sl) + (size_t)sl * 520 + 1024; };
        while (ks < 8 && ks * 2 <= nsets && (units * ks * seq_tiles < 148 || bytes(ks) > 200 * 1024)) ks *= 2;
    }
    return ks;
}

// act_quant_kernel lives in norm_quant.cu
cudaError_t launch_act_quant(const float* x, const float* norm_w, int do_norm, float eps, int K, int batch, int x_stride,
                             uint32_t* words, float* inv, int8_t* a_out, int* sum_out, int use_pdl, cudaStream_t st);
// tcgen05 GEMM for 16 or more sequences (tl1_umma.cu)
bool tl1_umma_applicable(const tenzo_tl1_gemv_args& a);
int launch_tl1_umma(const tenzo_tl1_gemv_args& a, const int8_t* a8, const float* inv, const int* sum_a, cudaStream_t st);
int tl1_umma_take_timeouts();

template <int NT, bool FUSED>
static cudaError_t launch_gemv(const GemvLaunch& L, cudaStream_t st) {
    using Lay = GemvSmem<NT, FUSED>;
    const tenzo_tl1_gemv_args& a = L.a;
    const int sets_per_cta = (L.nsets + L.ksplit - 1) / L.ksplit + 1;
    const size_t smem = Lay::bytes(sets_per_cta, a.K, a.epilogue == TENZO_EPI_RELU2_GLU ? 2 : 1);
    if (smem > 220 * 1024) return cudaErrorInvalidValue;
    if (smem > 48 * 1024) {
        cudaError_t ea = cudaFuncSetAttribute(tl1_mma_kernel<NT, FUSED>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (ea != cudaSuccess) return ea;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(L.units * L.ksplit), (unsigned)((a.batch + Lay::SL - 1) / Lay::SL), 1);
    cfg.blockDim = dim3((FUSED ? kFusedWarps : kBatchedWarps) * 32, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    int n_attr = 0;
    if (L.ksplit > 1) {
        attr[n_attr].id = cudaLaunchAttributeClusterDimension;
        attr[n_attr].val.clusterDim.x = (unsigned)L.ksplit;
        attr[n_attr].val.clusterDim.y = 1;
        attr[n_attr].val.clusterDim.z = 1;
        ++n_attr;
    }
    if (a.use_pdl) {
        attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
        ++n_attr;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n_attr;
    return cudaLaunchKernelEx(&cfg, tl1_mma_kernel<NT, FUSED>, L);
}

}  // namespace tz

extern "C" int tenzo_cuda_tl1_gemv_ksplit(int n_blocks, int K, int epilogue) {
    if (n_blocks <= 0 || K <= 0) return 1;
    return tz::pick_ksplit(n_blocks, K, epilogue, 1);
}

namespace tz {
// Self-test of the give-up path of the bounded waits: barrier A is told to expect 32 bytes that nobody sends, so the wait
// on it (a short one: 2^8 polls) runs out, the kernel raises the same flag a real give-up raises and carries on; barrier
// B tracks the one 16-byte copy the kernel does issue and is waited for before the CTA's shared memory goes away. Nothing
// here can fault or hang: both waits are bounded, and the only memory touched is the kernel's own.
__global__ void __launch_bounds__(32) wait_expiry_selftest_kernel(const unsigned char* src16) {
    __shared__ __align__(16) unsigned char s_dst[16];
    __shared__ uint64_t s_bar[2];
    if (threadIdx.x == 0) {
        mbar_init(&s_bar[0], 1);
        mbar_init(&s_bar[1], 1);
        mbar_init_fence();
        mbar_expect_tx(&s_bar[0], 32);
        mbar_expect_tx(&s_bar[1], 16);
        bulk_g2s(s_dst, src16, 16, &s_bar[1]);
        bool done = false;
        for (int it = 0; it < (1 << 8) && !done; ++it) done = mbar_test(&s_bar[0], 0);
        if (!done) atomicExch(&g_tl1_timeouts, 1);
        mbar_wait_bounded(&s_bar[1], 0);
    }
}
}  // namespace tz

extern "C" int tenzo_cuda_selftest_wait_expiry(void* stream) {
    static unsigned char* src = nullptr;
    if (!src) {
        if (cudaMalloc((void**)&src, 256) != cudaSuccess) return (int)cudaErrorMemoryAllocation;
        cudaMemset(src, 0, 256);
    }
    tz::wait_expiry_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(src);
    const cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : (int)e;
}

extern "C" int tenzo_cuda_tl1_gemv_take_timeouts(void) {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, tz::g_tl1_timeouts, sizeof v) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(tz::g_tl1_timeouts, &zero, sizeof zero);
    const int u = tz::tl1_umma_take_timeouts();
    if (u < 0) return -1;
    return v | u;
}

extern "C" size_t tenzo_cuda_tl1_gemv_workspace_bytes(int batch, int K) {
    if (batch <= 1 || K <= 0) return 0;
    const size_t nsets = ((size_t)(K >> 1) + 15) / 16;
    // packed activations (words path) or the plain int8 matrix (tensor-core path), then inv[batch], then sum_a[batch]
    const size_t act = (size_t)batch * nsets * 32 > (size_t)batch * K ? (size_t)batch * nsets * 32 : (size_t)batch * K;
    return ((act + 15) & ~(size_t)15) + 2 * (size_t)batch * sizeof(float) + 64;
}

extern "C" int tenzo_cuda_tl1_gemv(const tenzo_tl1_gemv_args* args, void* stream) {
    using namespace tz;
    if (!args || !args->x || !args->w || !args->out) return -1;
    const tenzo_tl1_gemv_args& a = *args;
    if (a.n_blocks <= 0 || a.K <= 0 || (a.K & 1) || a.batch <= 0) return -1;
    if ((reinterpret_cast<uintptr_t>(a.w) & 15) != 0) return -1;   /* bulk copies start on 16-byte boundaries */
    if (a.epilogue < 0 || a.epilogue > 2) return -1;
    if (a.epilogue == TENZO_EPI_RESIDUAL && !a.resid) return -1;
    if (a.epilogue == TENZO_EPI_RELU2_GLU && (a.n_blocks & 1)) return -1;
    if (a.K > 16384) return -5;   /* same bound as the reference engine's scratch vectors (:1227) */
    if (a.batch > 1 && (!a.workspace || (reinterpret_cast<uintptr_t>(a.workspace) & 15) != 0)) return -1;
    cudaStream_t st = static_cast<cudaStream_t>(stream);

    GemvLaunch L;
    L.a = a;
    L.nsets = ((a.K >> 1) + 15) / 16;
    L.units = a.epilogue == TENZO_EPI_RELU2_GLU ? a.n_blocks / 2 : a.n_blocks;
    L.ksplit = pick_ksplit(a.n_blocks, a.K, a.epilogue, a.batch);
    L.act_words = nullptr;
    L.act_inv = nullptr;
    cudaError_t e;
    if (a.batch == 1) {
        e = launch_gemv<1, true>(L, st);
    } else {
        uint32_t* words = static_cast<uint32_t*>(a.workspace);
        const size_t act_bytes = (((size_t)a.batch * L.nsets * 32 > (size_t)a.batch * a.K ? (size_t)a.batch * L.nsets * 32 : (size_t)a.batch * a.K) + 15) & ~(size_t)15;
        float* inv = reinterpret_cast<float*>(static_cast<unsigned char*>(a.workspace) + act_bytes);
        if (tl1_umma_applicable(a)) {
            int8_t* a8 = static_cast<int8_t*>(a.workspace);
            int* sums = reinterpret_cast<int*>(inv + a.batch);
            e = launch_act_quant(a.x, a.norm_w, a.do_norm, a.eps, a.K, a.batch, a.x_stride, nullptr, inv, a8, sums, a.use_pdl, st);
            if (e != cudaSuccess) return (int)e;
            if (a.inv_out && (e = cudaMemcpyAsync(a.inv_out, inv, (size_t)a.batch * sizeof(float), cudaMemcpyDeviceToDevice, st)) != cudaSuccess) return (int)e;
            if (a.a_out && (e = cudaMemcpyAsync(a.a_out, a8, (size_t)a.batch * a.K, cudaMemcpyDeviceToDevice, st)) != cudaSuccess) return (int)e;
            return launch_tl1_umma(a, a8, inv, sums, st);
        }
        e = launch_act_quant(a.x, a.norm_w, a.do_norm, a.eps, a.K, a.batch, a.x_stride, words, inv, a.a_out, nullptr, a.use_pdl, st);
        if (e != cudaSuccess) return (int)e;
        if (a.inv_out) {
            e = cudaMemcpyAsync(a.inv_out, inv, (size_t)a.batch * sizeof(float), cudaMemcpyDeviceToDevice, st);
            if (e != cudaSuccess) return (int)e;
        }
        L.act_words = words;
        L.act_inv = inv;
        L.a.a_out = nullptr;
        L.a.inv_out = nullptr;
        e = a.batch <= 8 ? launch_gemv<1, false>(L, st) : launch_gemv<4, false>(L, st);
    }
    return e == cudaSuccess ? 0 : (int)e;
}

#ifdef TZ_TRACE
// Measurement builds only: copies up to max_records timeline records (16 words each) to `out`, resets the buffer and
// returns how many were copied.
extern "C" __attribute__((visibility("default"))) int tenzo_trace_gemv(unsigned long long* out, int max_records) {
    unsigned int n = 0;
    if (cudaDeviceSynchronize() != cudaSuccess) return -1;
    if (cudaMemcpyFromSymbol(&n, tz::g_trace_n, sizeof n) != cudaSuccess) return -1;
    if (n > 4096u) n = 4096u;
    if ((int)n > max_records) n = (unsigned)max_records;
    if (n && cudaMemcpyFromSymbol(out, tz::g_trace, (size_t)n * 16 * sizeof(unsigned long long)) != cudaSuccess) return -1;
    const unsigned int zero = 0;
    if (cudaMemcpyToSymbol(tz::g_trace_n, &zero, sizeof zero) != cudaSuccess) return -1;
    return (int)n;
}
#endif
