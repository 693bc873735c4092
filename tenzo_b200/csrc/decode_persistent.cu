// Single-sequence decode step as one persistent cooperative kernel: embedding, every layer, final norm, LM head and
// greedy argmax of one token in ONE launch, one CTA per SM.
//
// What it replaces in the reference CPU engine (src/runtime/TenzoEngine.cpp): embedding_lookup (:1299-1315),
// forward_layer_raw (:1538-1632: rms_norm_raw, build_lut, compute_from_lut and the fused q|k|v and gate|up loops,
// FusedKVCache::forward_attention_raw, squared-ReLU GLU, residuals), compute_logits' int8 branch (:1661-1719), the
// greedy branch of sample_top_k_top_p (:1745-1755) and the sequencing of prefill_token / generate_step (:1809-1838).
//
// Why one kernel. A decoded token is a chain of ~150 dependent matrix-vector products of 1.6-8.8 MB each. As separate
// launches each costs several microseconds of launch, prologue and drain for bytes that HBM delivers in well under
// one. Here the chain's hand-offs are grid-wide barriers (~1.3 us) and the weights never wait for them:
//   * Every CTA owns a fixed, contiguous 1/grid share of every weight matrix. The TL1 layout [N/64][K/2][32 B] is a
//     sequence of 512-byte units (row block b, 16 column pairs s) when K is a multiple of 32, so an equal split of the
//     units is an equal split of the bytes with nothing to repack. A share may begin and end inside a row block: the
//     partial dot products of a (row block, CTA) pair are exact integers and meet in a global int32 accumulator
//     through red.add - order-free, hence bit-identical to any other evaluation.
//   * A dedicated producer warp streams the CTA's shares of ALL matrices of ALL layers, then its rows of the LM head,
//     through a ring of 16 KB shared-memory stages with 1-D bulk copies (TMA) and full/empty mbarriers. It runs ahead
//     of the phases by the size of the ring (about one layer at the BitNet-2B shape), so HBM keeps streaming while the
//     consumers sit in the dependent chain (barrier, RMS sum in the reference's order, quantiser).
//   * Nothing but integers and the attention output crosses CTAs. Every CTA keeps the residual stream in its own shared
//     memory and applies each epilogue itself when it reads the accumulators: h1 = x + float(acc)*scale, the squared-
//     ReLU GLU, x = h1 + float(acc)*scale - the same expressions, in the same order, as the per-operator kernels
//     (tl1_gemv.cu) and the reference (:1554, :1590, :1618-1619, :1628). RMSNorm + absmax quantiser are recomputed by
//     every CTA from identical inputs, so every CTA holds identical int8 activations.
//   * Attention for the one sequence runs on n_q CTAs (one query head each) with the arithmetic of attention.cu.
//   * The accumulators are left zeroed for the next launch: each is cleared by the grid after the barrier that follows
//     its last reader.
// Every wait (mbarrier or grid barrier) is bounded; a give-up raises the status word, makes every later wait of the
// CTA return at once, and the launch ends with a result the host discards.
#include <cuda_runtime.h>

#include "attn_common.cuh"
#include "common.cuh"
#include "decode_persistent.h"

namespace tz {

constexpr int kPcWarps = 15;                       // consumer warps: with the producer warp 16 in all, four per scheduler, 128 registers each
constexpr int kPcThreads = kPcWarps * 32;          // consumer threads
constexpr int kPcBlock = kPcThreads + 32;          // + the producer warp
constexpr int kPcStageBytes = 32768;                // a bulk copy costs about the same whatever its size: few, large stages
constexpr int kPcUnitsPerStage = kPcStageBytes / 512;
constexpr int kPcMaxStages = 6;
constexpr int kPcMaxSlots = 8;                     // row blocks one CTA's share of a matrix may touch
constexpr int kPcW4 = 4;                           // float4 norm-weight loads a thread holds between a phase's start and its norm pass (K <= 7680)
constexpr int kPcAttnFixed = 2048 + 2 * kChunk * kHd;   // attention scratch in front of the scores

// ---- small helpers ---------------------------------------------------------------------------------------------------
__device__ __forceinline__ void pc_cbar() { named_barrier_sync(1, kPcThreads); }          // the consumer threads only
__device__ __forceinline__ unsigned pc_ld_acquire(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void pc_mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ unsigned long long pc_gtime() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void pc_mma_u8s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Optional timeline for experiments (-DTZ_PC_TRACE): one thread of the first CTA stores GPU-timer readings of one layer's
// gate|up phase into phase_ns[8..]; compiled out of the library build.
#ifdef TZ_PC_TRACE
__device__ unsigned long long* g_pc_trace = nullptr;
#define PC_TR(i) do { if (g_pc_trace && threadIdx.x == 0 && blockIdx.x == 0) g_pc_trace[i] = pc_gtime(); } while (0)
#else
#define PC_TR(i) do {} while (0)
#endif

__device__ __forceinline__ void pc_fail(const PcParams& p, volatile int* s_abort, int code) {
    *s_abort = 1;
    atomicCAS(p.status, 0, code);
    if (p.host_status) {
        *reinterpret_cast<volatile int*>(p.host_status) = code;
        __threadfence_system();
    }
}

// Bounded wait on an mbarrier phase that also gives up as soon as the CTA has aborted.
__device__ __forceinline__ bool pc_wait(uint64_t* bar, unsigned parity, volatile int* s_abort) {
    const uint32_t addr = smem_addr(bar);
    for (int it = 0; it < (1 << 20); ++it) {
        uint32_t done;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(done) : "r"(addr), "r"(parity) : "memory");
        if (done) return true;
        if ((it & 63) == 63 && *s_abort) return false;
    }
    return false;
}

// The producer's wait for a free stage: it may take a whole phase, so the thread sleeps between looks instead of
// competing with the consumer warps of its scheduler for issue slots.
__device__ __forceinline__ bool pc_wait_sleepy(uint64_t* bar, unsigned parity, volatile int* s_abort) {
    for (int it = 0; it < (1 << 22); ++it) {
        if (mbar_test(bar, parity)) return true;
        if ((it & 63) == 63 && *s_abort) return false;
        __nanosleep(128);
    }
    return false;
}

// Grid-wide barrier among the consumer threads of all CTAs: arrivals are counted in one global word that only grows
// (the host passes its value at launch), thread 0 polls it. Release/acquire as in a cooperative-groups grid sync.
__device__ __noinline__ unsigned pc_grid_barrier(const PcParams& p, unsigned arrivals, int tid, volatile int* s_abort) {
    arrivals += gridDim.x;
    pc_cbar();
    if (tid == 0) {
        __threadfence();
        atomicAdd(p.bar_counter, 1u);
        const unsigned target = p.bar_base + arrivals;
        if (!*s_abort) {
            bool ok = false;
            for (int it = 0; it < (1 << 21); ++it) {
                if ((int)(pc_ld_acquire(p.bar_counter) - target) >= 0) { ok = true; break; }
                if ((it & 1023) == 1023 && *reinterpret_cast<volatile int*>(p.status) != 0) break;   // another CTA gave up
            }
            if (!ok) pc_fail(p, s_abort, PC_ERR_BARRIER);
        }
        __threadfence();
    }
    pc_cbar();
    return arrivals;
}

// Units per ring stage for a share of n units: as few copies as fit the stages, of even size (a bulk copy costs about
// the same whatever its size, so a 32 + 1 split would pay twice for 33 units).
__device__ __forceinline__ int pc_chunk_units(int n) {
    const int chunks = (n + kPcUnitsPerStage - 1) / kPcUnitsPerStage;
    return chunks > 0 ? (n + chunks - 1) / chunks : kPcUnitsPerStage;
}

// This CTA's share [u0, u1) of `total` units.
__device__ __forceinline__ void pc_share(unsigned total, int& u0, int& u1) {     // total * gridDim.x < 2^32 (checked by pc_plan)
    u0 = (int)((total * blockIdx.x) / gridDim.x);
    u1 = (int)((total * (blockIdx.x + 1u)) / gridDim.x);
}

__device__ __forceinline__ void pc_zero_slice(int32_t* buf, int n, int tid) {
    const int per = (n + (int)gridDim.x - 1) / (int)gridDim.x;
    const int i0 = (int)blockIdx.x * per, i1 = min(n, i0 + per);
#pragma unroll 1
    for (int i = i0 + tid; i < i1; i += kPcThreads) buf[i] = 0;
}

// Element-wise pass over an int32 accumulator vector in global memory (and up to one more at `second`), n a multiple of
// 4: every thread first requests all of its 16-byte pieces of a batch, then consumes them - the L2 round trip is paid
// once per batch, not once per element (shared-memory stores in between would otherwise order the loads).
template <bool TWO, typename F>
__device__ __forceinline__ void pc_for_acc(const int32_t* first, const int32_t* second, int n, int tid, F&& f) {
    constexpr int B = 4;
    const int n4 = n >> 2;
#pragma unroll 1
    for (int base = 0; base < n4; base += B * kPcThreads) {
        int4 va[B], vb[B];
#pragma unroll
        for (int r = 0; r < B; ++r) {
            const int i = base + r * kPcThreads + tid;
            va[r] = make_int4(0, 0, 0, 0);
            vb[r] = make_int4(0, 0, 0, 0);
            if (i < n4) {
                va[r] = __ldcg(reinterpret_cast<const int4*>(first) + i);
                if (TWO && second != first) vb[r] = __ldcg(reinterpret_cast<const int4*>(second) + i);
            }
        }
#pragma unroll
        for (int r = 0; r < B; ++r) {
            const int i = base + r * kPcThreads + tid;
            if (i < n4) {
                f(4 * i, va[r].x, vb[r].x);
                f(4 * i + 1, va[r].y, vb[r].y);
                f(4 * i + 2, va[r].z, vb[r].z);
                f(4 * i + 3, va[r].w, vb[r].w);
            }
        }
    }
}

// Ask L2 for the norm weights of the phase after this one (they are streamed out of L2 by every token's 852 MB of
// weights); one 128-byte line per thread. No registers, no shared memory, nothing to wait for.
__device__ __forceinline__ void pc_prefetch_norm(const float* w, int K, int tid) {
    if (!w) return;
#pragma unroll 1
    for (int i = tid * 32; i < K; i += kPcThreads * 32) asm volatile("prefetch.global.L2 [%0];" ::"l"(w + i));
}

// Where element i of a K-vector lives in the chain-major copy of its squares: the reference's sum of squares
// (common.cuh:sumsq_reference_order) runs eight chains, chain j over elements j, j+8, ...; keeping each chain contiguous
// (K/8 + 4 floats apart: 16-byte aligned, and the chains start four banks apart) lets a chain be read four elements
// per load, far enough ahead that the loop runs at the latency of the dependent add.
__device__ __forceinline__ int pc_sq_stride(int K) { return (K >> 3) + 4; }
__device__ __forceinline__ int pc_sq_index(int i, int stride) { return (i & 7) * stride + (i >> 3); }

// Sum of squares in the reference's order from the chain-major squares (each already rounded: product and sum are
// separate roundings in the reference, :149-153); one barrier. K is a multiple of 32.
__device__ __forceinline__ float pc_sumsq(const float* sq, int K, float* red, int tid) {
#ifdef TZ_PC_TRACE
    const long long c0 = clock64();
#endif
    if (tid < 8) red[tid] = sequential_sum(sq + tid * pc_sq_stride(K), K >> 3);
#ifdef TZ_PC_TRACE
    if (g_pc_trace && threadIdx.x == 0 && blockIdx.x == 0) g_pc_trace[40] = (unsigned long long)(clock64() - c0);
#endif
    pc_cbar();
    float t = red[0];
#pragma unroll
    for (int j = 1; j < 8; ++j) t = __fadd_rn(t, red[j]);
    return t;
}

// Maximum over the consumer threads, identical bits in every thread; one barrier. `slots` holds kPcWarps floats.
__device__ __forceinline__ float pc_block_max(float v, float* slots, int tid) {
    v = warp_max(v);
    if ((tid & 31) == 0) slots[tid >> 5] = v;
    pc_cbar();
    float t = slots[0];
#pragma unroll
    for (int i = 1; i < kPcWarps; ++i) t = fmaxf(t, slots[i]);
    return t;
}

// RMSNorm + absmax(31) quantiser of `src` (K floats in shared memory, complete and visible, their squares in `sq`), as
// build_lut and rms_norm_raw do (:27-42, :148-166): y = src*inv_rms*w into `y` (may alias src), the int8 activations as
// mma B-fragment words in s_b ([K/32 sets][4 t][even|odd] words, even columns pre-multiplied by 4, see tl1_gemv.cu) and
// the sum of the 32 activations of every set in s_suma. Returns m/31. Ends with a barrier: s_b and s_suma are complete.
// floor_m / qmax select the two quantisers of the path: 1e-6 and 31 here, 1e-8 and 127 in front of the LM head (then the
// caller rounds y itself and s_b is not written).
__device__ __forceinline__ float pc_norm_absmax(const float* src, const float* sq, float* y, const float* norm_w, int K, float eps, float* red,
                                                int tid) {
    // the norm weights are requested first and used after the sum of squares
    float4 w4[kPcW4];
    const int n4 = K >> 2;
    const bool w_regs = norm_w && n4 <= kPcW4 * kPcThreads;
    if (w_regs) {
#pragma unroll
        for (int r = 0; r < kPcW4; ++r) {
            const int v = tid + r * kPcThreads;
            w4[r] = v < n4 ? __ldg(reinterpret_cast<const float4*>(norm_w) + v) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    PC_TR(1);
    const float ss = pc_sumsq(sq, K, red, tid);
    PC_TR(2);
    const float inv_rms = rms_inv(ss, K, eps);
    float m = 0.0f;
    if (w_regs) {
#pragma unroll
        for (int r = 0; r < kPcW4; ++r) {
            const int v = tid + r * kPcThreads;
            if (v < n4) {
                float4 x = reinterpret_cast<const float4*>(src)[v];
                x.x = x.x * inv_rms * w4[r].x;                    // x * inv_rms * w, left to right (:158)
                x.y = x.y * inv_rms * w4[r].y;
                x.z = x.z * inv_rms * w4[r].z;
                x.w = x.w * inv_rms * w4[r].w;
                reinterpret_cast<float4*>(y)[v] = x;
                m = fmaxf(fmaxf(m, fmaxf(fabsf(x.x), fabsf(x.y))), fmaxf(fabsf(x.z), fabsf(x.w)));
            }
        }
    } else {
#pragma unroll 1
        for (int i = tid; i < K; i += kPcThreads) {
            const float v = rms_apply(src[i], inv_rms, norm_w, i);
            y[i] = v;
            m = fmaxf(m, fabsf(v));
        }
    }
    PC_TR(3);
    const float mm = pc_block_max(m, red + 16, tid);                        // the barrier also completes y
    PC_TR(4);
    return mm;
}

__device__ __forceinline__ float pc_quantise(const float* src, const float* sq, float* y, const float* norm_w, int K, float eps,
                                             uint32_t* s_b, int* s_suma, float* red, int tid) {
    const float m = fmaxf(pc_norm_absmax(src, sq, y, norm_w, K, eps, red, tid), 1e-6f);   // :28-32
    const float to_q = 31.0f / m;                                 // :34
    const int n_words = (K >> 5) * 8;
#pragma unroll 1
    for (int wd = tid; wd < n_words; wd += kPcThreads) {
        // lanes of this warp still in the loop: the first `left` (a multiple of eight, as n_words is)
        const int left = n_words - (wd - (tid & 31));
        const unsigned mask = left >= 32 ? 0xffffffffu : ((1u << left) - 1u);
        const int s = wd >> 3, tt = (wd >> 1) & 3, odd = wd & 1;
        uint32_t word = 0;
        int sa = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int col = 2 * (16 * s + 4 * i + tt) + odd;
            const int q = (int)roundf(y[col] * to_q);             // :41-42, half away from zero
            sa += q;
            word |= (uint32_t)(uint8_t)(int8_t)(odd ? q : 4 * q) << (8 * i);
        }
        s_b[wd] = word;
        sa += __shfl_xor_sync(mask, sa, 1);
        sa += __shfl_xor_sync(mask, sa, 2);
        sa += __shfl_xor_sync(mask, sa, 4);
        if ((wd & 7) == 0) s_suma[s] = sa;
    }
    PC_TR(5);
    pc_cbar();
    PC_TR(6);
    return m / 31.0f;                                             // :35
}

struct PcRing {
    uint64_t* full;
    uint64_t* empty;
    unsigned char* base;
    int n_stages;
};

// One matrix-vector product phase, consumer side: this CTA's share of the matrix ([n_blocks][nsets] units of 512 bytes)
// arrives through the ring; warps take the units of a stage round-robin (the main loop of tl1_gemv.cu: 4x4 byte
// transpose, masks as u8 A fragments, four mma.m16n8k32 per unit), partial sums of a row block meet in shared-memory
// atomics, and the CTA adds (sum code*a - sum a over its own columns) = sum w*a over its columns into acc_out.
// s_d [slots][64] and s_range [slots] are zero on entry and are left zero.
__device__ __forceinline__ void pc_flush(int (&acc)[4][4], int& sa, int slot, int* s_d, int* s_range, int lane) {
    const int g = lane >> 2, t4 = lane & 3;
    if (slot >= 0) {
        if (t4 == 0) {                         // column 0 of D (the one sequence) lives in the lanes with t4 == 0
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                atomicAdd(&s_d[slot * 64 + 4 * g + j], acc[j][0]);          // x4
                atomicAdd(&s_d[slot * 64 + 32 + 4 * g + j], acc[j][2]);     // x64
            }
        }
        if (lane == 0 && sa) atomicAdd(&s_range[slot], sa);                 // sum of the activations over this warp's columns
    }
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[j][e] = 0;
    sa = 0;
}

__device__ __forceinline__ void pc_matvec(const PcRing& ring, unsigned& chunk, int n_blocks, int nsets, const uint32_t* s_b, int* s_d,
                                          const int* s_suma, int* s_range, int32_t* acc_out, int tid, volatile int* s_abort, bool& copy_failed) {
    const int warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
    int u0, u1;
    pc_share((unsigned)(n_blocks * nsets), u0, u1);
    const int b_first = u0 / nsets;
    const int nslots = u1 > u0 ? (u1 - 1) / nsets - b_first + 1 : 0;
    int acc[4][4];
    int sa = 0, cur_slot = -1;
    pc_flush(acc, sa, -1, s_d, s_range, lane);
    PC_TR(7);
    int b = b_first, b_lim = (b_first + 1) * nsets;
    const int per_chunk = pc_chunk_units(u1 - u0);
    int trc = 8;
#pragma unroll 1
    for (int cu0 = u0; cu0 < u1; cu0 += per_chunk) {
        const int cu1 = min(cu0 + per_chunk, u1);
        const int stage = (int)(chunk % (unsigned)ring.n_stages);
        const unsigned par = (chunk / (unsigned)ring.n_stages) & 1u;
        PC_TR(trc); ++trc;
        if (lane == 0 && !pc_wait(&ring.full[stage], par, s_abort)) copy_failed = true;
        __syncwarp();
        PC_TR(trc); ++trc;
        const uint32_t* st = reinterpret_cast<const uint32_t*>(ring.base + (size_t)stage * kPcStageBytes);
#pragma unroll 1
        for (int u = cu0 + warp; u < cu1; u += kPcWarps) {
            while (u >= b_lim) { ++b; b_lim += nsets; }
            const int s = u - (b_lim - nsets), slot = b - b_first;
            if (slot != cur_slot) {
                pc_flush(acc, sa, cur_slot, s_d, s_range, lane);
                cur_slot = slot;
            }
            const uint32_t* wt = st + (u - cu0) * 128 + t4 * 8 + g;     // column pair 4*i + t4 of the unit, byte 4g
            const uint32_t W0 = wt[0], W1 = wt[32], W2 = wt[64], W3 = wt[96];
            sa += s_suma[s];
            const uint32_t p0 = prmt(W0, W1, 0x5140u), p1 = prmt(W2, W3, 0x5140u);
            const uint32_t p2 = prmt(W0, W1, 0x7362u), p3 = prmt(W2, W3, 0x7362u);
            const uint32_t T[4] = {prmt(p0, p1, 0x5410u), prmt(p0, p1, 0x7632u), prmt(p2, p3, 0x5410u), prmt(p2, p3, 0x7632u)};
            uint2 bb = make_uint2(0, 0);
            if (g == 0) bb = *reinterpret_cast<const uint2*>(s_b + s * 8 + t4 * 2);
#pragma unroll
            for (int j = 0; j < 4; ++j)
                pc_mma_u8s8(acc[j], T[j] & 0x03030303u, T[j] & 0x30303030u, T[j] & 0x0C0C0C0Cu, T[j] & 0xC0C0C0C0u, bb.x, bb.y);
        }
        PC_TR(trc); ++trc;
        __syncwarp();
        if (lane == 0) pc_mbar_arrive(&ring.empty[stage]);
        ++chunk;
    }
    PC_TR(28);
    pc_flush(acc, sa, cur_slot, s_d, s_range, lane);
    PC_TR(29);
    pc_cbar();
    PC_TR(30);
    if (tid < nslots * 64) {
        const int slot = tid >> 6, r = tid & 63;
        const int raw = s_d[tid];
        s_d[tid] = 0;
        const int part = (r < 32 ? (raw >> 2) : (raw >> 6)) - s_range[slot];
        atomicAdd(acc_out + (size_t)(b_first + slot) * 64 + r, part);
    }
    pc_cbar();                                 // every reader of s_range is done
    if (tid < kPcMaxSlots) s_range[tid] = 0;
    PC_TR(31);
}

// Producer side of the same share: one bulk copy per stage, in the order the consumers will ask for them.
struct PcProducer {
    const PcRing& ring;
    volatile int* s_abort;
    unsigned chunk = 0;
    bool stopped = false;
    __device__ PcProducer(const PcRing& r, volatile int* a) : ring(r), s_abort(a) {}
    __device__ __forceinline__ void issue(const void* src, unsigned bytes) {
        if (stopped) return;
        const int stage = (int)(chunk % (unsigned)ring.n_stages);
        const unsigned round = chunk / (unsigned)ring.n_stages;
        if (round > 0 && !pc_wait_sleepy(&ring.empty[stage], (round - 1) & 1u, s_abort)) { stopped = true; return; }
        mbar_expect_tx(&ring.full[stage], bytes);
        bulk_g2s(ring.base + (size_t)stage * kPcStageBytes, src, bytes, &ring.full[stage]);
        ++chunk;
    }
    __device__ __forceinline__ void matrix(const uint8_t* w, int n_blocks, int nsets) {
        int u0, u1;
        pc_share((unsigned)(n_blocks * nsets), u0, u1);
        const int per_chunk = pc_chunk_units(u1 - u0);
#pragma unroll 1
        for (int cu0 = u0; cu0 < u1; cu0 += per_chunk) {
            const int cu1 = min(cu0 + per_chunk, u1);
            issue(w + (size_t)cu0 * 512, (unsigned)(cu1 - cu0) * 512u);
        }
    }
};

// ---- attention for one query head (the arithmetic of attn_kernel<1, false, false> in attention.cu) ---------------------
// Not inlined: its own register allocation, and one copy of its code. `state` carries the use counts of the two V
// buffers' barriers in (x, y) and a copy-failure flag in z; the updated value is returned.
__device__ __noinline__ uint3 pc_attention_head(const PcParams& p, const PcLayer& ly, int layer, int hq, int pos, float inv_q, bool last_layer,
                                                unsigned char* scratch, uint64_t* vbar, uint3 state, int tid, volatile int* s_abort) {
    unsigned vuse[2] = {state.x, state.y};
    bool copy_failed = state.z != 0;
    float* s_q = reinterpret_cast<float*>(scratch);            // [128] rotated query
    float* s_new = s_q + kHd;                                   // [2][128] rotated k, v of the new token
    float* s_red = s_new + 2 * kHd;                             // [16] per-warp maxima
    float* s_stat = s_red + 16;                                 // max, 1/sum, new-row scales (k, v)
    int8_t* s_new8 = reinterpret_cast<int8_t*>(scratch + 1664); // [2][128] quantised new k, v
    unsigned char* s_v = scratch + 2048;                        // [2][kChunk][128] V rows as in memory
    float* s_sc = reinterpret_cast<float*>(scratch + kPcAttnFixed);   // [T] scores, then e_t, then weights
    const int lane = tid & 31, warp = tid >> 5;
    const int T = pos + 1, n_chunks = (T + kChunk - 1) / kChunk;
    const int G = p.n_q / p.n_kv, kvh = hq / G;
    const bool stores_new_row = (hq % G) == 0;
    const size_t row_base = ((size_t)layer * p.n_kv + kvh) * p.max_seq;       // :509-510
    int8_t* ck = p.cache_k + row_base * kHd;
    int8_t* cv = p.cache_v + row_base * kHd;
    float* sk = p.scale_k + row_base;
    float* sv = p.scale_v + row_base;
    const float* cs = p.rope_cos + (size_t)pos * (kHd / 2);
    const float* sn = p.rope_sin + (size_t)pos * (kHd / 2);
    const int tp = (T + 3) & ~3;

    // this thread's first key row and its scales are requested before anything else
    uint4 cur[8];
    float pre_ks = 0.0f, pre_vs = 0.0f;
    const bool pre_ok = tid < T && tid != pos;
    if (pre_ok) {
#pragma unroll
        for (int c = 0; c < 8; ++c) cur[c] = ld_cg_u4(reinterpret_cast<const uint4*>(ck + (size_t)tid * kHd) + c);
        pre_ks = __ldcg(sk + tid);
        pre_vs = __ldcg(sv + tid);
    }
    auto issue_v = [&](int c) {
        const int t0 = c * kChunk, nk = min(kChunk, T - t0);
        mbar_expect_tx(&vbar[c & 1], (unsigned)nk * kHd);
        bulk_g2s(s_v + (size_t)(c & 1) * kChunk * kHd, cv + (size_t)t0 * kHd, (unsigned)nk * kHd, &vbar[c & 1]);
    };
    if (tid == 0) {
        issue_v(0);
        if (n_chunks > 1) issue_v(1);
    }

    // q, k, v of this head from the accumulators: float(acc) * (m/31 * weight scale), the GEMV epilogue (:1554)
    const int32_t* aq = p.acc;
    if (tid < kHd / 2) {
        const float sc = inv_q * ly.s_q;
        const float x0 = (float)__ldcg(aq + hq * kHd + tid) * sc, x1 = (float)__ldcg(aq + hq * kHd + tid + kHd / 2) * sc;
        float r0, r1;
        rope_pair(x0, x1, cs, sn, tid, r0, r1);
        s_q[tid] = r0;
        s_q[tid + kHd / 2] = r1;
        if (last_layer) { p.b_qkv[hq * kHd + tid] = x0; p.b_qkv[hq * kHd + tid + kHd / 2] = x1; }
    } else if (tid < kHd) {
        const int i = tid - kHd / 2;
        const float sc = inv_q * ly.s_k;
        const float x0 = (float)__ldcg(aq + p.qd + kvh * kHd + i) * sc, x1 = (float)__ldcg(aq + p.qd + kvh * kHd + i + kHd / 2) * sc;
        float r0, r1;
        rope_pair(x0, x1, cs, sn, i, r0, r1);
        s_new[i] = r0;
        s_new[i + kHd / 2] = r1;
        if (last_layer && stores_new_row) { p.b_qkv[p.qd + kvh * kHd + i] = x0; p.b_qkv[p.qd + kvh * kHd + i + kHd / 2] = x1; }
    } else if (tid < kHd + kHd / 2) {
        const int i = tid - kHd;
        const float sc = inv_q * ly.s_v;
        const float x0 = (float)__ldcg(aq + p.qd + p.kvd + kvh * kHd + i) * sc;
        const float x1 = (float)__ldcg(aq + p.qd + p.kvd + kvh * kHd + i + kHd / 2) * sc;
        s_new[kHd + i] = x0;
        s_new[kHd + i + kHd / 2] = x1;
        if (last_layer && stores_new_row) { p.b_qkv[p.qd + p.kvd + kvh * kHd + i] = x0; p.b_qkv[p.qd + p.kvd + kvh * kHd + i + kHd / 2] = x1; }
    }
    pc_cbar();
    if (warp < 2) {                                  // warp 0: key row, warp 1: value row (:507-533)
        const float* src = s_new + warp * kHd;
        float amax = 1e-8f;
#pragma unroll
        for (int j = 0; j < 4; ++j) amax = fmaxf(amax, fabsf(src[lane * 4 + j]));
        amax = warp_max(amax);
        const float s = amax / 127.0f;               // :522
        const float inv = 1.0f / s;                  // :527
        uint32_t packed = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float qf = fminf(fmaxf(roundf(src[lane * 4 + j] * inv), -128.0f), 127.0f);   // :530
            packed |= ((uint32_t)(uint8_t)(int8_t)(int)qf) << (8 * j);
        }
        reinterpret_cast<uint32_t*>(s_new8 + warp * kHd)[lane] = packed;
        if (lane == 0) s_stat[2 + warp] = s;
        if (stores_new_row) {
            int8_t* dst = (warp == 0 ? ck : cv) + (size_t)pos * kHd;
            reinterpret_cast<uint32_t*>(dst)[lane] = packed;
            if (lane == 0) (warp == 0 ? sk : sv)[pos] = s;
        }
    }
    pc_cbar();

    // scores (:678-694): one key per thread, eight FMA lanes over d, lanes added left to right, times (s_k / sqrt(d))
    const float sm_scale = 1.0f / sqrtf((float)kHd);   // :660
    float tmax = -1e30f;                               // :670
    auto load_row = [&](int t, uint4 (&r)[8]) {
        if (t == pos) {
#pragma unroll
            for (int c = 0; c < 8; ++c) r[c] = reinterpret_cast<const uint4*>(s_new8)[c];
        } else {
#pragma unroll
            for (int c = 0; c < 8; ++c) r[c] = ld_cg_u4(reinterpret_cast<const uint4*>(ck + (size_t)t * kHd) + c);
        }
    };
#pragma unroll 1
    for (int t = tid; t < T; t += kPcThreads) {
        if (!(pre_ok && t == tid)) load_row(t, cur);
        const float ksc = t == pos ? s_stat[2] : ((pre_ok && t == tid) ? pre_ks : __ldcg(sk + t));
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.0f;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            const uint32_t w[4] = {cur[c].x ^ 0x80808080u, cur[c].y ^ 0x80808080u, cur[c].z ^ 0x80808080u, cur[c].w ^ 0x80808080u};
            const float4* q4 = reinterpret_cast<const float4*>(s_q + c * 16);
            const float4 qa = q4[0], qb = q4[1], qc = q4[2], qd = q4[3];
            const float qv[16] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w, qc.x, qc.y, qc.z, qc.w, qd.x, qd.y, qd.z, qd.w};
#pragma unroll
            for (int e = 0; e < 16; ++e) acc[e & 7] = __fmaf_rn(qv[e], s8_to_f(w[e >> 2], e & 3), acc[e & 7]);
        }
        const float ks = ksc * sm_scale;
        const float dot = (acc[0] + acc[1] + acc[2] + acc[3] + acc[4] + acc[5] + acc[6] + acc[7]) * ks;   // :691
        s_sc[t] = dot;
        tmax = fmaxf(tmax, dot);
    }
    const float mx = pc_block_max(tmax, s_red, tid);
    if (tid == 0) s_stat[0] = mx;
    pc_cbar();
    exp_in_place<1>(s_sc, T, tp, s_stat, tid, kPcThreads);        // e_t = expf(score - max) (:826)
    pc_cbar();
    if (tid == 0) s_stat[1] = 1.0f / sequential_sum(s_sc, T);     // :824-830
    pc_cbar();
    {
        const float inv_sum = s_stat[1];
#pragma unroll 1
        for (int t = tid; t < T; t += kPcThreads) {
            const float vs = t == pos ? s_stat[3] : ((pre_ok && t == tid) ? pre_vs : __ldcg(sv + t));
            s_sc[t] = (s_sc[t] * inv_sum) * vs;                   // p_t * s_v[t] (:830, :844)
        }
    }
    pc_cbar();

    // output: thread d owns dim d and walks t in order (:842-851)
    float o[1] = {0.0f};
#pragma unroll 1
    for (int c = 0; c < n_chunks; ++c) {
        const int t0 = c * kChunk, nkeys = min(kChunk, T - t0);
        unsigned char* vb = s_v + (size_t)(c & 1) * kChunk * kHd;
        if (lane == 0 && !pc_wait(&vbar[c & 1], vuse[c & 1] & 1u, s_abort)) copy_failed = true;
        vuse[c & 1] += 1;
        __syncwarp();
        if (pos >= t0 && pos < t0 + nkeys) {                      // the new token's row is not in the cache copy: patch it in
            pc_cbar();
            if (tid < 8) reinterpret_cast<uint4*>(vb + (size_t)(pos - t0) * kHd)[tid] = reinterpret_cast<const uint4*>(s_new8 + kHd)[tid];
            pc_cbar();
        }
        if (tid < kHd) value_sum_chunk<1>(vb + tid, s_sc + t0, tp, nkeys, o);
        pc_cbar();                                                // buffer free again
        if (tid == 0 && c + 2 < n_chunks) issue_v(c + 2);
    }
    if (tid < kHd) p.attn_out[hq * kHd + tid] = o[0];
    return make_uint3(vuse[0], vuse[1], copy_failed ? 1u : 0u);
}

// ---- the steps of a phase, each a function of its own ---------------------------------------------------------------------
// Not inlined on purpose: inlined into one kernel body their live values competed for the 128 registers a thread has and
// the latency-bound loops (the chain of adds, the product loop) ran out of spilled locals. Every step finds its buffers
// from the launch parameters and the shared-memory base.
enum { PC_PH_QKV = 0, PC_PH_OUT = 1, PC_PH_GATEUP = 2, PC_PH_DOWN = 3, PC_PH_FINAL = 4 };

struct PcView {
    volatile int* s_abort;
    const PcLayer* layers;
    int* s_d;
    float* s_red;
    int* s_range;
    int* s_suma;
    float *s_x, *s_h1, *s_sq, *s_y;
    uint32_t* s_b;
    unsigned char* scratch;
    int32_t *a_qkv, *a_o, *a_gu, *a_d;
};

__device__ __forceinline__ PcView pc_view(const PcParams& p, unsigned char* smem) {
    PcView v;
    v.s_abort = reinterpret_cast<volatile int*>(smem + 208);
    v.layers = reinterpret_cast<const PcLayer*>(smem + p.plan.off_layers);
    v.s_d = reinterpret_cast<int*>(smem + p.plan.off_sd);
    v.s_red = reinterpret_cast<float*>(smem + p.plan.off_red);
    v.s_range = reinterpret_cast<int*>(v.s_red + 48);
    v.s_suma = reinterpret_cast<int*>(smem + p.plan.off_suma);
    v.s_x = reinterpret_cast<float*>(smem + p.plan.off_x);
    v.s_h1 = reinterpret_cast<float*>(smem + p.plan.off_h1);
    v.s_sq = reinterpret_cast<float*>(smem + p.plan.off_sq);
    v.scratch = smem + p.plan.off_scratch;
    v.s_y = reinterpret_cast<float*>(v.scratch);
    v.s_b = reinterpret_cast<uint32_t*>(v.scratch + (size_t)(p.ffn > p.h ? p.ffn : p.h) * 4);
    v.a_qkv = p.acc;
    v.a_o = v.a_qkv + p.qd + 2 * p.kvd;
    v.a_gu = v.a_o + p.h;
    v.a_d = v.a_gu + 2 * p.ffn;
    return v;
}

__device__ __forceinline__ PcRing pc_ring(const PcParams& p, unsigned char* smem) {
    PcRing r;
    r.full = reinterpret_cast<uint64_t*>(smem);
    r.empty = r.full + kPcMaxStages;
    r.base = smem + p.plan.off_ring;
    r.n_stages = p.plan.n_stages;
    return r;
}

// This phase's input vector (and its squares): the previous phase's epilogue applied to that phase's accumulators.
// PC_PH_FINAL: the residual stream after the last layer (l = number of layers).
__device__ __noinline__ void pc_step_input(const PcParams& p, unsigned char* smem, int l, int ph, float inv_prev, int tid) {
    const PcView v = pc_view(p, smem);
    const bool lead = blockIdx.x == 0;
    const bool last = l == p.n_layers - 1;
    const bool resid_x = ph == PC_PH_QKV || ph == PC_PH_FINAL;            // x = h1 + down of layer l - 1
    const PcLayer& ly = v.layers[resid_x ? l - 1 : l];
    const float sc0 = resid_x ? inv_prev * ly.s_down : ph == PC_PH_GATEUP ? inv_prev * ly.s_o : ph == PC_PH_DOWN ? inv_prev * ly.s_gate : 0.0f;
    const float sc1 = ph == PC_PH_DOWN ? inv_prev * ly.s_up : 0.0f;
    const int32_t* in0 = resid_x ? v.a_d : ph == PC_PH_OUT ? reinterpret_cast<const int32_t*>(p.attn_out) : ph == PC_PH_GATEUP ? v.a_o : v.a_gu;
    const int n_in = ph == PC_PH_OUT ? p.qd : ph == PC_PH_DOWN ? p.ffn : p.h;
    const int stride = pc_sq_stride(n_in);
    pc_for_acc<true>(in0, ph == PC_PH_DOWN ? v.a_gu + p.ffn : in0, n_in, tid, [&](int i, int a0, int a1) {
        float x;
        if (resid_x) {
            x = v.s_h1[i] + (float)a0 * sc0;                                                  // x = h1 + down (:1628)
            v.s_x[i] = x;
            if (ph == PC_PH_FINAL && lead) p.b_x[i] = x;
        } else if (ph == PC_PH_OUT) {
            x = __int_as_float(a0);                                                           // attention output
            v.s_y[i] = x;
        } else if (ph == PC_PH_GATEUP) {
            x = v.s_x[i] + (float)a0 * sc0;                                                   // h1 = x + out (:1590)
            v.s_h1[i] = x;
            if (last && lead) p.b_h1[i] = x;
        } else {
            const float gv = (float)a0 * sc0, uv = (float)a1 * sc1;
            const float rl = fmaxf(0.0f, gv);
            x = (rl * rl) * uv;                                                               // :1618-1619
            v.s_y[i] = x;
            if (last && lead) p.b_act[i] = x;
        }
        v.s_sq[pc_sq_index(i, stride)] = __fmul_rn(x, x);
    });
    pc_cbar();
}

__device__ __noinline__ float pc_step_quantise(const PcParams& p, unsigned char* smem, int l, int ph, int tid) {
    const PcView v = pc_view(p, smem);
    const PcLayer& ly = v.layers[l];
    const float* src = ph == PC_PH_QKV ? v.s_x : ph == PC_PH_GATEUP ? v.s_h1 : v.s_y;
    const float* norm_w = ph == PC_PH_QKV ? ly.in_norm : ph == PC_PH_OUT ? ly.attn_sub_norm : ph == PC_PH_GATEUP ? ly.post_norm : ly.ffn_sub_norm;
    const int K = ph == PC_PH_OUT ? p.qd : ph == PC_PH_DOWN ? p.ffn : p.h;
    return pc_quantise(src, v.s_sq, v.s_y, norm_w, K, p.eps, v.s_b, v.s_suma, v.s_red, tid);
}

// Returns the ring position after the phase, with bit 31 set if a wait on a weight copy gave up.
__device__ __noinline__ unsigned pc_step_matvec(const PcParams& p, unsigned char* smem, int ph, unsigned chunk, int tid) {
    const PcView v = pc_view(p, smem);
    const PcRing ring = pc_ring(p, smem);
    const int n_blocks = ph == PC_PH_QKV ? (p.qd + 2 * p.kvd) / 64 : ph == PC_PH_GATEUP ? 2 * p.ffn / 64 : p.h / 64;
    const int nsets = ph == PC_PH_DOWN ? p.ffn / 32 : p.h / 32;
    int32_t* acc_out = ph == PC_PH_QKV ? v.a_qkv : ph == PC_PH_OUT ? v.a_o : ph == PC_PH_GATEUP ? v.a_gu : v.a_d;
    bool failed = false;
    pc_matvec(ring, chunk, n_blocks, nsets, v.s_b, v.s_d, v.s_suma, v.s_range, acc_out, tid, v.s_abort, failed);
    return chunk | (failed ? 0x80000000u : 0u);
}

// Final RMSNorm + absmax(127) quantiser (:1638, :1666-1678), this CTA's rows of the LM head, the CTA's best candidate.
__device__ __noinline__ void pc_step_lm_head(const PcParams& p, unsigned char* smem, int tid) {
    const PcView v = pc_view(p, smem);
    const int lane = tid & 31, warp = tid >> 5;
    int8_t* s_x8 = reinterpret_cast<int8_t*>(v.s_b);
    LmBest* s_best = reinterpret_cast<LmBest*>(v.s_d);
    const float m = fmaxf(pc_norm_absmax(v.s_x, v.s_sq, v.s_y, p.final_norm, p.h, p.eps, v.s_red, tid), 1e-8f);
    const float sx = m / 127.0f;                                  // :1671
    const float inv_s = 1.0f / sx;                                // :1672
#pragma unroll 1
    for (int i = tid; i < p.h; i += kPcThreads) s_x8[i] = (int8_t)(int)fminf(fmaxf(roundf(v.s_y[i] * inv_s), -128.0f), 127.0f);
    pc_cbar();
    // Rows straight from global memory, two per warp in flight (plain 128-bit streaming loads reach the HBM rate;
    // bulk copies of this size do not), dp4a against the int8 activations, first maximum wins.
    int lm_r0, lm_r1;
    pc_share((unsigned)p.V, lm_r0, lm_r1);
    float best_v = -INFINITY;
    int best_i = 0x7fffffff;
    const int nvec = p.h >> 4;
    const uint4* x8v = reinterpret_cast<const uint4*>(s_x8);
#pragma unroll 1
    for (int v0 = lm_r0 + 2 * warp; v0 < lm_r1; v0 += 2 * kPcWarps) {
        const bool two = v0 + 1 < lm_r1;
        const uint4* rowa = reinterpret_cast<const uint4*>(p.lm_w + (size_t)v0 * p.h);
        const uint4* rowb = reinterpret_cast<const uint4*>(p.lm_w + (size_t)(two ? v0 + 1 : v0) * p.h);
        const float rs = lane < 2 ? __ldg(p.lm_scales + (lane == 1 && two ? v0 + 1 : v0)) : 0.0f;
        int acc_a = 0, acc_b = 0;
#pragma unroll 1
        for (int q0 = 0; q0 < nvec; q0 += 32 * 4) {
            uint4 wa[4], wb[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int q = q0 + u * 32 + lane;
                wa[u] = wb[u] = make_uint4(0, 0, 0, 0);
                if (q < nvec) {
                    wa[u] = ld_stream_u4(rowa + q);
                    wb[u] = ld_stream_u4(rowb + q);
                }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int q = q0 + u * 32 + lane;
                if (q < nvec) {
                    const uint4 xv = x8v[q];
                    acc_a = dp4a_ss(wa[u].x, xv.x, acc_a); acc_a = dp4a_ss(wa[u].y, xv.y, acc_a);
                    acc_a = dp4a_ss(wa[u].z, xv.z, acc_a); acc_a = dp4a_ss(wa[u].w, xv.w, acc_a);
                    acc_b = dp4a_ss(wb[u].x, xv.x, acc_b); acc_b = dp4a_ss(wb[u].y, xv.y, acc_b);
                    acc_b = dp4a_ss(wb[u].z, xv.z, acc_b); acc_b = dp4a_ss(wb[u].w, xv.w, acc_b);
                }
            }
        }
        acc_a = warp_sum_i(acc_a);
        acc_b = warp_sum_i(acc_b);
        if (lane < 2 && (lane == 0 || two)) {
            const int vr = v0 + lane;
            const float lg = (float)(lane == 0 ? acc_a : acc_b) * (sx * rs);   // :1717
            p.b_logits[vr] = lg;
            if (better(lg, vr, best_v, best_i)) { best_v = lg; best_i = vr; }
            if (vr == 0 && lg != lg) { best_v = INFINITY; best_i = 0; }        // a NaN at index 0 is never displaced (:1747-1753)
        }
    }
    {   // lanes 0 and 1 of every warp hold candidates
        const float ov = __shfl_sync(0xffffffffu, best_v, 1);
        const int oi = __shfl_sync(0xffffffffu, best_i, 1);
        if (lane == 0) {
            if (better(ov, oi, best_v, best_i)) { best_v = ov; best_i = oi; }
            s_best[warp].val = best_v;
            s_best[warp].idx = best_i;
        }
    }
    pc_cbar();
    if (tid == 0) {
        LmBest b = s_best[0];
        for (int i = 1; i < kPcWarps; ++i)
            if (better(s_best[i].val, s_best[i].idx, b.val, b.idx)) b = s_best[i];
        p.cta_best[blockIdx.x] = b;
    }
}

// ---- the kernel -----------------------------------------------------------------------------------------------------
// The four matrix-vector phases of a layer run through ONE copy of the quantiser and of the product loop (a loop over
// phases that is deliberately not unrolled): the kernel's instructions must stay resident in the SM's instruction cache
// across layers - a first version with every phase inlined separately was 235 KB of code and ran every phase several
// times slower than the same code in a small kernel.
__global__ void __launch_bounds__(kPcBlock, 1) decode_persistent_kernel(const __grid_constant__ PcParams p) {
    extern __shared__ __align__(128) unsigned char smem[];
    uint64_t* s_full = reinterpret_cast<uint64_t*>(smem);                   // [kPcMaxStages]
    uint64_t* s_empty = s_full + kPcMaxStages;                              // [kPcMaxStages]
    uint64_t* s_vbar = s_empty + kPcMaxStages;                              // [2]
    volatile int* s_abort = reinterpret_cast<volatile int*>(smem + 208);
    unsigned long long* s_phase = reinterpret_cast<unsigned long long*>(smem + 216);   // [8] + last stamp: bytes 216..287
    const PcLayer* s_layers = reinterpret_cast<const PcLayer*>(smem + p.plan.off_layers);   // the layer table, copied once
    int* s_d = reinterpret_cast<int*>(smem + p.plan.off_sd);                // [kPcMaxSlots][64]
    float* s_red = reinterpret_cast<float*>(smem + p.plan.off_red);         // [48] reduction scratch
    int* s_range = reinterpret_cast<int*>(s_red + 48);                      // [kPcMaxSlots]
    int* s_suma = reinterpret_cast<int*>(smem + p.plan.off_suma);           // [Kmax / 32]
    float* s_x = reinterpret_cast<float*>(smem + p.plan.off_x);             // [h] residual stream
    float* s_h1 = reinterpret_cast<float*>(smem + p.plan.off_h1);           // [h]
    unsigned char* scratch = smem + p.plan.off_scratch;
    const int kmax = p.ffn > p.h ? p.ffn : p.h;
    float* s_y = reinterpret_cast<float*>(scratch);                         // [Kmax] normalised activations
    uint32_t* s_b = reinterpret_cast<uint32_t*>(scratch + (size_t)kmax * 4);   // [Kmax / 4] B-fragment words
    float* s_sq = reinterpret_cast<float*>(smem + p.plan.off_sq);           // [8][Kmax / 8 + 4] squares, chain-major
    PcRing ring;
    ring.full = s_full;
    ring.empty = s_empty;
    ring.base = smem + p.plan.off_ring;
    ring.n_stages = p.plan.n_stages;

    const int tid = threadIdx.x;
    if (tid == 0) {
        for (int i = 0; i < kPcMaxStages; ++i) {
            mbar_init(&s_full[i], 1);
            mbar_init(&s_empty[i], kPcWarps);
        }
        mbar_init(&s_vbar[0], 1);
        mbar_init(&s_vbar[1], 1);
        mbar_init_fence();
        *s_abort = 0;
    }
    for (int i = tid; i < kPcMaxSlots * 64; i += kPcBlock) s_d[i] = 0;
    if (tid < kPcMaxSlots) s_range[tid] = 0;
    {   // a field of the table read from global memory where it is needed would put an L2 round trip on the dependent chain
        const uint32_t* src = reinterpret_cast<const uint32_t*>(p.layers);
        uint32_t* dst = reinterpret_cast<uint32_t*>(smem + p.plan.off_layers);
        for (int i = tid; i < p.n_layers * (int)(sizeof(PcLayer) / 4); i += kPcBlock) dst[i] = __ldg(src + i);
    }
    __syncthreads();                                   // the only barrier that includes the producer warp

    const int pos = p.pos_arg >= 0 ? p.pos_arg : *p.pos;
    if (pos < 0 || pos >= p.max_seq || pos + 1 > p.plan.score_cap) {      // uniform over the grid: everyone leaves
        if (tid == 0 && blockIdx.x == 0) pc_fail(p, s_abort, PC_ERR_POSITION);
        return;
    }
    const int L = p.n_layers;
    const int nb_qkv = (p.qd + 2 * p.kvd) / 64, nb_h = p.h / 64, nb_gu = 2 * p.ffn / 64;
    const int ns_h = p.h / 32, ns_f = p.ffn / 32;

    // ---- producer warp ---------------------------------------------------------------------------------------------
    if (tid >= kPcThreads) {
        if (tid == kPcThreads) {
            PcProducer prod(ring, s_abort);
#pragma unroll 1
            for (int l = 0; l < L; ++l) {
                const PcLayer& ly = s_layers[l];
#pragma unroll 1
                for (int ph = 0; ph < 4; ++ph) {
                    const uint8_t* w = ph == PC_PH_QKV ? ly.qkv : ph == PC_PH_OUT ? ly.o : ph == PC_PH_GATEUP ? ly.gu : ly.down;
                    prod.matrix(w, ph == PC_PH_QKV ? nb_qkv : ph == PC_PH_GATEUP ? nb_gu : nb_h, ph == PC_PH_DOWN ? ns_f : ns_h);
                }
            }
            if (prod.stopped) {
                // the consumers gave up: wait (bounded) for the copies still in flight before this CTA's memory goes away
                const unsigned n = prod.chunk < (unsigned)ring.n_stages ? prod.chunk : (unsigned)ring.n_stages;
                for (unsigned k = 0; k < n; ++k) {
                    const unsigned c = prod.chunk - 1 - k;
                    mbar_wait_bounded(&ring.full[c % (unsigned)ring.n_stages], (c / (unsigned)ring.n_stages) & 1u);
                }
            }
        }
        return;
    }

    // ---- consumers -------------------------------------------------------------------------------------------------
    const int lane = tid & 31, warp = tid >> 5;
    const bool lead = blockIdx.x == 0;
    unsigned arrivals = 0, chunk = 0;
    uint3 attn_state = make_uint3(0u, 0u, 0u);
    bool copy_failed = false;
    int32_t* a_qkv = p.acc;
    int32_t* a_o = a_qkv + p.qd + 2 * p.kvd;
    int32_t* a_gu = a_o + p.h;
    int32_t* a_d = a_gu + 2 * p.ffn;
    // per-phase time of the first CTA, summed in shared memory and added to the global counters once, at the end
    const bool timing = p.phase_ns && lead && tid == 0;
    if (timing) {
        for (int k = 0; k < 8; ++k) s_phase[k] = 0;
        s_phase[8] = pc_gtime();
        s_phase[7] = (unsigned long long)clock64();
    }
    auto stamp = [&](int k) {
        if (timing) {
            const unsigned long long now = pc_gtime();
            s_phase[k] += now - s_phase[8];
            s_phase[8] = now;
        }
    };

    {   // embedding row (:1299-1315)
        int tok = p.token_arg >= 0 ? p.token_arg : *p.tokens;
        if (tok < 0 || tok >= p.V) tok = 0;
        const int8_t* row = p.lm_w + (size_t)tok * p.h;
        const float sc = p.lm_scales[tok];
        const int stride = pc_sq_stride(p.h);
#pragma unroll 1
        for (int i = tid; i < p.h; i += kPcThreads) {
            const float v = (float)row[i] * sc;                        // :1313
            s_x[i] = v;
            s_sq[pc_sq_index(i, stride)] = __fmul_rn(v, v);
        }
    }
    pc_cbar();
    float inv_prev = 0.0f;                             // m/31 of the previous phase's activations
#pragma unroll 1
    for (int l = 0; l < L; ++l) {
        const PcLayer& ly = s_layers[l];
        const bool last = l == L - 1;
#pragma unroll 1
        for (int ph = 0; ph < 4; ++ph) {
#ifdef TZ_PC_TRACE
            if (tid == 0 && lead) g_pc_trace = (p.phase_ns && l == (L > 2 ? 2 : 0) && ph == TZ_PC_TRACE) ? p.phase_ns + 8 : nullptr;
            PC_TR(34);
#endif
            if (!(ph == PC_PH_QKV && l == 0)) pc_step_input(p, smem, l, ph, inv_prev, tid);   // layer 0 starts from the embedding row
            PC_TR(0);
            const float inv_act = pc_step_quantise(p, smem, l, ph, tid);
            chunk = pc_step_matvec(p, smem, ph, chunk, tid);
            if (chunk & 0x80000000u) { copy_failed = true; chunk &= 0x7fffffffu; }
            // the next phase's norm weights on their way into L2 during the barrier
            if (ph == PC_PH_QKV) pc_prefetch_norm(ly.attn_sub_norm, p.qd, tid);
            else if (ph == PC_PH_OUT) pc_prefetch_norm(ly.post_norm, p.h, tid);
            else if (ph == PC_PH_GATEUP) pc_prefetch_norm(ly.ffn_sub_norm, p.ffn, tid);
            else pc_prefetch_norm(last ? p.final_norm : s_layers[l + 1].in_norm, p.h, tid);
            PC_TR(32);
            arrivals = pc_grid_barrier(p, arrivals, tid, s_abort);
            PC_TR(33);
            stamp(ph == PC_PH_QKV ? 0 : ph + 1);
            // clear what every CTA has finished reading before the barrier above
            if (ph == PC_PH_QKV) { if (l > 0) pc_zero_slice(a_d, p.h, tid); }
            else if (ph == PC_PH_GATEUP) pc_zero_slice(a_o, p.h, tid);
            else if (ph == PC_PH_DOWN) pc_zero_slice(a_gu, 2 * p.ffn, tid);
            if (ph == PC_PH_QKV) {
                // ---- attention: one query head per CTA ------------------------------------------------------------------
                if ((int)blockIdx.x < p.n_q)
                    attn_state = pc_attention_head(p, ly, l, blockIdx.x, pos, inv_act, last, scratch, s_vbar, attn_state, tid, s_abort);
                arrivals = pc_grid_barrier(p, arrivals, tid, s_abort);
                stamp(1);
                pc_zero_slice(a_qkv, p.qd + 2 * p.kvd, tid);
            }
            inv_prev = inv_act;
        }
    }
    pc_step_input(p, smem, L, PC_PH_FINAL, inv_prev, tid);         // residual stream after the last layer
    int next_token = 0;
    if (p.with_logits) pc_step_lm_head(p, smem, tid);
    arrivals = pc_grid_barrier(p, arrivals, tid, s_abort);
    stamp(5);
    pc_zero_slice(a_d, p.h, tid);
    if (lead && p.with_logits) {
        LmBest* s_best = reinterpret_cast<LmBest*>(s_d);
        pc_cbar();
        LmBest b = {-INFINITY, 0x7fffffff};
#pragma unroll 1
        for (int i = tid; i < (int)gridDim.x; i += kPcThreads) {
            LmBest c;
            c.val = __ldcg(&p.cta_best[i].val);
            c.idx = __ldcg(&p.cta_best[i].idx);
            if (better(c.val, c.idx, b.val, b.idx)) b = c;
        }
#pragma unroll
        for (int msk = 16; msk > 0; msk >>= 1) {
            LmBest o;
            o.val = __shfl_xor_sync(0xffffffffu, b.val, msk);
            o.idx = __shfl_xor_sync(0xffffffffu, b.idx, msk);
            if (better(o.val, o.idx, b.val, b.idx)) b = o;
        }
        if (lane == 0) s_best[warp] = b;
        pc_cbar();
        if (tid == 0) {
            b = s_best[0];
            for (int i = 1; i < kPcWarps; ++i)
                if (better(s_best[i].val, s_best[i].idx, b.val, b.idx)) b = s_best[i];
            next_token = b.idx == 0x7fffffff ? 0 : b.idx;             // nothing compared greater: index 0 (:1746)
            *p.next = next_token;
            if (p.host_next) {
                *reinterpret_cast<volatile int*>(p.host_next) = next_token;
                __threadfence_system();
            }
        }
    }
    if (lead && tid == 0) {
        *p.pos = pos + 1;                                             // once per token, after all layers (:1831-1835)
        if (p.with_logits && p.feed_back) *p.tokens = next_token;
    }
    if (copy_failed) pc_fail(p, s_abort, PC_ERR_WEIGHT_COPY);
    if (attn_state.z) pc_fail(p, s_abort, PC_ERR_VALUE_COPY);
    stamp(6);
    if (timing) {
        for (int k = 0; k < 7; ++k) p.phase_ns[k] += s_phase[k];
        p.phase_ns[7] += (unsigned long long)clock64() - s_phase[7];      // SM cycles of the launch: with the sum above, the clock it ran at
    }
}

// ---- host side ------------------------------------------------------------------------------------------------------
int pc_grid_size() {
    int dev = 0, coop = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    if (cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev) != cudaSuccess || !coop) return 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    return sms;
}

bool pc_plan(int h, int qd, int kvd, int ffn, int n_q, int n_kv, int V, int n_layers, int max_len, int grid, PcSmemPlan* out) {
    if (n_layers <= 0 || n_layers > 256) return false;
    if (grid <= 0 || n_q > grid || n_q <= 0 || n_kv <= 0 || n_q % n_kv) return false;
    if (h % 32 || ffn % 32 || qd != h || kvd % 64 || h % 64 || ffn % 64 || h > kPcStageBytes || V <= 0 || max_len <= 0) return false;
    if ((unsigned long long)(2 * ffn / 64) * (h / 32) * grid >= (1ull << 32) || (unsigned long long)(h / 64) * (ffn / 32) * grid >= (1ull << 32) ||
        (unsigned long long)V * grid >= (1ull << 32))
        return false;
    const int kmax = ffn > h ? ffn : h;
    // row blocks one CTA's share of a matrix can touch: ceil(units per CTA / units per row block) + 1
    auto slots = [&](long long n_blocks, long long nsets) { return (int)(((n_blocks * nsets + grid - 1) / grid + nsets - 1) / nsets + 1); };
    if (slots((qd + 2 * kvd) / 64, h / 32) > kPcMaxSlots || slots(h / 64, h / 32) > kPcMaxSlots || slots(2 * ffn / 64, h / 32) > kPcMaxSlots ||
        slots(h / 64, ffn / 32) > kPcMaxSlots)
        return false;
    auto up = [](int v, int a) { return (v + a - 1) / a * a; };
    PcSmemPlan pl;
    pl.off_sd = 384;
    pl.off_red = pl.off_sd + kPcMaxSlots * 64 * 4;
    pl.off_suma = pl.off_red + 256;
    pl.off_layers = pl.off_suma + up(kmax / 32 * 4, 128);
    pl.off_x = pl.off_layers + up(n_layers * (int)sizeof(PcLayer), 128);
    pl.off_h1 = pl.off_x + up(h * 4, 128);
    pl.off_sq = pl.off_h1 + up(h * 4, 128);
    pl.off_scratch = pl.off_sq + up((kmax + 32) * 4, 128);
    const int gemv_bytes = kmax * 5;                                        // y floats + B-fragment words
    const int attn_bytes = kPcAttnFixed + 4 * ((max_len + 3) & ~3);
    pl.scratch_bytes = up(gemv_bytes > attn_bytes ? gemv_bytes : attn_bytes, 128);
    pl.off_ring = pl.off_scratch + pl.scratch_bytes;
    const int room = 227 * 1024 - pl.off_ring;
    pl.n_stages = room / kPcStageBytes;
    if (pl.n_stages > kPcMaxStages) pl.n_stages = kPcMaxStages;
    if (pl.n_stages < 2) return false;
    pl.total_bytes = pl.off_ring + pl.n_stages * kPcStageBytes;
    pl.score_cap = (pl.scratch_bytes - kPcAttnFixed) / 4;
    *out = pl;
    return true;
}

cudaError_t pc_launch(const PcParams& p, int grid, cudaStream_t st) {
    static int attr_bytes = 0;
    if (p.plan.total_bytes > attr_bytes) {
        cudaError_t e = cudaFuncSetAttribute(decode_persistent_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (e != cudaSuccess) return e;
        attr_bytes = 227 * 1024;
    }
    void* args[] = {const_cast<PcParams*>(&p)};
    return cudaLaunchCooperativeKernel((const void*)decode_persistent_kernel, dim3((unsigned)grid), dim3(kPcBlock), args,
                                       (size_t)p.plan.total_bytes, st);
}

}  // namespace tz
