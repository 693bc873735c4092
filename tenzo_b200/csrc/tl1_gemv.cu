// TL1 ternary GEMV for sm_100a with the RMSNorm + absmax(31) activation quantiser fused into its
// prologue and the reference's three epilogues (store / residual add / squared-ReLU GLU).
//
// What it replaces in the reference CPU engine (src/runtime/TenzoEngine.cpp): rms_norm_raw
// (:148-166), build_lut (:22-62), compute_single_block (:64-127) and their call sites (:1542-1628).
//
// How the arithmetic is organised on the GPU
//   * The reference looks every 4-bit index up in a 16-entry table of clamp(w0*a0+w1*a1). With
//     |a| <= 31 the clamp can never fire, so the accumulator is the plain integer dot product
//     sum_k w[r][k]*a[k]; any exact integer evaluation gives the same int32.
//   * A warp streams one 64-row block in tiles of 64 column pairs (2 KB, four coalesced 128-bit
//     loads per lane, all issued before anything else so HBM latency is paid once).
//     Lane l's i-th load holds, for column pair g = 64t + 16i + (l>>1), the 16 bytes of row pairs
//     c = 16(l&1) .. +15. A 4x4 byte transpose (8 PRMT per 16 bytes) turns that into words that
//     carry ONE row pair at four column pairs, which is the shape dp4a wants.
//   * Each byte is c0 | c1<<2 | c2<<4 | c3<<6 with codes c = w+1 in {0,1,2}: (c0,c1) = row c at
//     columns (2g,2g+1), (c2,c3) = row c+32. Masking (no shifts) gives bytes c0, 4*c1, 16*c2,
//     64*c3; the even-column activation is stored pre-multiplied by 4 (|4a| <= 124 fits int8), so
//     dp4a(mask0,4a_even)+dp4a(mask1,a_odd) = 4*sum(c*a) for the low row and the other two masks
//     give 64*sum(c*a) for the high row. One LOP3 + one DP4A per 4 weights.
//   * sum(w*a) = sum(c*a) - sum(a); sum(a) falls out of two extra dp4a per tile.
//   * Lanes of equal parity hold partial sums for the same 32 rows at different columns: a
//     halving butterfly (30 shuffles) leaves every lane with two finished rows.
//   * K can be split across CTAs; partials meet in an int32 scratch through atomicAdd (integer,
//     hence order-free and exact) and the last CTA to arrive runs the epilogue and re-zeroes the
//     scratch.
#include "common.cuh"
#include "../../include/tenzo_kernels.h"

namespace tz {

constexpr int kGemvWarps = 8;
constexpr int kGemvThreads = kGemvWarps * 32;
constexpr int kTileGroups = 64;   // column pairs per warp tile
constexpr int kUnroll = 4;        // tiles whose loads are in flight per warp at once

struct GemvLaunch {
    tenzo_tl1_gemv_args a;
    int ksplit;
    int units;       // CTAs along the row dimension (n_blocks, or n_blocks/2 in GLU mode)
    int tiles;       // ceil(K/2 / 64)
};

__device__ __forceinline__ float seg_scale_for(const tenzo_tl1_gemv_args& a, int block) {
    return block < a.seg_end[0] ? a.seg_scale[0] : (block < a.seg_end[1] ? a.seg_scale[1] : a.seg_scale[2]);
}

// One tile: 4 registers-worth (uint4) per lane already loaded; accumulate into lo/hi.
__device__ __forceinline__ void consume_tile(const uint4 (&r)[4], uint32_t ae4, uint32_t ao,
                                             int (&lo)[16], int (&hi)[16], int& sa4) {
    sa4 = dp4a_us(0x01010101u, ae4, sa4);
    sa4 = dp4a_us(0x04040404u, ao, sa4);
    const uint32_t* w0 = reinterpret_cast<const uint32_t*>(&r[0]);
    const uint32_t* w1 = reinterpret_cast<const uint32_t*>(&r[1]);
    const uint32_t* w2 = reinterpret_cast<const uint32_t*>(&r[2]);
    const uint32_t* w3 = reinterpret_cast<const uint32_t*>(&r[3]);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        // 4x4 byte transpose: T[m] = (R0.m, R1.m, R2.m, R3.m)
        const uint32_t t0 = prmt(w0[j], w1[j], 0x5140u), t1 = prmt(w2[j], w3[j], 0x5140u);
        const uint32_t t2 = prmt(w0[j], w1[j], 0x7362u), t3 = prmt(w2[j], w3[j], 0x7362u);
        uint32_t T[4];
        T[0] = prmt(t0, t1, 0x5410u);
        T[1] = prmt(t0, t1, 0x7632u);
        T[2] = prmt(t2, t3, 0x5410u);
        T[3] = prmt(t2, t3, 0x7632u);
#pragma unroll
        for (int m = 0; m < 4; ++m) {
            const int c = 4 * j + m;
            lo[c] = dp4a_us(T[m] & 0x03030303u, ae4, lo[c]);
            lo[c] = dp4a_us(T[m] & 0x0C0C0C0Cu, ao, lo[c]);
            hi[c] = dp4a_us(T[m] & 0x30303030u, ae4, hi[c]);
            hi[c] = dp4a_us(T[m] & 0xC0C0C0C0u, ao, hi[c]);
        }
    }
}

__global__ void __launch_bounds__(kGemvThreads) tl1_gemv_kernel(const GemvLaunch L) {
    const tenzo_tl1_gemv_args& a = L.a;
    extern __shared__ __align__(16) uint32_t smem[];
    // smem: act_e[tiles*16] | act_o[tiles*16] | red[128] | fscratch[32] | flag[4] | x[K]
    uint32_t* s_ae = smem;
    uint32_t* s_ao = smem + L.tiles * 16;
    int* s_red = reinterpret_cast<int*>(smem + 2 * L.tiles * 16);
    float* s_f = reinterpret_cast<float*>(s_red + 128);
    int* s_flag = reinterpret_cast<int*>(s_f + 32);
    float* s_x = reinterpret_cast<float*>(s_flag + 4);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int unit = blockIdx.x / L.ksplit, split = blockIdx.x % L.ksplit, seq = blockIdx.y;
    const bool glu = a.epilogue == TENZO_EPI_RELU2_GLU;
    const int nb_cta = glu ? 2 : 1;                 // row blocks handled by this CTA
    const int wb = kGemvWarps / nb_cta;             // warps per row block
    const int my_blk = glu ? (warp & 1) : 0;        // which of the CTA's row blocks this warp feeds
    const int wi = glu ? (warp >> 1) : warp;        // index among the warps of that row block
    const int block = glu ? (my_blk ? unit + L.units : unit) : unit;
    const int kh = a.K >> 1;                        // column pairs

    // K range of this CTA in tiles, and this warp's tiles: t_begin + wi, + wb, ...
    const int t_begin = (int)(((long long)L.tiles * split) / L.ksplit);
    const int t_end = (int)(((long long)L.tiles * (split + 1)) / L.ksplit);
    const int my_tiles = (t_end - t_begin - wi + wb - 1) / wb;   // may be <= 0

    const uint8_t* wblk = a.w + (size_t)block * kh * 32;
    uint4 r[kUnroll][4];
    auto load_tiles = [&](int first) {
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const int t = t_begin + wi + (first + u) * wb;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int g = t * kTileGroups + 16 * i + (lane >> 1);
                if (first + u < my_tiles && g < kh)
                    r[u][i] = ld_stream_u4(wblk + (size_t)g * 32 + (lane & 1) * 16);
                else
                    r[u][i] = make_uint4(0, 0, 0, 0);
            }
        }
    };
    // Weights do not depend on the previous kernel: get them moving before anything else.
    load_tiles(0);

    if (tid < 128) s_red[tid] = 0;
    for (int i = tid; i < 2 * L.tiles * 16; i += kGemvThreads) smem[i] = 0;   // zero pad ragged K

    if (a.use_pdl) pdl_wait();

    // ---- prologue: RMSNorm + absmax(31) quantiser, recomputed identically by every CTA ----------
    // x is staged in shared memory once; the normalised value replaces it in place.
    const float* x = a.x + (size_t)seq * a.x_stride;
    for (int i = tid; i < a.K; i += kGemvThreads) s_x[i] = __ldcg(x + i);
    float m = 0.0f;
    if (a.do_norm) {
        __syncthreads();
        const float ss = sumsq_reference_order(s_x, a.K, s_f);
        const float inv_rms = rms_inv(ss, a.K, a.eps);
        for (int i = tid; i < a.K; i += kGemvThreads) {   // same thread wrote s_x[i]
            const float y = rms_apply(s_x[i], inv_rms, a.norm_w, i);
            s_x[i] = y;
            m = fmaxf(m, fabsf(y));
        }
    } else {
        for (int i = tid; i < a.K; i += kGemvThreads) m = fmaxf(m, fabsf(s_x[i]));
    }
    m = fmaxf(block_max(m, s_f), 1e-6f);            // TenzoEngine.cpp:28-32 (barriers also cover the zero fill)
    const float to_q = 31.0f / m;                   // :34
    const float inv_act = m / 31.0f;                // :35
    {
        uint8_t* be = reinterpret_cast<uint8_t*>(s_ae);
        uint8_t* bo = reinterpret_cast<uint8_t*>(s_ao);
        for (int i = tid; i < a.K; i += kGemvThreads) {
            const int q = (int)roundf(s_x[i] * to_q);   // :41-42, half away from zero
            const int g = i >> 1, t = g >> 6, within = g & 63;
            const int pos = ((t * 16 + (within & 15)) << 2) + (within >> 4);
            if (i & 1) bo[pos] = (uint8_t)(int8_t)q;
            else       be[pos] = (uint8_t)(int8_t)(4 * q);
            if (a.a_out && blockIdx.x == 0) a.a_out[(size_t)seq * a.K + i] = (int8_t)q;
        }
        if (a.inv_out && blockIdx.x == 0 && tid == 0) a.inv_out[seq] = inv_act;
    }
    __syncthreads();
    if (a.use_pdl) pdl_launch_dependents();

    // ---- main loop ---------------------------------------------------------------------------
    int lo[16], hi[16], sa4 = 0;
#pragma unroll
    for (int c = 0; c < 16; ++c) { lo[c] = 0; hi[c] = 0; }
    for (int first = 0; first < my_tiles; first += kUnroll) {
        if (first > 0) load_tiles(first);
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            if (first + u < my_tiles) {
                const int t = t_begin + wi + (first + u) * wb;
                consume_tile(r[u], s_ae[t * 16 + (lane >> 1)], s_ao[t * 16 + (lane >> 1)], lo, hi, sa4);
            }
        }
    }

    // ---- reduce across the 16 lanes of equal parity: halving butterfly -------------------------
    int v[32];
#pragma unroll
    for (int c = 0; c < 16; ++c) { v[c] = lo[c]; v[16 + c] = hi[c]; }
#pragma unroll
    for (int h = 16; h >= 2; h >>= 1) {             // xor masks 16, 8, 4, 2
        const bool up = (lane & h) != 0;
#pragma unroll
        for (int i = 0; i < h; ++i) {
            const int keep = up ? v[i + h] : v[i];
            const int send = up ? v[i] : v[i + h];
            v[i] = keep + __shfl_xor_sync(0xffffffffu, send, h);
        }
    }
#pragma unroll
    for (int msk = 2; msk <= 16; msk <<= 1) sa4 += __shfl_xor_sync(0xffffffffu, sa4, msk);
    const int sum_a = sa4 >> 2;                     // sum of a over this warp's columns (exact)
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int o = i + (lane & 30);              // index in the original lo|hi array
        const int row = (o & 15) + 16 * (lane & 1) + 32 * (o >> 4);
        const int val = (o < 16 ? (v[i] >> 2) : (v[i] >> 6)) - sum_a;
        if (my_tiles > 0) atomicAdd(&s_red[my_blk * 64 + row], val);
    }
    __syncthreads();

    // ---- cross-CTA split-K meeting point ------------------------------------------------------
    const int rows_cta = nb_cta * 64;
    int acc = tid < rows_cta ? s_red[tid] : 0;
    if (L.ksplit > 1) {
        const size_t slot = (size_t)seq * L.units + unit;
        int* gacc = a.splitk_acc + slot * rows_cta;
        if (tid < rows_cta) atomicAdd(&gacc[tid], acc);
        __threadfence();
        __syncthreads();
        if (tid == 0) *s_flag = (atomicAdd(&a.splitk_cnt[slot], 1u) == (unsigned)(L.ksplit - 1));
        __syncthreads();
        if (!*s_flag) return;
        __threadfence();
        if (tid < rows_cta) acc = atomicExch(&gacc[tid], 0);   // take the total and leave zero behind
        if (tid == 0) a.splitk_cnt[slot] = 0;
    }

    // ---- epilogue -----------------------------------------------------------------------------
    if (tid < rows_cta) {
        const int blk = glu ? (tid < 64 ? unit : unit + L.units) : unit;
        const int row = blk * 64 + (tid & 63);
        if (a.acc_out) a.acc_out[(size_t)seq * a.n_blocks * 64 + row] = acc;
        const float val = (float)acc * (inv_act * seg_scale_for(a, blk));   // :1554, :118
        if (a.epilogue == TENZO_EPI_STORE) {
            a.out[(size_t)seq * a.out_stride + row] = val;
        } else if (a.epilogue == TENZO_EPI_RESIDUAL) {
            a.out[(size_t)seq * a.out_stride + row] = __ldcg(a.resid + (size_t)seq * a.out_stride + row) + val;  // :1590
        } else {
            reinterpret_cast<float*>(s_red)[tid] = val;
        }
    }
    if (glu) {
        __syncthreads();
        if (tid < 64) {
            const float g = reinterpret_cast<float*>(s_red)[tid], u = reinterpret_cast<float*>(s_red)[64 + tid];
            const float rl = fmaxf(0.0f, g);
            a.out[(size_t)seq * a.out_stride + unit * 64 + tid] = (rl * rl) * u;   // :1618-1619
        }
    }
}

static int pick_ksplit(int n_blocks, int K, int epilogue) {
    const int tiles = ((K >> 1) + kTileGroups - 1) / kTileGroups;
    const int nb_cta = epilogue == TENZO_EPI_RELU2_GLU ? 2 : 1;
    const int units = n_blocks / nb_cta, wb = kGemvWarps / nb_cta;
    int for_regs = (tiles + wb * kUnroll - 1) / (wb * kUnroll);   // at most kUnroll tiles per warp
    int for_fill = (148 + units - 1) / units;                     // at least one CTA per SM
    int ks = for_regs > for_fill ? for_regs : for_fill;
    int cap = tiles / wb > 0 ? tiles / wb : 1;                    // keep >= one tile per warp
    if (ks > cap) ks = cap;
    if (ks < 1) ks = 1;
    if (ks > 16) ks = 16;
    return ks;
}

}  // namespace tz

extern "C" int tenzo_cuda_tl1_gemv_ksplit(int n_blocks, int K, int epilogue) {
    if (n_blocks <= 0 || K <= 0) return 1;
    return tz::pick_ksplit(n_blocks, K, epilogue);
}

extern "C" int tenzo_cuda_tl1_gemv(const tenzo_tl1_gemv_args* args, void* stream) {
    using namespace tz;
    if (!args || !args->x || !args->w || !args->out) return -1;
    const tenzo_tl1_gemv_args& a = *args;
    if (a.n_blocks <= 0 || a.K <= 0 || (a.K & 1) || a.batch <= 0) return -1;
    if ((reinterpret_cast<uintptr_t>(a.w) & 15) != 0) return -1;
    if (a.epilogue < 0 || a.epilogue > 2) return -1;
    if (a.epilogue == TENZO_EPI_RESIDUAL && !a.resid) return -1;
    if (a.epilogue == TENZO_EPI_RELU2_GLU && (a.n_blocks & 1)) return -1;
    if (a.K > 16384) return -5;   /* same bound as the reference engine's scratch vectors (:1227) */

    GemvLaunch L;
    L.a = a;
    L.tiles = ((a.K >> 1) + kTileGroups - 1) / kTileGroups;
    L.units = a.epilogue == TENZO_EPI_RELU2_GLU ? a.n_blocks / 2 : a.n_blocks;
    L.ksplit = pick_ksplit(a.n_blocks, a.K, a.epilogue);
    if (L.ksplit > 1 && (!a.splitk_acc || !a.splitk_cnt)) return -1;

    const size_t smem = (size_t)(2 * L.tiles * 16 + 128 + 32 + 4 + a.K) * sizeof(uint32_t);
    if (smem > 48 * 1024) {   // staging for K > ~11k columns exceeds the default dynamic limit
        cudaError_t ea = cudaFuncSetAttribute(tl1_gemv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
        if (ea != cudaSuccess) return (int)ea;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(L.units * L.ksplit), (unsigned)a.batch, 1);
    cfg.blockDim = dim3(kGemvThreads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = a.use_pdl ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, tl1_gemv_kernel, L);
    return e == cudaSuccess ? 0 : (int)e;
}
