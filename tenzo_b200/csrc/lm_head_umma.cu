// INT8 LM head for 16 or more sequences on tcgen05 (kind::i8, accumulators in tensor memory), sm_100a.
//
// Same computation as lm_head_kernel (compute_logits' int8 branch and the greedy argmax of the
// reference, src/runtime/TenzoEngine.cpp:1661-1719 and :1745-1755): the activations arrive already
// normalised and quantised to +-127 (rmsnorm_quant_kernel), the int32 dot products are exact, and
//   logit[seq][v] = (float)acc * (s_x[seq] * scale_v[v])           (:1717, product of scales first)
// so logits and argmax are bit-identical to the one-sequence path; the vocabulary matrix is read
// once for all sequences instead of once per eight.
//
// One CTA per 128 vocabulary rows. Both operands are K-major int8 matrices in global memory, so both
// tiles come straight from TMA with the 128-byte swizzle: warp 0 (one lane) loads {128 rows x 128 B}
// of W and {N sequences x 128 B} of the activations per stage, warp 1 (one lane) issues four
// tcgen05.mma per stage and commits them to the stage's "empty" barrier, warps 2-5 run the epilogue:
// one TMEM lane (vocabulary row) per thread, the tile of logits assembled in the pipeline's shared
// memory, per-sequence argmax candidates (first maximum wins) read back from that tile, and the
// tile written out by one TMA store when logits are wanted. All mbarrier waits are bounded.
#include "umma.cuh"
#include "lm_head.cuh"
#include "../../include/tenzo_kernels.h"

namespace tz {

constexpr int kLmuThreads = 192;
constexpr int kLmuStages = 4;
constexpr int kLmuKc = 128;                    // bytes of K per stage
constexpr int kLmuRows = 128;                  // vocabulary rows per CTA
constexpr int kLmuMaxN = 256;

struct LmUmmaLaunch {
    const float* sx;             // [batch] activation scales m/127
    const float* row_scales;     // [vocab]
    float* logits;               // [batch][vocab] or null
    int32_t* acc_out;            // [batch][vocab] or null
    LmBest* cand;                // [batch][n_tiles] argmax candidates or null
    int vocab, hidden, batch, n_tiles;
    int n_box, tmem_cols, use_pdl;
};

struct LmUmmaSmem {
    // [1024-aligned] stages x { W tile 16 KB | activation tile n_box*128 } | barriers | tmem slot | s_sx[256]
    static __host__ __device__ int stage_bytes(int n_box) { return kLmuRows * kLmuKc + n_box * kLmuKc; }
    static constexpr int n_bars = 2 * kLmuStages + 1;
    static __host__ __device__ size_t bytes(int n_box) {
        return 1024 + (size_t)kLmuStages * stage_bytes(n_box) + ((8 * n_bars + 15) & ~15) + 16 + kLmuMaxN * 4;
    }
};

__device__ int g_lmu_timeouts = 0;

__global__ void __launch_bounds__(kLmuThreads, 1) lm_head_umma_kernel(const LmUmmaLaunch L, const __grid_constant__ CUtensorMap wmap,
                                                                       const __grid_constant__ CUtensorMap amap,
                                                                       const __grid_constant__ CUtensorMap omap) {
    extern __shared__ unsigned char smem_raw[];
    const uint32_t base_off = ((smem_addr(smem_raw) + 1023u) & ~1023u) - smem_addr(smem_raw);
    unsigned char* stages = smem_raw + base_off;
    const int N = L.n_box, stage_bytes = LmUmmaSmem::stage_bytes(N);
    uint64_t* bars = reinterpret_cast<uint64_t*>(stages + (size_t)kLmuStages * stage_bytes);
    uint64_t* bar_full = bars;                         // [stages] both tiles have landed
    uint64_t* bar_empty = bars + kLmuStages;           // [stages] the stage's MMAs have completed
    uint64_t* bar_accum = bars + 2 * kLmuStages;       // all MMAs have completed
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(reinterpret_cast<unsigned char*>(bars) + ((8 * LmUmmaSmem::n_bars + 15) & ~15));
    float* s_sx = reinterpret_cast<float*>(tmem_slot + 4);   // [kLmuMaxN]

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int tile = blockIdx.x, seq0 = blockIdx.y * kLmuMaxN;
    const int n_chunks = L.hidden / kLmuKc;

    if (tid == 0) {
        for (int s = 0; s < kLmuStages; ++s) {
            mbar_init(&bar_full[s], 1);
            mbar_init(&bar_empty[s], 1);
        }
        mbar_init(bar_accum, 1);
        mbar_init_fence();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(tmem_slot)), "r"(L.tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);
    if (L.use_pdl) {
        pdl_wait();
        pdl_launch_dependents();
    }
    for (int i = tid; i < N; i += kLmuThreads) s_sx[i] = seq0 + i < L.batch ? __ldcg(L.sx + seq0 + i) : 0.0f;
    __syncthreads();
    bool timed_out = false;

    if (warp == 0) {
        if (lane == 0) {
            for (int j = 0; j < n_chunks; ++j) {
                const int s = j % kLmuStages, use = j / kLmuStages;
                if (use > 0 && !mbar_spin_bounded(&bar_empty[s], (unsigned)(use - 1) & 1u)) { timed_out = true; break; }
                unsigned char* st = stages + (size_t)s * stage_bytes;
                mbar_expect_tx(&bar_full[s], (unsigned)stage_bytes);
                tma_load_2d(st, &wmap, j * kLmuKc, tile * kLmuRows, &bar_full[s]);
                tma_load_2d(st + kLmuRows * kLmuKc, &amap, j * kLmuKc, seq0, &bar_full[s]);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // c = s32, a = s8, b = s8, both K-major, N at bit 17 (>>3), M at bit 24 (>>4)
            const uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(kLmuRows >> 4) << 24);
            for (int j = 0; j < n_chunks; ++j) {
                const int s = j % kLmuStages, use = j / kLmuStages;
                if (!mbar_spin_bounded(&bar_full[s], (unsigned)use & 1u)) { timed_out = true; break; }
                tc_fence_after();
                const uint32_t sa = smem_addr(stages + (size_t)s * stage_bytes);
                const uint64_t da = umma_desc_sw128(sa), db = umma_desc_sw128(sa + kLmuRows * kLmuKc);
#pragma unroll
                for (int k4 = 0; k4 < kLmuKc / 32; ++k4)
                    umma_i8(tmem_base, da + (uint64_t)(2 * k4), db + (uint64_t)(2 * k4), idesc, (j > 0 || k4 > 0) ? 1u : 0u);
                umma_commit(&bar_empty[s]);
            }
            umma_commit(bar_accum);
        }
    } else {
        // ---- epilogue: TMEM lane = vocabulary row ----------------------------------------------------
        bool ok = true;
        if (lane == 0) ok = mbar_spin_bounded(bar_accum, 0u);
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) timed_out = true;
        tc_fence_after();
        const int q = warp & 3;
        const int row = 32 * q + lane, v = tile * kLmuRows + row;
        const float vscale = v < L.vocab ? __ldg(L.row_scales + v) : 0.0f;
        float* s_out = reinterpret_cast<float*>(stages);        // [N][128] logits of this tile
        for (int c0 = 0; c0 < N; c0 += 16) {
            uint32_t r[16];
            if (ok) tmem_ld16(tmem_base + ((uint32_t)(32 * q) << 16) + (uint32_t)c0, r);
            float sx[16];
#pragma unroll
            for (int i = 0; i < 16; i += 4) {
                const float4 t = *reinterpret_cast<const float4*>(s_sx + c0 + i);
                sx[i] = t.x; sx[i + 1] = t.y; sx[i + 2] = t.z; sx[i + 3] = t.w;
            }
#pragma unroll
            for (int i = 0; i < 16; ++i) s_out[(c0 + i) * kLmuRows + row] = (float)(int)r[i] * (sx[i] * vscale);   // :1717
            if (L.acc_out && ok && v < L.vocab) {
#pragma unroll
                for (int i = 0; i < 16; ++i)
                    if (seq0 + c0 + i < L.batch) L.acc_out[(size_t)(seq0 + c0 + i) * L.vocab + v] = (int)r[i];
            }
        }
        fence_proxy_async_smem();
        named_barrier_sync(1, 128);
        const int et = tid - 64;                                 // 0..127
        if (et == 0 && ok && L.logits) {
            asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];"
                         ::"l"(&omap), "r"(tile * kLmuRows), "r"(seq0), "r"(smem_addr(s_out)) : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
        if (L.cand && ok) {
            // thread et takes sequences et and et + 128; it walks the 128 rows starting at row et so that a
            // warp's lanes hit 32 different banks; "first maximum wins" is decided by index, not by visiting order
            for (int sidx = et; sidx < N; sidx += 128) {
                const int seq = seq0 + sidx;
                if (seq >= L.batch) break;
                LmBest b = {-INFINITY, 0x7fffffff};
                const float* col = s_out + (size_t)sidx * kLmuRows;
#pragma unroll 8
                for (int k = 0; k < kLmuRows; ++k) {
                    const int rr = (k + et) & (kLmuRows - 1), idx = tile * kLmuRows + rr;
                    const float val = col[rr];
                    if (idx < L.vocab && better(val, idx, b.val, b.idx)) { b.val = val; b.idx = idx; }
                }
                if (tile == 0 && col[0] != col[0]) { b.val = INFINITY; b.idx = 0; }   // a NaN at index 0 is never displaced (:1747-1753)
                L.cand[(size_t)seq * L.n_tiles + tile] = b;
            }
        }
        if (et == 0 && ok && L.logits) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // the tile has left shared memory
    }
    if (timed_out) atomicExch(&g_lmu_timeouts, 1);
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(L.tmem_cols) : "memory");
    }
}

bool lm_head_umma_applicable(int vocab, int hidden, int batch, const int8_t* w, const float* logits) {
    return batch >= 16 && hidden % kLmuKc == 0 && hidden >= kLmuKc && vocab % 4 == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0 &&
           (reinterpret_cast<uintptr_t>(logits) & 15) == 0 && (vocab + kLmuRows - 1) / kLmuRows <= kLmuMaxTiles;
}

// q8 [batch][hidden] int8 and sx [batch] already produced on `st`; cand holds batch * n_tiles entries.
int launch_lm_head_umma(const int8_t* q8, const float* sx, const int8_t* w, const float* row_scales, int vocab, int hidden, int batch,
                        float* logits, int32_t* acc_out, LmBest* cand, int use_pdl, cudaStream_t st) {
    LmUmmaLaunch L;
    L.sx = sx; L.row_scales = row_scales; L.logits = logits; L.acc_out = acc_out; L.cand = cand;
    L.vocab = vocab; L.hidden = hidden; L.batch = batch;
    L.n_tiles = (vocab + kLmuRows - 1) / kLmuRows;
    const int per_cta = batch < kLmuMaxN ? batch : kLmuMaxN;
    L.n_box = (per_cta + 15) & ~15;
    L.tmem_cols = 32;
    while (L.tmem_cols < L.n_box) L.tmem_cols *= 2;
    L.use_pdl = use_pdl;
    CUtensorMap wmap, amap, omap;
    if (int rc = encode_2d(&wmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, w, (uint64_t)hidden, (uint64_t)vocab, (uint64_t)hidden, kLmuKc, kLmuRows,
                           CU_TENSOR_MAP_SWIZZLE_128B)) return rc;
    if (int rc = encode_2d(&amap, CU_TENSOR_MAP_DATA_TYPE_UINT8, q8, (uint64_t)hidden, (uint64_t)batch, (uint64_t)hidden, kLmuKc, (uint32_t)L.n_box,
                           CU_TENSOR_MAP_SWIZZLE_128B)) return rc;
    // the store map is encoded on the logits when present, else on any valid address (it is then never used)
    const void* obase = logits ? static_cast<const void*>(logits) : static_cast<const void*>(w);
    if (int rc = encode_2d(&omap, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, obase, (uint64_t)vocab, (uint64_t)batch, (uint64_t)vocab * 4, kLmuRows,
                           (uint32_t)L.n_box, CU_TENSOR_MAP_SWIZZLE_NONE)) return rc;
    const size_t smem = LmUmmaSmem::bytes(L.n_box);
    cudaError_t e = cudaFuncSetAttribute(lm_head_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)L.n_tiles, (unsigned)((batch + kLmuMaxN - 1) / kLmuMaxN), 1);
    cfg.blockDim = dim3(kLmuThreads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = use_pdl ? 1 : 0;
    e = cudaLaunchKernelEx(&cfg, lm_head_umma_kernel, L, wmap, amap, omap);
    return e == cudaSuccess ? 0 : (int)e;
}

int lm_head_umma_take_timeouts() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_lmu_timeouts, sizeof v) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(g_lmu_timeouts, &zero, sizeof zero);
    return v;
}

}  // namespace tz
