/* tenzo_kernels.h — flat C entry points, one per CUDA kernel of the quantized decode path.
 *
 * These are the device-pointer calls that sit underneath the engine ABI (tenzo.h) and the
 * tenzo::CUDARuntime backend class. Every pointer is a CUDA device pointer unless the name ends
 * in _host; `stream` is a cudaStream_t passed as void* (NULL = default stream). Calls enqueue
 * work and return without synchronising. Return value: 0 on success, a negative tenzo_status_t
 * value (tenzo.h) on bad arguments, or a positive cudaError_t if the launch failed.
 *
 * All kernels are sm_100a only; there is no CPU or other-backend fallback.
 *
 * Each entry names the reference code it replaces (paths inside catdlia/tenzo).
 */
#ifndef TENZO_KERNELS_H
#define TENZO_KERNELS_H
#include <stddef.h>
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

#ifndef TENZO_API
#define TENZO_API __attribute__((visibility("default")))
#endif

/* ---- TL1 ternary GEMV with fused RMSNorm + absmax(31) quantiser ------------------------------
 * Replaces rms_norm_raw + build_lut + compute_single_block / compute_from_lut
 * (src/runtime/TenzoEngine.cpp:22-166) and the three call shapes that use them: the fused QKV
 * loop (:1547-1572), the fused gate/up loop + squared-ReLU GLU (:1593-1620), and the single
 * projections with residual add (:1585-1590, :1624-1628).
 *
 * Weights are the reference's own TL1 layout: [n_blocks][K/2][32 bytes]; byte c of a 32-byte
 * group carries row 64b+c (low nibble) and row 64b+32+c (high nibble) for columns (2k, 2k+1),
 * nibble = (w0+1)|((w1+1)<<2). K must be even, the weight pointer 16-byte aligned.
 *
 * Per sequence s in [0,batch):
 *   y   = do_norm ? x*(1/sqrt(mean(x^2)+eps))*norm_w : x                       (fp32)
 *   m   = max(1e-6, max|y|);  a_k = round(y_k*(31/m));  inv = m/31              (exact)
 *   acc_r = sum_k w[r][k]*a_k                                                    (int32, exact)
 *   v_r = (float)acc_r * (inv * scale_of_row_block)
 *   epilogue 0: out[r] = v_r
 *   epilogue 1: out[r] = resid[r] + v_r
 *   epilogue 2: rows [0,N/2) are gate, [N/2,N) up: out[r] = max(0,v_r)^2 * v_{r+N/2}, r < N/2
 */
enum { TENZO_EPI_STORE = 0, TENZO_EPI_RESIDUAL = 1, TENZO_EPI_RELU2_GLU = 2 };

typedef struct {
    const float* x;        /* [batch][x_stride] input activations */
    const float* norm_w;   /* [K] RMSNorm weight or NULL */
    int do_norm;
    float eps;             /* reference uses 1e-5 */
    const uint8_t* w;      /* TL1-packed weights, n_blocks*K/2*32 bytes */
    int n_blocks;          /* N/64 */
    int K;
    int seg_end[3];        /* row blocks [0,seg_end[0]) use seg_scale[0], [seg_end[0],seg_end[1]) ... */
    float seg_scale[3];    /* per-tensor weight scales (q/k/v or gate/up packed back to back) */
    int epilogue;
    const float* resid;    /* [batch][out_stride], epilogue 1 only */
    float* out;            /* [batch][out_stride] */
    int32_t* acc_out;      /* optional [batch][n_blocks*64] raw accumulators (parity checks) */
    int8_t* a_out;         /* optional [batch][K] quantised activations */
    float* inv_out;        /* optional [batch] m/31 */
    int batch;
    int x_stride, out_stride;
    const void* prefetch;  /* optional: memory the NEXT kernel in the stream will read (e.g. the next
                              layer's weights); requested into L2 while this kernel runs */
    size_t prefetch_bytes;
    void* workspace;       /* batch > 1 only: tenzo_cuda_tl1_gemv_workspace_bytes(batch, K) bytes, 16-byte
                              aligned; receives the packed int8 activations (contents need not be kept) */
    int use_pdl;           /* launch with programmatic stream serialisation (weights prefetch
                              overlaps the previous kernel's tail); 0 = ordinary launch */
} tenzo_tl1_gemv_args;

TENZO_API int tenzo_cuda_tl1_gemv(const tenzo_tl1_gemv_args* args, void* stream);
/* Cluster size along K (1, 2, 4 or 8 CTAs share one row block) the launcher picks for this shape; informational. */
TENZO_API int tenzo_cuda_tl1_gemv_ksplit(int n_blocks, int K, int epilogue);
/* 16 or more sequences (tensor-core path): CTAs of a thread-block cluster that share one 128-row tile's K range
 * (1, 2, 4 or 8; more than 1 when the row tiles alone would leave most SMs idle); 0 if that path does not take the
 * shape. Informational. */
TENZO_API int tenzo_cuda_tl1_gemm_ksplit(int n_blocks, int K, int batch, int epilogue);
/* The tensor-core path's per-CTA layout for `batch` sequences (what a CTA holds: min(batch, 256) padded to 16):
 * ring slots (a multiple of four), groups of eight weight chunks in flight, dynamic shared memory in bytes, and the
 * bytes the epilogue may need in the two rings. Host arithmetic only (no device call); returns 0, or -1 for
 * batch < 16. Informational; no counterpart in the reference. */
TENZO_API int tenzo_cuda_tl1_gemm_layout(int batch, int* slots, int* weight_groups, size_t* smem_bytes, size_t* epilogue_bytes);
TENZO_API size_t tenzo_cuda_tl1_gemv_workspace_bytes(int batch, int K);
/* The kernel's waits on asynchronous copies are bounded. Returns 1 (and clears the flag) if any launch
 * since the last call gave up waiting — its output is then invalid; 0 otherwise; -1 if the query failed.
 * Synchronises with the device. */
TENZO_API int tenzo_cuda_tl1_gemv_take_timeouts(void);
/* Test aid: launches a tiny kernel whose wait on a copy that is never issued runs out (after 2^8 polls), so that the flag
 * above is raised exactly as a real give-up raises it, without any fault or hang (the kernel finishes normally). Lets a
 * host exercise its own handling of the failure: the next tenzo_cuda_tl1_gemv_take_timeouts() returns 1, and an engine
 * call that checks the flags fails with its documented status. */
TENZO_API int tenzo_cuda_selftest_wait_expiry(void* stream);

/* ---- standalone fused RMSNorm + per-token absmax quantiser ------------------------------------
 * Replaces rms_norm_raw (:148-166) followed by the quantiser half of build_lut (:27-42,
 * qmax = 31) or of compute_logits (:1666-1678, qmax = 127: floor 1e-8, scale = amax/127,
 * q = clamp(round(y*(1/scale)))). y_out / q_out / scale_out are each optional.
 * scale_out receives m/31 (qmax 31) or amax/127 (qmax 127). */
TENZO_API int tenzo_cuda_rmsnorm_quant(const float* x, const float* norm_w, int do_norm, float eps, int dim,
                                       int qmax, int batch, int x_stride, float* y_out, int8_t* q_out,
                                       float* scale_out, void* stream);

/* ---- fused RoPE + INT8 KV append + GQA decode attention ---------------------------------------
 * Replaces FusedKVCache::forward_attention_raw in int8_fused mode (:447-533, :657-694, :823-851,
 * :911-913). Cache layout per sequence is the reference's: K,V int8 [layer][kv_head][max_seq][128],
 * scales fp32 [layer][kv_head][max_seq]; sequences are seq_stride_* apart. pos[s] is the slot the
 * new token is written to (= tokens already cached); attention then covers pos[s]+1 keys.
 * rope_cos/sin: [max_seq][head_dim/2] tables (built on the host with the reference's float
 * expressions so rotations are bit-identical); NULL skips RoPE. head_dim must be 128.
 * The kernel reproduces the reference's fp32 operation order (sequential sums over t, glibc expf
 * bits), so its output is bit-identical, not merely close. No scratch memory: score vectors live
 * in shared memory, which bounds max_len at 36864 keys. */
typedef struct {
    const float* q;        /* [batch][q_stride]  n_q*128 used, pre-RoPE */
    const float* k;        /* [batch][kv_stride] n_kv*128 used, pre-RoPE new key */
    const float* v;        /* [batch][kv_stride] n_kv*128 used, new value */
    float* out;            /* [batch][n_q*128] */
    int q_stride, kv_stride; /* floats between sequences; 0 = dense (n_q*128 / n_kv*128) */
    int8_t* cache_k; int8_t* cache_v; float* scale_k; float* scale_v;
    size_t seq_stride_kv;  /* elements between sequences in cache_k/v */
    size_t seq_stride_sc;  /* elements between sequences in scale_k/v */
    const int* pos;        /* [batch] device */
    const float* rope_cos; const float* rope_sin;
    int layer, n_q, n_kv, head_dim, max_seq, batch;
    int max_len;           /* upper bound on pos[s]+1 for this launch (sizes the grid) */
    int append;            /* 1: quantise and store the new k,v at pos (normal decode); 0: the
                              cache already holds pos[s]+1 keys, k/v are ignored */
    int heads_per_cta;     /* 0 = choose automatically; 1, 2, 4 or 8 forces the query heads one CTA processes */
    int use_pdl;           /* launch with programmatic stream serialisation. The kernel launched immediately before must
                              then write none of pos, rope_cos / rope_sin or the cache rows below pos[s]: with the contiguous
                              cache and few items those are read before the wait for that kernel (q, k, v are read after) */
    int tiles;             /* 0 = choose automatically; 1 = force the variant whose scoring warps read K through TMA tiles
                              (two keys per lane; for many (sequence, kv head) items; returns -5 if it does not fit:
                              needs four 16 KB tile rings beside the weights, n_q/n_kv <= 4 heads per CTA, cache_k and
                              seq_stride_kv 16-byte aligned); 2 = force per-lane global loads */
    /* kv_mode "paged_int8" (PagedKVCache of the reference, TenzoEngine.cpp:220-445, TenzoEngine.h:154-193). A non-NULL
     * block_table selects it: cache_k/cache_v are then the block pools int8 [block][n_layers][kv_head][16][128] and
     * scale_k/scale_v fp32 [block][n_layers][kv_head][16]; token t of sequence s lives in block
     * block_table[s*table_stride + t/16], slot t%16 (the entry for pos[s]/16 must exist before the call); seq_stride_*
     * are ignored. The arithmetic is that of PagedKVCache::forward_attention_raw, which is not the contiguous cache's
     * (two sets of eight FMA lanes, (dot*s_k)*scale, 1/(sum+1e-8), weights under 1e-7 dropped); outputs are
     * bit-identical to it. */
    const int* block_table; /* device */
    int table_stride;       /* ints between the tables of consecutive sequences; 0 = all query rows share one table */
    int n_layers;
    int n_pool_blocks;      /* blocks in the pools; 0 = not given, which rules out the TMA-tile variant (tiles == 1 then
                               returns -5): its tensor map needs the pool's extent */
    /* mode 0 (default): the reference's fp32 operation order, bit-identical outputs (above).
     * mode 1: tolerance mode. Same function, free evaluation order: the keys of a sequence are split over CTAs and
     * warps (online softmax, partials merged by log-sum-exp), both products run as fp16 tensor-core MMAs with fp32
     * accumulation (INT8 K/V are exact in fp16; the rotated query and the weights are rounded to fp16), exp is the
     * hardware ex2. Outputs agree with mode 0 to about 1e-4 of the output's largest magnitude (the specification asks
     * 1e-3 for floating-point outputs); the cache bytes written for the new token are identical in both modes.
     * Contiguous cache only (block_table must be NULL), 16-byte aligned caches, scales and out, max_seq a multiple of 4;
     * returns -5 otherwise. */
    int mode;
    int split_keys;         /* mode 1: keys per CTA (rounded up to 128); 0 = choose automatically */
    void* workspace;        /* mode 1: tenzo_cuda_attention_workspace_bytes(...) bytes, 16-byte aligned, for the partial
                               results of the splits (contents need not be kept) */
    size_t workspace_bytes;
} tenzo_attention_args;

TENZO_API int tenzo_cuda_attention_int8(const tenzo_attention_args* args, void* stream);
/* As tenzo_cuda_tl1_gemv_take_timeouts, for the attention kernel's bounded waits on its V-chunk copies (1). Also
 * returns 2 when a launch found a pos[s] outside [0, max_len): that CTA wrote nothing. */
TENZO_API int tenzo_cuda_attention_take_timeouts(void);
/* Scratch bytes mode 1 may need for these sizes (an upper bound over every split it can choose). */
TENZO_API size_t tenzo_cuda_attention_workspace_bytes(int batch, int n_q, int n_kv, int max_len);
/* Query heads one CTA will process for this shape (1..n_q/n_kv); informational. */
TENZO_API int tenzo_cuda_attention_heads_per_cta(int batch, int n_q, int n_kv, int max_len);

/* ---- INT8 LM head GEMV with fused final RMSNorm + absmax(127) quantiser + argmax --------------
 * Replaces compute_logits' int8 branch (:1634-1638, :1661-1719) and the greedy branch of
 * sample_top_k_top_p (:1745-1755: first maximum wins). logits/argmax_out/acc_out optional.
 * scratch: tenzo_cuda_lm_head_scratch_bytes(batch) bytes, 16-byte aligned. With 16 or more sequences, hidden a
 * multiple of 128 and vocab <= 262144 the product runs on the tensor cores (tcgen05 kind::i8): the activations are
 * normalised and quantised once, the vocabulary matrix is read once for all sequences; results are identical. */
TENZO_API int tenzo_cuda_lm_head_i8(const float* x, const float* norm_w, int do_norm, float eps,
                                    const int8_t* w, const float* row_scales, int vocab, int hidden,
                                    int batch, int x_stride, float* logits, int32_t* acc_out,
                                    int* argmax_out, void* scratch, int use_pdl, void* stream);
TENZO_API size_t tenzo_cuda_lm_head_scratch_bytes(int batch);
/* As tenzo_cuda_tl1_gemv_take_timeouts, for the bounded waits of the tensor-core LM head (16 or more sequences). */
TENZO_API int tenzo_cuda_lm_head_take_timeouts(void);

/* ---- LM head without any allocation -------------------------------------------------------------
 * No counterpart in the reference. Same computation and results as tenzo_cuda_lm_head_i8, for
 * callers that are not allowed to allocate device memory while running (a server whose memory is
 * fully committed to its KV pool, a host application that bans cudaMalloc after start-up): the
 * argmax scratch is a fixed array inside the library (151,552 bytes held on each GPU that loads the
 * library, for the life of the process) instead of a caller-provided buffer, and the call performs
 * no cudaMalloc/cudaFree or other allocating routine.
 *   - batch <= tenzo_cuda_lm_head_static_max_batch() (32); larger batches return
 *     TENZO_ERROR_UNSUPPORTED (-5) and should use tenzo_cuda_lm_head_i8 with their own scratch.
 *   - The first call on each device looks up the array's device address (the device must be
 *     current); make that first call before starting any stream capture.
 *   - All calls on a device share the one array. It is fully rewritten by every call, so nothing
 *     needs clearing, but two calls that overlap on the GPU (different streams) would race on it:
 *     keep calls on one stream or otherwise ordered. */
TENZO_API int tenzo_cuda_lm_head_i8_static(const float* x, const float* norm_w, int do_norm, float eps,
                                           const int8_t* w, const float* row_scales, int vocab, int hidden,
                                           int batch, int x_stride, float* logits, int32_t* acc_out,
                                           int* argmax_out, int use_pdl, void* stream);
TENZO_API int tenzo_cuda_lm_head_static_max_batch(void);

/* ---- Sampling support: repetition penalty and top-k candidate selection on the device ----------------
 * Replaces the first half of sample_top_k_top_p (:1735-1768). tenzo_cuda_repetition_penalty applies
 * l > 0 ? l / penalty : l * penalty to logits[tokens[i]], counts[i] times (tokens distinct).
 * tenzo_cuda_topk_candidates finds the k-th largest logit v* (three-pass radix select, one CTA) and writes every
 * (value, index) with value >= v* in ascending index order: *count gets their number; values/indices (each
 * tenzo_cuda_topk_max_candidates() entries) are written only if it does not exceed that capacity. Running the
 * reference's streaming top-k over these candidates gives the same heap as over the whole vector. */
TENZO_API int tenzo_cuda_repetition_penalty(float* logits, int vocab, const int* tokens, const int* counts, int n, float penalty, void* stream);
TENZO_API int tenzo_cuda_topk_candidates(const float* logits, int vocab, int k, int* count, float* values, int* indices, void* stream);
TENZO_API int tenzo_cuda_topk_max_candidates(void);

/* ---- INT8 embedding row dequantisation ---------------------------------------------------------
 * Replaces embedding_lookup's int8 branch (:1299-1315): x = (float)W8[tok] * scale[tok].
 * vocab > 0: token ids outside [0, vocab) are read as row 0 rather than past the table; 0 = unchecked. */
TENZO_API int tenzo_cuda_embedding_i8(const int8_t* w, const float* row_scales, int hidden,
                                      const int* tokens, int batch, float* x, int x_stride, int vocab, void* stream);

/* ---- checkpoint rows -> TL1 layout --------------------------------------------------------------
 * Replaces pack_ternary_weights_raw (:1842-1884): raw [N/4][K] bytes (row r in bits 2*(r%4)) to
 * the [N/64][K/2][32] layout above. */
TENZO_API int tenzo_cuda_tl1_pack_rows2bit(const uint8_t* raw, int N, int K, uint8_t* packed, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* TENZO_KERNELS_H */
