/* tenzo_ext.h — additive extension of the engine ABI (nothing in tenzo.h changes).
 *
 * The reference engine is one sequence, one token per call, RoPE base fixed at 10000
 * (src/runtime/TenzoEngine.cpp:456, :1809-1838) and exposes its KV arrays and scratch vectors
 * only as public C++ members (src/runtime/TenzoEngine.h:75-78, :216-230). Batched decode, a
 * configurable RoPE base, KV import/export and intermediate read-back need entry points it does
 * not have; they live here. An engine made by tenzo_ext_create_engine with batch == 1 behaves
 * exactly like one made by tenzo_create_engine.
 */
#ifndef TENZO_EXT_H
#define TENZO_EXT_H
#include "tenzo.h"
#ifdef __cplusplus
extern "C" {
#endif

typedef struct {
    int batch;          /* independent sequences decoded per step (>= 1) */
    float rope_theta;   /* <= 0 selects the reference's 10000 */
    int use_graph;      /* 1: replay each decode step as a CUDA graph; 0: plain launches; -1 default */
    int use_pdl;        /* 1: programmatic dependent launch between kernels; 0: off; -1 default */
    int persistent;     /* batch 1 only. 1: run each token as ONE persistent cooperative kernel (grid-wide barriers between
                           the operators, weights streamed ahead through shared memory) when the shapes allow it; 0: the
                           chain of one kernel per operator; -1 default (0, or the TENZO_PERSISTENT environment variable).
                           Results are bit-identical either way; on B200 the chain is the faster of the two (the barriers and
                           L2 round trips of the one-kernel form cost more than the launches they replace). */
    int attention_mode; /* 0: attention in the reference's fp32 operation order, bit-identical outputs (default; greedy
                           streams equal the reference's). 1: tolerance mode for the kernel-chain engine (see
                           tenzo_attention_args.mode in tenzo_kernels.h): split over the keys, tensor-core products, about
                           1e-4 relative on the attention output, several times faster at long contexts. -1 default (0, or
                           the TENZO_ATTENTION_MODE environment variable). Contiguous KV cache only. */
} tenzo_ext_options_t;

TENZO_API tenzo_ext_options_t tenzo_ext_default_options(void);
TENZO_API tenzo_engine_t tenzo_ext_create_engine(const tenzo_config_t* config, const tenzo_ext_options_t* opt);
TENZO_API int tenzo_ext_batch(tenzo_engine_t engine);

/* One token per sequence through all layers, no logits (batched tenzo_prefill_token). */
TENZO_API tenzo_status_t tenzo_ext_prefill_tokens(tenzo_engine_t engine, const int* tokens);
/* One decode step per sequence; greedy only (temperature <= 0, repetition_penalty == 1) when
 * batch > 1. out_tokens[batch] receives the sampled ids. */
TENZO_API tenzo_status_t tenzo_ext_generate_step(tenzo_engine_t engine, const int* cur_tokens,
                                                 const tenzo_sampling_params_t* params, int* out_tokens);
/* n_steps greedy decode steps with the token fed back on the device: no host round trip between
 * steps. out_tokens[n_steps][batch]. */
TENZO_API tenzo_status_t tenzo_ext_decode_greedy(tenzo_engine_t engine, const int* first_tokens, int n_steps,
                                                 int* out_tokens);

/* KV cache of one sequence and layer, host arrays k,v: [kv_heads][len][head_dim] int8 and
 * sk,sv: [kv_heads][len] fp32 — the reference's per-layer slice (TenzoEngine.cpp:509-510). */
TENZO_API tenzo_status_t tenzo_ext_kv_import(tenzo_engine_t engine, int seq, int layer, const int8_t* k,
                                             const int8_t* v, const float* sk, const float* sv, int len);
TENZO_API tenzo_status_t tenzo_ext_kv_export(tenzo_engine_t engine, int seq, int layer, int8_t* k, int8_t* v,
                                             float* sk, float* sv, int len);
/* Fill every layer of every sequence with the same device-generated pseudo-random int8 rows and
 * scales up to `len` tokens (benchmark prefill stand-in; values depend only on seed). */
TENZO_API tenzo_status_t tenzo_ext_kv_fill_random(tenzo_engine_t engine, int len, uint64_t seed);
TENZO_API tenzo_status_t tenzo_ext_set_seq_len(tenzo_engine_t engine, int seq, int len);
TENZO_API int tenzo_ext_get_seq_len(tenzo_engine_t engine, int seq);

/* Intermediate vectors of the most recent step, copied to host: */
enum {
    TENZO_BUF_X = 0,        /* residual stream after the last layer run   [hidden] */
    TENZO_BUF_Q = 2,        /* q projection, before RoPE                  [q_dim]  */
    TENZO_BUF_K = 3,        /* k projection, before RoPE                  [kv_dim] */
    TENZO_BUF_V = 4,        /* v projection                               [kv_dim] */
    TENZO_BUF_ATTN_OUT = 5, /* attention output                           [q_dim]  */
    TENZO_BUF_H1 = 8,       /* x + out projection                         [hidden] */
    TENZO_BUF_ACT = 12,     /* relu(gate)^2 * up                          [ffn]    */
    TENZO_BUF_LOGITS = 15   /* logits of the last generate step           [vocab]  */
};
TENZO_API tenzo_status_t tenzo_ext_read_buffer(tenzo_engine_t engine, int which, int seq, float* dst, size_t count);
/* Run single pieces of a step (teacher-forced checks): embedding, one layer, logits. */
TENZO_API tenzo_status_t tenzo_ext_write_x(tenzo_engine_t engine, int seq, const float* x);
TENZO_API tenzo_status_t tenzo_ext_run_layer(tenzo_engine_t engine, int layer);
TENZO_API tenzo_status_t tenzo_ext_synchronize(tenzo_engine_t engine);
/* Device time of the most recent step / decode_greedy call, from CUDA events on the engine's stream (ms). */
TENZO_API float tenzo_ext_last_device_ms(tenzo_engine_t engine);
/* Measurement aid: runs the engine's own TL1 matrices (q|k|v, out, gate|up, down of every layer,
 * in layer order, on the engine's activation buffers) `iters` times back to back with no attention
 * or LM head in between, and returns the CUDA-event time in ms (< 0 on failure). *launches
 * receives the number of GEMV kernels timed. */
TENZO_API float tenzo_ext_bench_gemv_stack(tenzo_engine_t engine, int iters, unsigned long long* launches);
/* Measurement aid for the persistent single-sequence kernel: nanoseconds (GPU global timer, read by one thread of the
 * first CTA at every grid-wide barrier) spent since the last reset in each phase kind - [0] norm + q|k|v product,
 * [1] attention, [2] out product, [3] gate|up product, [4] down product, [5] final norm + LM head, [6] argmax and exit.
 * Returns 1 and fills out8[8] when that kernel is in use, 0 when the engine runs the per-operator kernel chain, -1 on
 * failure. Synchronises with the engine's stream. */
TENZO_API int tenzo_ext_persistent_phase_ns(tenzo_engine_t engine, unsigned long long* out8, int reset);
/* Number of kernels launched (or replayed through a graph) since the engine was created. */
TENZO_API unsigned long long tenzo_ext_kernel_launches(tenzo_engine_t engine);
/* Message for the most recent failure on this thread ("" if none). */
/* Chunked prefill (single-sequence engines): feeds n consecutive prompt tokens through every layer together - the
 * TL1 layers as GEMMs over the n rows, causal attention as n queries over the one cache - instead of n calls of
 * tenzo_prefill_token (TenzoEngine.cpp:1809-1819, main_inference.cpp:469-474 of the reference). Cache contents, state
 * and every later token are bit-identical to the token-by-token path. */
TENZO_API tenzo_status_t tenzo_ext_prefill_chunk(tenzo_engine_t engine, const int* tokens, int n);

/* RoPE tables cos/sin [max_seq][head_dim/2] as the engine builds them (the reference's float expressions,
 * TenzoEngine.cpp:466-469), written to host memory: for callers that drive the per-kernel entry points
 * themselves (tensor-parallel decode) and need the same bits. */
TENZO_API tenzo_status_t tenzo_ext_rope_tables(int max_seq, int head_dim, float rope_theta, float* cos_host, float* sin_host);

/* The manifest reader of tenzo_load_model on its own (host only): byte offsets of the memref.view constants and the
 * f32 scale constants feeding "tenzo.bitlinear_elut", in order of appearance (TenzoEngine.cpp:1946-1963 of the
 * reference). Writes at most max_* entries; the counts found are always returned. */
TENZO_API int tenzo_ext_parse_manifest(const char* text, unsigned long long* views, int max_views, int* n_views,
                                       float* scales, int max_scales, int* n_scales);

/* The host half of the sampler on its own (no GPU needed): the reference's streaming top-k, softmax, top-p and draw
 * (TenzoEngine.cpp:1745-1806) over `n` (value, index) pairs given in ascending index order; indices NULL means 0..n-1
 * (a whole logit vector). r in [0,1] replaces rand()/RAND_MAX, r < 0 draws from rand(). The engine feeds it only the
 * logits at or above the k-th largest, selected on the device; the result equals a scan of the whole vector. */
TENZO_API int tenzo_ext_sample_pairs(const float* values, const int* indices, int n, const tenzo_sampling_params_t* params, float r);

TENZO_API const char* tenzo_ext_last_error(void);

#ifdef __cplusplus
}
#endif
#endif /* TENZO_EXT_H */
