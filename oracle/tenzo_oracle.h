/* CPU oracle for the quantized decode path — TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * A plain-C restatement of what the reference engine (src/runtime/TenzoEngine.cpp of
 * catdlia/tenzo) computes for one decoded token in its "cpu" device, int8_fused (or paged_int8) KV mode, with
 * TL1-packed ternary layers and an INT8 LM head. Every function names the reference lines it
 * follows. Only tests, the smoke check and the CPU-baseline leg of the benchmark may load this
 * library; the CUDA product never does.
 *
 * Pinning: the reference ships no golden vectors for this path, so this restatement is pinned
 * against the reference engine itself, compiled unmodified (oracle/Makefile target `ref`):
 * tests/test_oracle_vs_reference.py checks every function here against it on seeded inputs, and
 * tests/golden/ holds vectors produced by that compiled reference.
 *
 * One deliberate extension: rope_theta is a parameter (the reference hard-codes 10000,
 * TenzoEngine.cpp:456).
 */
#ifndef TENZO_ORACLE_H
#define TENZO_ORACLE_H
#include <stddef.h>
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

/* ---- TL1 weights --------------------------------------------------------------------------- */
/* tern[N][K] in {-1,0,1} -> packed[N/64][K/2][32]; byte c of a group: low nibble row 64b+c,
 * high nibble row 64b+32+c, nibble = (w[2k]+1) | ((w[2k+1]+1)<<2). TenzoEngine.cpp:1861-1881. */
void ora_tl1_pack(const int8_t* tern, int64_t N, int64_t K, uint8_t* packed);
/* Same target layout from the checkpoint form [N/4][K] (2 bits per weight, row r in bits
 * 2*(r%4) of byte (r/4, c), value-1). TenzoEngine.cpp:1842-1884. */
void ora_tl1_pack_from_rows2bit(const uint8_t* raw, int64_t N, int64_t K, uint8_t* packed);
/* Inverse of ora_tl1_pack (for round-trip tests). */
void ora_tl1_unpack(const uint8_t* packed, int64_t N, int64_t K, int8_t* tern);

/* ---- TL1 activation quantiser + GEMV -------------------------------------------------------- */
/* m = max(1e-6, max|x|); a_k = (int16)round(x_k * (31/m)); returns m/31. TenzoEngine.cpp:27-42. */
float ora_act_quant31(const float* x, int64_t K, int8_t* a);
/* The K/2 x 32-byte lookup tables exactly as build_lut lays them out. TenzoEngine.cpp:22-62. */
float ora_build_lut(const float* x, int64_t K, int8_t* lut /* [K/2][32] */);
/* acc[r] = sum_k lut_k[nibble(r,k)], int16 partials flushed every 64 pairs. :64-116. */
void ora_tl1_gemv_lut(const int8_t* lut, const uint8_t* packed, int64_t N, int64_t K, int32_t* acc);
/* x -> (acc, out = (float)acc * (inv_act * w_scale)); returns inv_act. :118-146, :1554. */
float ora_bitlinear_tl1(const float* x, const uint8_t* packed, int64_t N, int64_t K, float w_scale,
                        float* out, int32_t* acc /* may be NULL */);

/* ---- norms, element-wise ------------------------------------------------------------------- */
/* y = x * (1/sqrt(mean(x^2)+eps)) * w, w may be NULL. TenzoEngine.cpp:148-166. */
void ora_rms_norm(const float* x, const float* w, float* y, int dim, float eps);
/* act = max(0,g)^2 * u evaluated (r*r)*u. TenzoEngine.cpp:1616-1620. */
void ora_relu2_glu(const float* gate, const float* up, float* act, int n);

/* ---- attention ------------------------------------------------------------------------------ */
/* cos/sin for position pos: f = 1/powf(theta, 2i/head_dim), ang = (float)pos*f. :466-469. */
void ora_rope_table(int pos, int head_dim, float theta, float* cos_out, float* sin_out /* [hd/2] */);
/* r0 = fms(x0,c,x1*s), r1 = fma(x0,s,x1*c) on pairs (i, i+hd/2), in place. :471-478. */
void ora_rope_apply(float* heads, int n_heads, int head_dim, const float* cos_t, const float* sin_t);
/* amax = max(1e-8,max|x|); s = amax/127; q = clamp(round(x*(1/s)),-128,127). :517-532. */
float ora_kv_quant_row(const float* x, int head_dim, int8_t* q);
/* Full attention step of FusedKVCache::forward_attention_raw (int8_fused): RoPE q,k in place,
 * append k,v at slot pos, then softmax(QK)V over pos+1 keys. Cache layout
 * [layer][kv_head][max_seq][head_dim] / scales [layer][kv_head][max_seq]. :447-533, :657-694,
 * :823-851, :911-913. */
void ora_attention_int8(int layer, int pos, int n_q, int n_kv, int head_dim, int max_seq, float theta,
                        float* q, float* k, float* v, float* out,
                        int8_t* cache_k, int8_t* cache_v, float* scale_k, float* scale_v);

/* PagedKVCache::forward_attention_raw (kv_mode "paged_int8", :242-445): same RoPE and append, but the
 * pools are [block][n_layers][kv_head][16][head_dim] behind block_table, and the arithmetic differs
 * from int8_fused (two sets of eight FMA lanes, (dot*s_k)*scale, 1/(sum+1e-8), weights < 1e-7
 * skipped). block_table must already map logical block pos/16. */
void ora_attention_paged_int8(int layer, int pos, int n_q, int n_kv, int head_dim, int n_layers, float theta,
                              float* q, float* k, float* v, float* out,
                              int8_t* pool_k, int8_t* pool_v, float* pool_sk, float* pool_sv,
                              const int32_t* block_table);

/* ---- embedding, LM head, sampler ------------------------------------------------------------ */
/* x = (float)W8[tok] * scale[tok]. TenzoEngine.cpp:1299-1315. */
void ora_embedding_i8(const int8_t* w, const float* scales, int hidden, int tok, float* x);
/* amax = max(1e-8,..); s = amax/127; q = clamp(round(x*(1/s)),-128,127); returns s. :1666-1678. */
float ora_act_quant127(const float* x, int n, int8_t* q);
/* logit_v = (float)(sum x8*W8[v]) * (s_x * scale_v). :1688-1718. acc may be NULL. */
void ora_lm_head_i8(const int8_t* x8, float s_x, const int8_t* w, const float* scales,
                    int vocab, int hidden, float* logits, int32_t* acc);
/* Per-row absmax int8 quantisation of an fp32 table, clamp +-127. :1934-1946. */
void ora_quantize_rows_i8(const float* w, int rows, int cols, int8_t* q, float* scales);
/* Repetition penalty then greedy first-max, or top-k/top-p draw with u in [0,1] supplied by the
 * caller in place of rand()/RAND_MAX. Mutates logits like the reference. :1722-1807. */
int ora_sample(float* logits, int vocab, float temperature, float top_p, int top_k,
               float repetition_penalty, const int* past, int n_past, float u);

/* ---- whole engine --------------------------------------------------------------------------- */
typedef struct {
    int hidden, n_q, n_kv, head_dim, layers, ffn, vocab, max_seq;
    float rope_theta;
} ora_config;
typedef struct {
    const uint8_t *q_w, *k_w, *v_w, *o_w, *gate_w, *up_w, *down_w; /* TL1 packed */
    float q_s, k_s, v_s, o_s, gate_s, up_s, down_s;
    const float *in_norm, *attn_sub_norm, *post_norm, *ffn_sub_norm;
} ora_layer;
typedef struct ora_engine ora_engine;

ora_engine* ora_engine_create(const ora_config* cfg);
void ora_engine_destroy(ora_engine* e);
/* Pointers are borrowed, as in the reference (TenzoEngine.cpp:1257-1281). */
void ora_engine_set_layer(ora_engine* e, int layer, const ora_layer* w);
void ora_engine_set_final_norm(ora_engine* e, const float* w);
void ora_engine_set_lm_head_i8(ora_engine* e, const int8_t* w, const float* scales);
/* Switch a fresh engine to kv_mode "paged_int8" (:1218-1220, :1575-1576). */
void ora_engine_use_paged_kv(ora_engine* e);
void ora_engine_paged_kv(ora_engine* e, int8_t** k, int8_t** v, float** sk, float** sv, int32_t** table, int* n_table);
void ora_engine_reset(ora_engine* e);
int ora_engine_seq_len(const ora_engine* e);
void ora_engine_prefill(ora_engine* e, int tok);                       /* :1809-1819 */
int ora_engine_generate(ora_engine* e, int tok, float temperature, float top_p, int top_k,
                        float repetition_penalty, const int* past, int n_past, float u); /* :1821-1838 */
/* Intermediate buffers of the most recent layer/step, same numbering as the test shim:
 * 0 x, 1 norm_x, 2 q, 3 k, 4 v, 5 attn_out, 6 attn_sub, 7 out, 8 h1, 9 post_norm, 10 gate,
 * 11 up, 12 act, 13 ffn_norm, 14 down, 15 logits. */
float* ora_engine_buffer(ora_engine* e, int which);
void ora_engine_kv(ora_engine* e, int8_t** k, int8_t** v, float** sk, float** sv);
/* Single pieces, for teacher-forced tests. */
void ora_engine_embedding(ora_engine* e, int tok);
void ora_engine_forward_layer(ora_engine* e, int layer);
void ora_engine_advance(ora_engine* e);
void ora_engine_logits(ora_engine* e);

#ifdef __cplusplus
}
#endif
#endif
