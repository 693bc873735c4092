/* CPU oracle for the quantized decode path — TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 * See tenzo_oracle.h for scope and pinning. Citations are to src/runtime/TenzoEngine.cpp of the
 * reference unless another file is named.
 *
 * Build note: compiled as gnu11 with -mfma so that, like a stock reference build (gnu++17), the
 * compiler may contract the scalar sum-of-squares in ora_rms_norm; every other place where the
 * reference fuses a multiply-add does so through an explicit intrinsic and is an explicit fmaf here.
 */
#include "tenzo_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

static inline int clampi(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }
static inline float clampf(float v, float lo, float hi) { return v < lo ? lo : (v > hi ? hi : v); }

/* ------------------------------------------------------------------------------------------- */
/* TL1 packing                                                                                 */
/* ------------------------------------------------------------------------------------------- */

static inline uint8_t tl1_nibble(int w_even, int w_odd) {
    /* :50 and :1873 — (w0+1) | ((w1+1)<<2), giving {0,1,2,4,5,6,8,9,10}. */
    return (uint8_t)(((w_even + 1) | ((w_odd + 1) << 2)) & 0x0F);
}

void ora_tl1_pack(const int8_t* tern, int64_t N, int64_t K, uint8_t* packed) {
    const int64_t nb = N / 64, kh = K / 2;
    for (int64_t b = 0; b < nb; ++b)
        for (int64_t k = 0; k < kh; ++k) {
            uint8_t* g = packed + (b * kh + k) * 32;
            for (int c = 0; c < 32; ++c) {
                const int8_t* lo = tern + (b * 64 + c) * K + 2 * k;       /* row 64b+c     */
                const int8_t* hi = tern + (b * 64 + 32 + c) * K + 2 * k;  /* row 64b+32+c  */
                g[c] = (uint8_t)(tl1_nibble(lo[0], lo[1]) | (tl1_nibble(hi[0], hi[1]) << 4));
            }
        }
}

void ora_tl1_pack_from_rows2bit(const uint8_t* raw, int64_t N, int64_t K, uint8_t* packed) {
    /* :1854-1859 — weight (r,c) = ((raw[(r/4)*K + c] >> 2*(r%4)) & 3) - 1 */
    const int64_t nb = N / 64, kh = K / 2;
#define W2(r, c) ((int)((raw[((r) / 4) * K + (c)] >> (((r) % 4) * 2)) & 3) - 1)
    for (int64_t b = 0; b < nb; ++b)
        for (int64_t k = 0; k < kh; ++k) {
            uint8_t* g = packed + (b * kh + k) * 32;
            for (int c = 0; c < 32; ++c) {
                int64_t r0 = b * 64 + c, r1 = r0 + 32;
                g[c] = (uint8_t)(tl1_nibble(W2(r0, 2 * k), W2(r0, 2 * k + 1)) |
                                 (tl1_nibble(W2(r1, 2 * k), W2(r1, 2 * k + 1)) << 4));
            }
        }
#undef W2
}

void ora_tl1_unpack(const uint8_t* packed, int64_t N, int64_t K, int8_t* tern) {
    const int64_t nb = N / 64, kh = K / 2;
    for (int64_t b = 0; b < nb; ++b)
        for (int64_t k = 0; k < kh; ++k) {
            const uint8_t* g = packed + (b * kh + k) * 32;
            for (int c = 0; c < 32; ++c) {
                int lo = g[c] & 15, hi = g[c] >> 4;
                tern[(b * 64 + c) * K + 2 * k] = (int8_t)((lo & 3) - 1);
                tern[(b * 64 + c) * K + 2 * k + 1] = (int8_t)((lo >> 2) - 1);
                tern[(b * 64 + 32 + c) * K + 2 * k] = (int8_t)((hi & 3) - 1);
                tern[(b * 64 + 32 + c) * K + 2 * k + 1] = (int8_t)((hi >> 2) - 1);
            }
        }
}

/* ------------------------------------------------------------------------------------------- */
/* TL1 activation quantiser, LUT, GEMV                                                         */
/* ------------------------------------------------------------------------------------------- */

static float absmax_floor(const float* x, int64_t n, float floor_v) {
    float m = floor_v;
    for (int64_t i = 0; i < n; ++i) {
        float a = fabsf(x[i]);
        if (a > m) m = a;
    }
    return m;
}

float ora_act_quant31(const float* x, int64_t K, int8_t* a) {
    const float m = absmax_floor(x, K, 1e-6f);          /* :28-32 */
    const float to_q = 31.0f / m;                       /* :34    */
    for (int64_t k = 0; k < K; ++k) a[k] = (int8_t)(int16_t)roundf(x[k] * to_q); /* :41-42 */
    return m / 31.0f;                                   /* :35    */
}

float ora_build_lut(const float* x, int64_t K, int8_t* lut) {
    const float m = absmax_floor(x, K, 1e-6f);
    const float to_q = 31.0f / m;
    for (int64_t k = 0; k < K / 2; ++k) {
        int a0 = (int16_t)roundf(x[2 * k] * to_q), a1 = (int16_t)roundf(x[2 * k + 1] * to_q);
        int8_t* t = lut + k * 32;
        memset(t, 0, 32);                               /* :44 unused slots stay 0 */
        for (int w0 = -1; w0 <= 1; ++w0)
            for (int w1 = -1; w1 <= 1; ++w1) {
                int8_t v = (int8_t)clampi(w0 * a0 + w1 * a1, -128, 127); /* :52-53 */
                int idx = tl1_nibble(w0, w1);
                t[idx] = v;
                t[idx + 16] = v;                        /* :56 second 128-bit lane */
            }
    }
    return m / 31.0f;
}

void ora_tl1_gemv_lut(const int8_t* lut, const uint8_t* packed, int64_t N, int64_t K, int32_t* acc) {
    const int64_t nb = N / 64, kh = K / 2;
#pragma omp parallel for schedule(dynamic, 4)
    for (int64_t b = 0; b < nb; ++b) {
        const uint8_t* w = packed + b * kh * 32;
        int32_t a32[64];
        memset(a32, 0, sizeof a32);
        for (int64_t k0 = 0; k0 < kh; k0 += 64) {       /* :83-84 chunks of 64 pairs */
            int64_t k1 = k0 + 64 < kh ? k0 + 64 : kh;
            int16_t a16[64];
            memset(a16, 0, sizeof a16);
            for (int64_t k = k0; k < k1; ++k) {
                const int8_t* t = lut + k * 32;
                const uint8_t* g = w + k * 32;
                for (int c = 0; c < 32; ++c) {
                    /* :94-98 — pshufb picks within a 128-bit lane; both lanes hold the same table */
                    a16[c] = (int16_t)(a16[c] + t[g[c] & 15]);
                    a16[32 + c] = (int16_t)(a16[32 + c] + t[g[c] >> 4]);
                }
            }
            for (int r = 0; r < 64; ++r) a32[r] += a16[r]; /* :107-115 */
        }
        memcpy(acc + b * 64, a32, sizeof a32);
    }
}

float ora_bitlinear_tl1(const float* x, const uint8_t* packed, int64_t N, int64_t K, float w_scale,
                        float* out, int32_t* acc) {
    int8_t* lut = (int8_t*)malloc((size_t)(K / 2) * 32);
    int32_t* a = acc ? acc : (int32_t*)malloc((size_t)N * sizeof(int32_t));
    const float inv_act = ora_build_lut(x, K, lut);
    ora_tl1_gemv_lut(lut, packed, N, K, a);
    const float s = inv_act * w_scale;                  /* :1554 — product first, in fp32 */
    if (out)
        for (int64_t r = 0; r < N; ++r) out[r] = (float)a[r] * s; /* :118 */
    if (!acc) free(a);
    free(lut);
    return inv_act;
}

/* ------------------------------------------------------------------------------------------- */
/* norms and element-wise                                                                      */
/* ------------------------------------------------------------------------------------------- */

void ora_rms_norm(const float* x, const float* w, float* y, int dim, float eps) {
    float ss = 0.0f;
#pragma omp simd reduction(+ : ss)
    for (int i = 0; i < dim; ++i) ss += x[i] * x[i];    /* :149-153 */
    const float inv_rms = 1.0f / sqrtf((ss / (float)dim) + eps); /* :154 */
    if (w)
        for (int i = 0; i < dim; ++i) y[i] = x[i] * inv_rms * w[i]; /* :158 left to right */
    else
        for (int i = 0; i < dim; ++i) y[i] = x[i] * inv_rms;
}

void ora_relu2_glu(const float* gate, const float* up, float* act, int n) {
    for (int i = 0; i < n; ++i) {
        float r = gate[i] > 0.0f ? gate[i] : 0.0f;
        act[i] = (r * r) * up[i];
    }
}

/* ------------------------------------------------------------------------------------------- */
/* attention                                                                                   */
/* ------------------------------------------------------------------------------------------- */

void ora_rope_table(int pos, int head_dim, float theta, float* cos_out, float* sin_out) {
    for (int i = 0; i < head_dim / 2; ++i) {
        float freq = 1.0f / powf(theta, (float)(2 * i) / head_dim); /* :466 */
        float ang = (float)pos * freq;                              /* :467 */
        cos_out[i] = cosf(ang);
        sin_out[i] = sinf(ang);
    }
}

void ora_rope_apply(float* heads, int n_heads, int head_dim, const float* cos_t, const float* sin_t) {
    const int half = head_dim / 2;
    for (int h = 0; h < n_heads; ++h) {
        float* x = heads + (size_t)h * head_dim;
        for (int i = 0; i < half; ++i) {
            float x0 = x[i], x1 = x[i + half];
            float p0 = x1 * sin_t[i], p1 = x1 * cos_t[i];  /* the separately rounded products */
            x[i] = fmaf(x0, cos_t[i], -p0);                /* :475 fmsub */
            x[i + half] = fmaf(x0, sin_t[i], p1);          /* :476 fmadd */
        }
    }
}

float ora_kv_quant_row(const float* x, int head_dim, int8_t* q) {
    float amax = 1e-8f;
    for (int d = 0; d < head_dim; ++d) amax = fmaxf(amax, fabsf(x[d])); /* :517-521 */
    const float s = amax / 127.0f;                                        /* :522 */
    const float inv = 1.0f / s;                                           /* :527 */
    for (int d = 0; d < head_dim; ++d) q[d] = (int8_t)clampf(roundf(x[d] * inv), -128.0f, 127.0f);
    return s;
}

void ora_attention_int8(int layer, int pos, int n_q, int n_kv, int head_dim, int max_seq, float theta,
                        float* q, float* k, float* v, float* out,
                        int8_t* cache_k, int8_t* cache_v, float* scale_k, float* scale_v) {
    float cs[256], sn[256];
    ora_rope_table(pos, head_dim, theta, cs, sn);
    ora_rope_apply(q, n_q, head_dim, cs, sn);
    ora_rope_apply(k, n_kv, head_dim, cs, sn);

    for (int h = 0; h < n_kv; ++h) {                                   /* :508-533 */
        size_t row = ((size_t)layer * n_kv + h) * max_seq + pos;
        scale_k[row] = ora_kv_quant_row(k + (size_t)h * head_dim, head_dim, cache_k + row * head_dim);
        scale_v[row] = ora_kv_quant_row(v + (size_t)h * head_dim, head_dim, cache_v + row * head_dim);
    }

    const int T = pos + 1, group = n_q / n_kv;
    const float sm_scale = 1.0f / sqrtf((float)head_dim);             /* :660 */
#pragma omp parallel for schedule(dynamic, 2)
    for (int qh = 0; qh < n_q; ++qh) {
        const int kvh = qh / group;
        const size_t base = ((size_t)layer * n_kv + kvh) * max_seq;
        const float* qv = q + (size_t)qh * head_dim;
        float* p = (float*)malloc((size_t)T * sizeof(float));
        float mx = -1e30f;                                             /* :670 */
        for (int t = 0; t < T; ++t) {
            const int8_t* kr = cache_k + (base + t) * head_dim;
            float lane[8] = {0, 0, 0, 0, 0, 0, 0, 0};                 /* :682-688 eight FMA lanes */
            for (int d = 0; d < head_dim; d += 8)
                for (int j = 0; j < 8; ++j) lane[j] = fmaf(qv[d + j], (float)kr[d + j], lane[j]);
            float dot = (lane[0] + lane[1] + lane[2] + lane[3] + lane[4] + lane[5] + lane[6] + lane[7]) *
                        (scale_k[base + t] * sm_scale);                /* :691 */
            p[t] = dot;
            if (dot > mx) mx = dot;
        }
        float sum = 0.0f;                                              /* :824-830 */
        for (int t = 0; t < T; ++t) {
            p[t] = expf(p[t] - mx);
            sum += p[t];
        }
        const float inv = 1.0f / sum;
        for (int t = 0; t < T; ++t) p[t] *= inv;

        float* o = out + (size_t)qh * head_dim;
        for (int d = 0; d < head_dim; ++d) o[d] = 0.0f;
        for (int t = 0; t < T; ++t) {                                  /* :842-851 */
            const int8_t* vr = cache_v + (base + t) * head_dim;
            const float wgt = p[t] * scale_v[base + t];
            for (int d = 0; d < head_dim; ++d) o[d] = fmaf((float)vr[d], wgt, o[d]);
        }
        free(p);
    }
}

/* PagedKVCache::forward_attention_raw (:242-445). Not the int8_fused arithmetic with another address
 * map: the dot product runs in two sets of eight FMA lanes (elements d..d+7 and d+8..d+15 of every
 * 16, :371-381) added lane by lane (:382) and then left to right starting from 0.0f (:385-386), the
 * score is (dot * s_k) * (1/sqrt(hd)) (:388), the weights are e_t * (1/(sum + 1e-8f)) (:400-403)
 * and keys whose weight is below 1e-7f are skipped (:416). Pools are
 * [block][n_layers][kv_head][16][head_dim] (scales [..][16]); block_table[b] is the physical block
 * of tokens 16b..16b+15 and must already hold an entry for pos/16 (the reference takes one from its
 * free list at :294-300 when layer 0 reaches a new block). */
void ora_attention_paged_int8(int layer, int pos, int n_q, int n_kv, int head_dim, int n_layers, float theta,
                              float* q, float* k, float* v, float* out,
                              int8_t* pool_k, int8_t* pool_v, float* pool_sk, float* pool_sv,
                              const int32_t* block_table) {
    enum { BS = 16 };
    float cs[256], sn[256];
    ora_rope_table(pos, head_dim, theta, cs, sn);                      /* :250-289 */
    ora_rope_apply(q, n_q, head_dim, cs, sn);
    ora_rope_apply(k, n_kv, head_dim, cs, sn);

    const int slot = pos % BS;
    const int32_t new_blk = block_table[pos / BS];
    for (int h = 0; h < n_kv; ++h) {                                   /* :318-347 */
        size_t row = (((size_t)new_blk * n_layers + layer) * n_kv + h) * BS + slot;
        pool_sk[row] = ora_kv_quant_row(k + (size_t)h * head_dim, head_dim, pool_k + row * head_dim);
        pool_sv[row] = ora_kv_quant_row(v + (size_t)h * head_dim, head_dim, pool_v + row * head_dim);
    }

    const int T = pos + 1, group = n_q / n_kv;
    const float qk_scale = 1.0f / sqrtf((float)head_dim);             /* :352 */
#pragma omp parallel for schedule(dynamic, 2)
    for (int qh = 0; qh < n_q; ++qh) {
        const int kvh = qh / group;
        const float* qv = q + (size_t)qh * head_dim;
        float* p = (float*)malloc((size_t)T * sizeof(float));
        float mx = -1e30f;                                             /* :360 */
        for (int t = 0; t < T; ++t) {
            const size_t row = (((size_t)block_table[t / BS] * n_layers + layer) * n_kv + kvh) * BS + t % BS;
            const int8_t* kr = pool_k + row * head_dim;
            float a0[8] = {0, 0, 0, 0, 0, 0, 0, 0}, a1[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            for (int d = 0; d < head_dim; d += 16)                     /* :371-381 */
                for (int j = 0; j < 8; ++j) {
                    a0[j] = fmaf(qv[d + j], (float)kr[d + j], a0[j]);
                    a1[j] = fmaf(qv[d + 8 + j], (float)kr[d + 8 + j], a1[j]);
                }
            float dot = 0.0f;
            for (int j = 0; j < 8; ++j) dot += a0[j] + a1[j];          /* :382-386 */
            const float score = dot * pool_sk[row] * qk_scale;         /* :388 */
            p[t] = score;
            mx = mx > score ? mx : score;
        }
        float sum = 0.0f;                                              /* :395-403 */
        for (int t = 0; t < T; ++t) {
            p[t] = expf(p[t] - mx);
            sum += p[t];
        }
        const float inv = 1.0f / (sum + 1e-8f);
        for (int t = 0; t < T; ++t) p[t] *= inv;

        float* o = out + (size_t)qh * head_dim;
        for (int d = 0; d < head_dim; ++d) o[d] = 0.0f;
        for (int t = 0; t < T; ++t) {                                  /* :409-441 */
            if (p[t] < 1e-7f) continue;
            const size_t row = (((size_t)block_table[t / BS] * n_layers + layer) * n_kv + kvh) * BS + t % BS;
            const int8_t* vr = pool_v + row * head_dim;
            const float wgt = p[t] * pool_sv[row];
            for (int d = 0; d < head_dim; ++d) o[d] = fmaf(wgt, (float)vr[d], o[d]);
        }
        free(p);
    }
}

/* ------------------------------------------------------------------------------------------- */
/* embedding, LM head, sampler                                                                 */
/* ------------------------------------------------------------------------------------------- */

void ora_embedding_i8(const int8_t* w, const float* scales, int hidden, int tok, float* x) {
    const int8_t* row = w + (size_t)tok * hidden;
    const float s = scales[tok];
    for (int i = 0; i < hidden; ++i) x[i] = (float)row[i] * s;
}

float ora_act_quant127(const float* x, int n, int8_t* q) {
    const float amax = absmax_floor(x, n, 1e-8f);
    const float s = amax / 127.0f, inv = 1.0f / s;
    for (int i = 0; i < n; ++i) q[i] = (int8_t)clampf(roundf(x[i] * inv), -128.0f, 127.0f);
    return s;
}

void ora_lm_head_i8(const int8_t* x8, float s_x, const int8_t* w, const float* scales,
                    int vocab, int hidden, float* logits, int32_t* acc) {
#pragma omp parallel for schedule(dynamic, 1024)
    for (int v = 0; v < vocab; ++v) {
        const int8_t* row = w + (size_t)v * hidden;
        int32_t s = 0;
        for (int i = 0; i < hidden; ++i) s += (int32_t)x8[i] * (int32_t)row[i];
        if (acc) acc[v] = s;
        if (logits) logits[v] = (float)s * (s_x * scales[v]);         /* :1717 */
    }
}

void ora_quantize_rows_i8(const float* w, int rows, int cols, int8_t* q, float* scales) {
#pragma omp parallel for
    for (int r = 0; r < rows; ++r) {
        const float* x = w + (size_t)r * cols;
        float amax = 1e-8f;
        for (int i = 0; i < cols; ++i) amax = fmaxf(amax, fabsf(x[i]));
        const float s = amax / 127.0f, inv = 1.0f / s;
        scales[r] = s;
        for (int i = 0; i < cols; ++i)
            q[(size_t)r * cols + i] = (int8_t)clampf(roundf(x[i] * inv), -127.0f, 127.0f);
    }
}

/* (logit, index) pairs ordered as std::pair<float,int> orders them. */
static int pair_less(float la, int ia, float lb, int ib) { return la < lb || (!(lb < la) && ia < ib); }

int ora_sample(float* logits, int vocab, float temperature, float top_p, int top_k,
               float repetition_penalty, const int* past, int n_past, float u) {
    top_k = clampi(top_k, 1, 64);                                      /* :1731 */
    if (repetition_penalty != 1.0f && past && n_past > 0)              /* :1735-1743 */
        for (int i = 0; i < n_past; ++i) {
            int t = past[i];
            if (t >= 0 && t < vocab) {
                float l = logits[t];
                logits[t] = (l > 0.0f) ? (l / repetition_penalty) : (l * repetition_penalty);
            }
        }
    if (temperature <= 0.0f) {                                         /* :1745-1755 first max */
        int best = 0;
        float bv = logits[0];
        for (int i = 1; i < vocab; ++i)
            if (logits[i] > bv) { bv = logits[i]; best = i; }
        return best;
    }
    /* :1757-1775 — min-heap of top_k pairs; here a small array kept sorted descending. */
    float cl[64];
    int ci[64], n = 0;
    for (int i = 0; i < vocab; ++i) {
        float l = logits[i];
        if (n == top_k) {
            if (!(l > cl[n - 1])) continue;   /* :1764 strict compare against the smallest kept logit */
            --n;                              /* drop the smallest pair */
        }
        int p = n;
        while (p > 0 && pair_less(cl[p - 1], ci[p - 1], l, i)) { cl[p] = cl[p - 1]; ci[p] = ci[p - 1]; --p; }
        cl[p] = l; ci[p] = i; ++n;
    }
    float probs[64], sum = 0.0f;
    for (int i = 0; i < n; ++i) { probs[i] = expf((cl[i] - cl[0]) / temperature); sum += probs[i]; }
    for (int i = 0; i < n; ++i) probs[i] /= sum;
    float cum = 0.0f;
    int cut = n;
    for (int i = 0; i < n; ++i) { cum += probs[i]; if (cum >= top_p) { cut = i + 1; break; } }
    float sub = 0.0f;
    for (int i = 0; i < cut; ++i) sub += probs[i];
    for (int i = 0; i < cut; ++i) probs[i] /= sub;
    float acc = 0.0f;
    for (int i = 0; i < cut; ++i) { acc += probs[i]; if (u <= acc) return ci[i]; }
    return ci[0];
}

/* ------------------------------------------------------------------------------------------- */
/* whole engine                                                                                */
/* ------------------------------------------------------------------------------------------- */

struct ora_engine {
    ora_config c;
    ora_layer* L;
    const float* final_norm;
    const int8_t* lm_w;
    const float* lm_s;
    int8_t *ck, *cv;
    float *sk, *sv;
    int seq_len;
    float* buf[16];
    int8_t* x8;
    /* kv_mode "paged_int8" (:1218-1220): pools, block table, blocks handed out so far */
    int paged, total_blocks, n_table;
    int8_t *pk, *pv;
    float *psk, *psv;
    int32_t* table;
};

ora_engine* ora_engine_create(const ora_config* cfg) {
    ora_engine* e = (ora_engine*)calloc(1, sizeof *e);
    e->c = *cfg;
    if (e->c.rope_theta <= 0.0f) e->c.rope_theta = 10000.0f;
    e->L = (ora_layer*)calloc((size_t)cfg->layers, sizeof(ora_layer));
    size_t rows = (size_t)cfg->layers * cfg->n_kv * cfg->max_seq;
    e->ck = (int8_t*)calloc(rows * cfg->head_dim, 1);
    e->cv = (int8_t*)calloc(rows * cfg->head_dim, 1);
    e->sk = (float*)calloc(rows, sizeof(float));
    e->sv = (float*)calloc(rows, sizeof(float));
    int wide = cfg->hidden > cfg->ffn ? cfg->hidden : cfg->ffn;
    if (cfg->n_q * cfg->head_dim > wide) wide = cfg->n_q * cfg->head_dim;
    for (int i = 0; i < 15; ++i) e->buf[i] = (float*)calloc((size_t)wide, sizeof(float));
    e->buf[15] = (float*)calloc((size_t)cfg->vocab, sizeof(float));
    e->x8 = (int8_t*)calloc((size_t)wide, 1);
    return e;
}

void ora_engine_destroy(ora_engine* e) {
    if (!e) return;
    for (int i = 0; i < 16; ++i) free(e->buf[i]);
    free(e->x8); free(e->ck); free(e->cv); free(e->sk); free(e->sv); free(e->L);
    free(e->pk); free(e->pv); free(e->psk); free(e->psv); free(e->table); free(e);
}

/* kv_mode = "paged_int8": (max_seq+15)/16 blocks of 16 tokens (:1218), scales preset to 1 (:238-239).
 * The reference's free list hands out block 0, 1, 2, ... after every reset (TenzoEngine.h:128-141: filled
 * from total-1 down to 0 and popped from the back), so a counter restates it. */
void ora_engine_use_paged_kv(ora_engine* e) {
    const ora_config* c = &e->c;
    if (e->paged) return;
    e->paged = 1;
    e->total_blocks = (c->max_seq + 15) / 16;
    size_t rows = (size_t)e->total_blocks * c->layers * c->n_kv * 16;
    e->pk = (int8_t*)calloc(rows * c->head_dim, 1);
    e->pv = (int8_t*)calloc(rows * c->head_dim, 1);
    e->psk = (float*)malloc(rows * sizeof(float));
    e->psv = (float*)malloc(rows * sizeof(float));
    for (size_t i = 0; i < rows; ++i) e->psk[i] = e->psv[i] = 1.0f;
    e->table = (int32_t*)calloc((size_t)e->total_blocks + 1, sizeof(int32_t));
    e->n_table = 0;
}
void ora_engine_paged_kv(ora_engine* e, int8_t** k, int8_t** v, float** sk, float** sv, int32_t** table, int* n_table) {
    if (k) *k = e->pk;
    if (v) *v = e->pv;
    if (sk) *sk = e->psk;
    if (sv) *sv = e->psv;
    if (table) *table = e->table;
    if (n_table) *n_table = e->n_table;
}

void ora_engine_set_layer(ora_engine* e, int layer, const ora_layer* w) {
    if (layer < 0 || layer >= e->c.layers || !w) return;              /* :1258 silently ignored */
    e->L[layer] = *w;
}
void ora_engine_set_final_norm(ora_engine* e, const float* w) { e->final_norm = w; }
void ora_engine_set_lm_head_i8(ora_engine* e, const int8_t* w, const float* s) { e->lm_w = w; e->lm_s = s; }
void ora_engine_reset(ora_engine* e) { e->seq_len = 0; e->n_table = 0; }
int ora_engine_seq_len(const ora_engine* e) { return e->seq_len; }
float* ora_engine_buffer(ora_engine* e, int which) { return (which >= 0 && which < 16) ? e->buf[which] : NULL; }
void ora_engine_kv(ora_engine* e, int8_t** k, int8_t** v, float** sk, float** sv) {
    if (k) *k = e->ck;
    if (v) *v = e->cv;
    if (sk) *sk = e->sk;
    if (sv) *sv = e->sv;
}

enum { B_X, B_NORM, B_Q, B_K, B_V, B_ATT, B_ATTSUB, B_OUT, B_H1, B_POST, B_GATE, B_UP, B_ACT, B_FFNN, B_DOWN, B_LOGITS };

void ora_engine_embedding(ora_engine* e, int tok) {
    ora_embedding_i8(e->lm_w, e->lm_s, e->c.hidden, tok, e->buf[B_X]);
}

void ora_engine_forward_layer(ora_engine* e, int l) {                  /* :1538-1632 */
    const ora_config* c = &e->c;
    const ora_layer* w = &e->L[l];
    const int h = c->hidden, qd = c->n_q * c->head_dim, kvd = c->n_kv * c->head_dim, f = c->ffn;
    float** b = e->buf;

    ora_rms_norm(b[B_X], w->in_norm, b[B_NORM], h, 1e-5f);
    ora_bitlinear_tl1(b[B_NORM], w->q_w, qd, h, w->q_s, b[B_Q], NULL);
    ora_bitlinear_tl1(b[B_NORM], w->k_w, kvd, h, w->k_s, b[B_K], NULL);
    ora_bitlinear_tl1(b[B_NORM], w->v_w, kvd, h, w->v_s, b[B_V], NULL);

    if (e->paged) {
        if (e->seq_len / 16 >= e->n_table && e->n_table < e->total_blocks) {   /* :294-300 */
            e->table[e->n_table] = e->n_table;
            e->n_table += 1;
        }
        ora_attention_paged_int8(l, e->seq_len, c->n_q, c->n_kv, c->head_dim, c->layers, c->rope_theta,
                                 b[B_Q], b[B_K], b[B_V], b[B_ATT], e->pk, e->pv, e->psk, e->psv, e->table);
    } else {
        ora_attention_int8(l, e->seq_len, c->n_q, c->n_kv, c->head_dim, c->max_seq, c->rope_theta,
                           b[B_Q], b[B_K], b[B_V], b[B_ATT], e->ck, e->cv, e->sk, e->sv);
    }

    ora_rms_norm(b[B_ATT], w->attn_sub_norm, b[B_ATTSUB], h, 1e-5f);  /* :1582 uses hidden, not q_dim */
    ora_bitlinear_tl1(b[B_ATTSUB], w->o_w, h, h, w->o_s, b[B_OUT], NULL);
    for (int i = 0; i < h; ++i) b[B_H1][i] = b[B_X][i] + b[B_OUT][i];

    if (w->gate_w && w->up_w && w->down_w) {
        ora_rms_norm(b[B_H1], w->post_norm, b[B_POST], h, 1e-5f);
        ora_bitlinear_tl1(b[B_POST], w->gate_w, f, h, w->gate_s, b[B_GATE], NULL);
        ora_bitlinear_tl1(b[B_POST], w->up_w, f, h, w->up_s, b[B_UP], NULL);
        ora_relu2_glu(b[B_GATE], b[B_UP], b[B_ACT], f);
        ora_rms_norm(b[B_ACT], w->ffn_sub_norm, b[B_FFNN], f, 1e-5f);
        ora_bitlinear_tl1(b[B_FFNN], w->down_w, h, f, w->down_s, b[B_DOWN], NULL);
        for (int i = 0; i < h; ++i) b[B_X][i] = b[B_H1][i] + b[B_DOWN][i];
    } else {
        memcpy(b[B_X], b[B_H1], (size_t)h * sizeof(float));
    }
}

void ora_engine_advance(ora_engine* e) { e->seq_len += 1; }

void ora_engine_logits(ora_engine* e) {                                /* :1634-1720 int8 branch */
    const int h = e->c.hidden;
    ora_rms_norm(e->buf[B_X], e->final_norm, e->buf[B_NORM], h, 1e-5f);
    float s_x = ora_act_quant127(e->buf[B_NORM], h, e->x8);
    ora_lm_head_i8(e->x8, s_x, e->lm_w, e->lm_s, e->c.vocab, h, e->buf[B_LOGITS], NULL);
}

void ora_engine_prefill(ora_engine* e, int tok) {
    ora_engine_embedding(e, tok);
    for (int l = 0; l < e->c.layers; ++l) ora_engine_forward_layer(e, l);
    ora_engine_advance(e);
}

int ora_engine_generate(ora_engine* e, int tok, float temperature, float top_p, int top_k,
                        float repetition_penalty, const int* past, int n_past, float u) {
    ora_engine_prefill(e, tok);
    ora_engine_logits(e);
    return ora_sample(e->buf[B_LOGITS], e->c.vocab, temperature, top_p, top_k, repetition_penalty,
                      past, n_past, u);
}
