// Test infrastructure only: a kernel-granular handle on the UNMODIFIED reference engine.
//
// The reference keeps its TL1 kernels (build_lut, compute_from_lut, rms_norm_raw) in an anonymous
// namespace of src/runtime/TenzoEngine.cpp, so the only way to call them without editing the
// reference is to compile that file as part of this translation unit. Nothing is copied: the
// #include below resolves through -I<reference>/src at build time (see oracle/Makefile, target
// _ref/libtenzo_ref_kernels.so). The resulting library also carries the reference's 14 C-API
// symbols, so one dlopen serves both whole-engine and per-kernel parity checks.
//
// Every export is a thin trampoline; no arithmetic happens in this file.
#include "runtime/TenzoEngine.cpp"

#include <cstdint>
#include <cstring>
#include <vector>

extern "C" {

// build_lut (TenzoEngine.cpp:22-62): fp32 activation -> K/2 x 32-byte tables; returns max|x|/31.
__attribute__((visibility("default")))
float refk_build_lut(const float* act, int64_t K, uint8_t* lut_bytes_out) {
    std::vector<tenzo::Vec256i> lut(K / 2);
    float inv = tenzo::build_lut(act, K, reinterpret_cast<__m256i*>(lut.data()));
    if (lut_bytes_out) std::memcpy(lut_bytes_out, lut.data(), static_cast<size_t>(K / 2) * 32);
    return inv;
}

// build_lut + compute_from_lut (TenzoEngine.cpp:129-146) for one N x K TL1 matrix.
// out_f32 = float(acc) * (inv_act * w_scale); acc_i32 (optional) comes from a second pass with
// total_scale = 1.0f, which is exact because |acc| < 2^24.
__attribute__((visibility("default")))
float refk_bitlinear_tl1(const float* act, const int8_t* packed_w, int64_t N, int64_t K,
                         float w_scale, float* out_f32, int32_t* acc_i32) {
    std::vector<tenzo::Vec256i> lut(K / 2);
    __m256i* lp = reinterpret_cast<__m256i*>(lut.data());
    float inv = tenzo::build_lut(act, K, lp);
    if (out_f32) tenzo::compute_from_lut(lp, packed_w, N / 64, K / 2, out_f32, inv * w_scale);
    if (acc_i32) {
        std::vector<float> tmp(N);
        tenzo::compute_from_lut(lp, packed_w, N / 64, K / 2, tmp.data(), 1.0f);
        for (int64_t i = 0; i < N; ++i) acc_i32[i] = static_cast<int32_t>(tmp[i]);
    }
    return inv;
}

// rms_norm_raw (TenzoEngine.cpp:148-166).
__attribute__((visibility("default")))
void refk_rms_norm(const float* src, const float* w, float* dst, int dim, float eps) {
    tenzo::rms_norm_raw(src, w, dst, dim, eps);
}

// FusedKVCache in int8_fused mode (TenzoEngine.h:60-115); arrays are public members.
__attribute__((visibility("default")))
void* refk_kv_create(int layers, int q_heads, int kv_heads, int head_dim, int max_seq) {
    return new tenzo::FusedKVCache(layers, q_heads, kv_heads, head_dim, max_seq, "int8_fused");
}
__attribute__((visibility("default")))
void refk_kv_destroy(void* kv) { delete static_cast<tenzo::FusedKVCache*>(kv); }
__attribute__((visibility("default")))
void refk_kv_set_len(void* kv, int len) { static_cast<tenzo::FusedKVCache*>(kv)->cur_seq_len = len; }
__attribute__((visibility("default")))
int8_t* refk_kv_k(void* kv) { return static_cast<tenzo::FusedKVCache*>(kv)->int8_k.data(); }
__attribute__((visibility("default")))
int8_t* refk_kv_v(void* kv) { return static_cast<tenzo::FusedKVCache*>(kv)->int8_v.data(); }
__attribute__((visibility("default")))
float* refk_kv_k_scales(void* kv) { return static_cast<tenzo::FusedKVCache*>(kv)->int8_k_scales.data(); }
__attribute__((visibility("default")))
float* refk_kv_v_scales(void* kv) { return static_cast<tenzo::FusedKVCache*>(kv)->int8_v_scales.data(); }
// forward_attention_raw (TenzoEngine.cpp:447-919): RoPE in place on q,k; append at cur_seq_len;
// attention over cur_seq_len+1 keys. Does NOT advance cur_seq_len (the engine does, :1831-1835).
__attribute__((visibility("default")))
void refk_kv_attention(void* kv, int layer, float* q, float* k, float* v, float* out) {
    static_cast<tenzo::FusedKVCache*>(kv)->forward_attention_raw(layer, q, k, v, out);
}

// PagedKVCache (kv_mode "paged_int8", TenzoEngine.h:154-193); pools and block table are public members.
__attribute__((visibility("default")))
void* refk_paged_create(int layers, int q_heads, int kv_heads, int head_dim, int total_blocks) {
    return new tenzo::PagedKVCache(layers, q_heads, kv_heads, head_dim, total_blocks);
}
__attribute__((visibility("default")))
void refk_paged_destroy(void* kv) { delete static_cast<tenzo::PagedKVCache*>(kv); }
__attribute__((visibility("default")))
void refk_paged_set_len(void* kv, int len) { static_cast<tenzo::PagedKVCache*>(kv)->cur_seq_len = len; }
__attribute__((visibility("default")))
int8_t* refk_paged_k(void* kv) { return static_cast<tenzo::PagedKVCache*>(kv)->paged_k_pool.data(); }
__attribute__((visibility("default")))
int8_t* refk_paged_v(void* kv) { return static_cast<tenzo::PagedKVCache*>(kv)->paged_v_pool.data(); }
__attribute__((visibility("default")))
float* refk_paged_k_scales(void* kv) { return static_cast<tenzo::PagedKVCache*>(kv)->paged_k_scales.data(); }
__attribute__((visibility("default")))
float* refk_paged_v_scales(void* kv) { return static_cast<tenzo::PagedKVCache*>(kv)->paged_v_scales.data(); }
// Block table as the cache holds it after the calls so far; returns its length.
__attribute__((visibility("default")))
int refk_paged_table(void* kv, int32_t* out, int max_n) {
    auto& t = static_cast<tenzo::PagedKVCache*>(kv)->block_table;
    for (int i = 0; i < static_cast<int>(t.size()) && i < max_n; ++i) out[i] = t[i];
    return static_cast<int>(t.size());
}
// Hands the next logical block a physical block chosen by the caller (the reference's own allocator only ever
// yields 0, 1, 2, ...): lets a test exercise the table translation with a scattered placement.
__attribute__((visibility("default")))
void refk_paged_push_block(void* kv, int32_t blk) { static_cast<tenzo::PagedKVCache*>(kv)->block_table.push_back(blk); }
// forward_attention_raw (TenzoEngine.cpp:242-445); does not advance cur_seq_len.
__attribute__((visibility("default")))
void refk_paged_attention(void* kv, int layer, float* q, float* k, float* v, float* out) {
    static_cast<tenzo::PagedKVCache*>(kv)->forward_attention_raw(layer, q, k, v, out);
}
__attribute__((visibility("default")))
void* refk_engine_paged_kv(tenzo_engine_t e) { return &e->impl->paged_kv_cache; }

// Engine internals for teacher forcing (TenzoEngine.h:195-262, all public).
// which: 0 x, 1 norm_x, 2 q, 3 k, 4 v, 5 attn_out, 6 attn_sub, 7 out, 8 h1, 9 post_norm,
//        10 gate, 11 up, 12 act, 13 ffn_norm, 14 down, 15 logits
__attribute__((visibility("default")))
float* refk_engine_buffer(tenzo_engine_t e, int which) {
    auto* m = e->impl.get();
    switch (which) {
        case 0: return m->buf_x.data();        case 1: return m->buf_norm_x.data();
        case 2: return m->buf_q.data();        case 3: return m->buf_k.data();
        case 4: return m->buf_v.data();        case 5: return m->buf_attn_out.data();
        case 6: return m->buf_attn_sub.data(); case 7: return m->buf_out.data();
        case 8: return m->buf_h1.data();       case 9: return m->buf_post_norm.data();
        case 10: return m->buf_gate.data();    case 11: return m->buf_up.data();
        case 12: return m->buf_act.data();     case 13: return m->buf_ffn_norm.data();
        case 14: return m->buf_down.data();    case 15: return m->logits_scratch.data();
        default: return nullptr;
    }
}
__attribute__((visibility("default")))
int8_t* refk_engine_x_i8(tenzo_engine_t e) { return e->impl->buf_x_i8.data(); }
__attribute__((visibility("default")))
void* refk_engine_kv(tenzo_engine_t e) { return &e->impl->kv_cache; }
__attribute__((visibility("default")))
void refk_engine_embedding(tenzo_engine_t e, int tok) { e->impl->embedding_lookup(tok); }
__attribute__((visibility("default")))
void refk_engine_forward_layer(tenzo_engine_t e, int layer) { e->impl->forward_layer_raw(layer); }
__attribute__((visibility("default")))
void refk_engine_advance(tenzo_engine_t e) { e->impl->kv_cache.increment_seq_len(1); }
__attribute__((visibility("default")))
void refk_engine_logits(tenzo_engine_t e) { e->impl->compute_logits(); }
__attribute__((visibility("default")))
int refk_engine_sample(tenzo_engine_t e, const tenzo_sampling_params_t* p, const int* past, int n) {
    return e->impl->sample_top_k_top_p(p, past, n);
}

}  // extern "C"
