// extern "C" boundary: the fourteen tenzo.h entry points (reference: include/tenzo.h:92-193,
// implemented in src/runtime/TenzoEngine.cpp:2086-2204) and the additive tenzo_ext.h calls.
// No exception crosses this file; failures become the reference's status codes and a message
// retrievable through tenzo_ext_last_error().
#include <cstring>
#include <new>
#include <stdexcept>
#include <string>
#include <vector>

#include "../../include/tenzo.h"
#include "../../include/tenzo_ext.h"
#include "../../include/tenzo_kernels.h"
#include "engine.h"
#include "sampler.h"

namespace tz {
tenzo_status_t load_model_files(Engine& e, const char* weights_path, const char* mlir_path);
}

namespace {

template <typename F>
tenzo_status_t guarded(F&& f) {
    try {
        tz::g_last_error.clear();
        return f();
    } catch (const std::bad_alloc&) {
        tz::set_error("host allocation failed");
        return TENZO_ERROR_OUT_OF_MEMORY;
    } catch (const std::invalid_argument& e) {
        tz::set_error(e.what());
        return TENZO_ERROR_INVALID_ARGUMENT;
    } catch (const std::out_of_range& e) {
        tz::set_error(e.what());
        return TENZO_ERROR_INVALID_ARGUMENT;
    } catch (const std::exception& e) {
        tz::set_error(e.what());
        const std::string m = e.what();
        if (m.find("out of memory") != std::string::npos) return TENZO_ERROR_OUT_OF_MEMORY;
        return TENZO_ERROR_UNSUPPORTED;
    } catch (...) {
        tz::set_error("unknown failure");
        return TENZO_ERROR_UNSUPPORTED;
    }
}

bool live(tenzo_engine_t e) { return e && e->impl; }

}  // namespace

extern "C" {

const char* tenzo_get_version(void) { return TENZO_VERSION_STRING; }

tenzo_config_t tenzo_default_config(void) {
    tenzo_config_t c;
    c.hidden_size = 2560;
    c.num_q_heads = 20;
    c.num_kv_heads = 5;
    c.head_dim = 128;
    c.num_layers = 30;
    c.ffn_dim = 6912;
    c.vocab_size = 128256;
    c.max_seq_len = 8192;
    c.kv_mode = "int8_fused";
    c.device = "cpu";   // kept for struct-level compatibility (TenzoEngine.cpp:2103); the engine is CUDA regardless
    return c;
}

tenzo_sampling_params_t tenzo_default_sampling_params(void) {
    tenzo_sampling_params_t p;
    p.temperature = 0.7f;
    p.top_p = 0.9f;
    p.top_k = 40;
    p.repetition_penalty = 1.15f;
    return p;
}

tenzo_ext_options_t tenzo_ext_default_options(void) {
    tenzo_ext_options_t o;
    o.batch = 1;
    o.rope_theta = 10000.0f;
    o.use_graph = -1;
    o.use_pdl = -1;
    o.persistent = -1;
    o.attention_mode = -1;
    return o;
}

tenzo_engine_t tenzo_ext_create_engine(const tenzo_config_t* config, const tenzo_ext_options_t* opt) {
    tenzo_engine_t handle = nullptr;
    guarded([&]() -> tenzo_status_t {
        tenzo_config_t c = config ? *config : tenzo_default_config();
        tenzo_ext_options_t o = opt ? *opt : tenzo_ext_default_options();
        if (c.kv_mode && std::strcmp(c.kv_mode, "int8_fused") != 0 && std::strcmp(c.kv_mode, "paged_int8") != 0)
            throw std::invalid_argument(std::string("kv_mode '") + c.kv_mode + "' is not implemented; only int8_fused and paged_int8");
        int n_dev = 0;
        if (cudaGetDeviceCount(&n_dev) != cudaSuccess || n_dev == 0)
            throw std::runtime_error("no CUDA device is visible; this library has no CPU path");
        tz::Engine* e = new tz::Engine(c, o);
        handle = new tenzo_engine_opaque{e};
        return TENZO_SUCCESS;
    });
    return handle;
}

tenzo_engine_t tenzo_create_engine(const tenzo_config_t* config) { return tenzo_ext_create_engine(config, nullptr); }

void tenzo_destroy_engine(tenzo_engine_t engine) {
    if (!engine) return;
    delete engine->impl;
    delete engine;
}

void tenzo_reset(tenzo_engine_t engine) {
    if (!live(engine)) return;
    try {
        engine->impl->reset_kv();                  // TenzoEngine.cpp:213-215, :242-246
    } catch (const std::exception& ex) {
        tz::set_error(ex.what());
    }
}

int tenzo_get_seq_len(tenzo_engine_t engine) { return live(engine) ? engine->impl->seq_len[0] : 0; }

tenzo_status_t tenzo_set_layer_weights(tenzo_engine_t engine, int layer_idx, const tenzo_layer_weights_t* weights) {
    if (!live(engine) || !weights) return TENZO_ERROR_INVALID_ARGUMENT;
    return guarded([&]() -> tenzo_status_t {
        if (layer_idx < 0 || layer_idx >= engine->impl->L) throw std::out_of_range("layer index outside [0, num_layers)");
        engine->impl->set_layer(layer_idx, *weights);
        return TENZO_SUCCESS;
    });
}

tenzo_status_t tenzo_set_final_norm(tenzo_engine_t engine, const float* norm_w) {
    if (!live(engine) || !norm_w) return TENZO_ERROR_INVALID_ARGUMENT;
    return guarded([&]() -> tenzo_status_t {
        engine->impl->set_final_norm(norm_w);
        return TENZO_SUCCESS;
    });
}

tenzo_status_t tenzo_set_lm_head_f32(tenzo_engine_t engine, const float* embed_w, int, int) {
    if (!live(engine) || !embed_w) return TENZO_ERROR_INVALID_ARGUMENT;
    tz::set_error("the fp32 LM head is outside the quantized decode path; quantise per row and use tenzo_set_lm_head_i8");
    return TENZO_ERROR_UNSUPPORTED;
}

tenzo_status_t tenzo_set_lm_head_i8(tenzo_engine_t engine, const int8_t* embed_w, const float* embed_scales,
                                    int vocab_size, int hidden_size) {
    if (!live(engine) || !embed_w || !embed_scales) return TENZO_ERROR_INVALID_ARGUMENT;
    return guarded([&]() -> tenzo_status_t {
        if (vocab_size != engine->impl->V || hidden_size != engine->impl->h)
            throw std::invalid_argument("LM head shape differs from the engine configuration");
        engine->impl->set_lm_head(embed_w, embed_scales);
        return TENZO_SUCCESS;
    });
}

tenzo_status_t tenzo_load_model(tenzo_engine_t engine, const char* weights_path, const char* mlir_path) {
    if (!live(engine) || !weights_path || !mlir_path) return TENZO_ERROR_INVALID_ARGUMENT;
    tenzo_status_t inner = TENZO_SUCCESS;
    tenzo_status_t outer = guarded([&]() -> tenzo_status_t {
        inner = tz::load_model_files(*engine->impl, weights_path, mlir_path);
        return inner;
    });
    return outer;
}

tenzo_status_t tenzo_prefill_token(tenzo_engine_t engine, int token_id) {
    if (!live(engine)) return TENZO_ERROR_INVALID_ARGUMENT;
    return guarded([&]() -> tenzo_status_t {
        if (engine->impl->batch != 1) throw std::invalid_argument("batched engine: use tenzo_ext_prefill_tokens");
        engine->impl->prefill(&token_id);
        return TENZO_SUCCESS;
    });
}

int tenzo_generate_step(tenzo_engine_t engine, int cur_token, const tenzo_sampling_params_t* params,
                        const int* past_tokens, int past_tokens_len) {
    if (!live(engine)) return -1;
    int out = -1;
    tenzo_status_t st = guarded([&]() -> tenzo_status_t {
        tz::Engine& e = *engine->impl;
        if (e.batch != 1) throw std::invalid_argument("batched engine: use tenzo_ext_generate_step");
        const tenzo_sampling_params_t p = params ? *params : tenzo_default_sampling_params();   // :1729-1732
        e.generate(&cur_token, &out);
        const bool penalised = p.repetition_penalty != 1.0f && past_tokens && past_tokens_len > 0;
        if (p.temperature > 0.0f || penalised) out = e.sample(p, past_tokens, past_tokens_len);
        return TENZO_SUCCESS;
    });
    return st == TENZO_SUCCESS ? out : -1;
}

// ---------------------------------------------------------------------------------------------
// extension
// ---------------------------------------------------------------------------------------------

int tenzo_ext_batch(tenzo_engine_t engine) { return live(engine) ? engine->impl->batch : 0; }

tenzo_status_t tenzo_ext_prefill_tokens(tenzo_engine_t engine, const int* tokens) {
    if (!live(engine) || !tokens) return TENZO_ERROR_INVALID_ARGUMENT;
    return guarded([&]() -> tenzo_status_t {
        engine->impl->prefill(tokens);
        return TENZO_SUCCESS;
    });
}

tenzo_status_t tenzo_ext_generate_step(tenzo_engine_t engine, const int* cur_tokens,
                                       const tenzo_sampling_params_t* params, int* out_tokens) {
    if (!live(engine) || !cur_tokens || !out_tokens) return TENZO_ERROR_INVALID_ARGUMENT;
    return guarded([&]() -> tenzo_status_t {
        if (params && (params->temperature > 0.0f))
            throw std::invalid_argument("batched decode is greedy: pass temperature <= 0 (or NULL params)");
        engine->impl->generate(cur_tokens, out_tokens);
        return TENZO_SUCCESS;
    });
}

tenzo_status_t tenzo_ext_decode_greedy(tenzo_engine_t engine, const int* first_tokens, int n_steps, int* out_tokens) {
    if (!live(engine) || !first_tokens || !out_tokens || n_steps < 0) return TENZO_ERROR_INVALID_ARGUMENT;
    return guarded([&]() -> tenzo_status_t {
        tz::Engine& e = *engine->impl;
        for (int s = 0; s < e.batch; ++s)
            if (e.seq_len[s] + n_steps > e.cfg.max_seq_len) throw std::out_of_range("n_steps would overflow the KV cache");
        e.decode_greedy(first_tokens, n_steps, out_tokens);
        return TENZO_SUCCESS;
    });
}

static tenzo_status_t kv_copy(tenzo_engine_t engine, int seq, int layer, void* k, void* v, void* sk, void* sv, int len,
                              bool to_device) {
    if (!live(engine) || !k || !v || !sk || !sv) return TENZO_ERROR_INVALID_ARGUMENT;
    return guarded([&]() -> tenzo_status_t {
        tz::Engine& e = *engine->impl;
        if (seq < 0 || seq >= e.batch || layer < 0 || layer >= e.L || len < 0 || len > e.cfg.max_seq_len)
            throw std::out_of_range("sequence, layer or length out of range");
        cudaStreamSynchronize(e.stream);
        const int nkv = e.cfg.num_kv_heads;
        if (e.paged) {
            if (to_device) e.reserve_blocks(seq, len);            // an import brings its own blocks
            else if (e.n_blocks[seq] * tz::Engine::kBlock < len) throw std::out_of_range("the sequence holds fewer tokens than asked for");
        }
        const int run = e.paged ? tz::Engine::kBlock : (len > 0 ? len : 1);   // tokens that are contiguous in the cache
        for (int hh = 0; hh < nkv; ++hh) {
            for (int t0 = 0; t0 < len; t0 += run) {
                const size_t n = (size_t)(len - t0 < run ? len - t0 : run);
                const size_t row = e.kv_row(seq, layer, hh, t0);
                const size_t hb = (size_t)hh * len + t0;
                cudaError_t c0, c1, c2, c3;
                if (to_device) {
                    c0 = cudaMemcpy(e.cache_k + row * 128, (const int8_t*)k + hb * 128, n * 128, cudaMemcpyHostToDevice);
                    c1 = cudaMemcpy(e.cache_v + row * 128, (const int8_t*)v + hb * 128, n * 128, cudaMemcpyHostToDevice);
                    c2 = cudaMemcpy(e.scale_k + row, (const float*)sk + hb, n * 4, cudaMemcpyHostToDevice);
                    c3 = cudaMemcpy(e.scale_v + row, (const float*)sv + hb, n * 4, cudaMemcpyHostToDevice);
                } else {
                    c0 = cudaMemcpy((int8_t*)k + hb * 128, e.cache_k + row * 128, n * 128, cudaMemcpyDeviceToHost);
                    c1 = cudaMemcpy((int8_t*)v + hb * 128, e.cache_v + row * 128, n * 128, cudaMemcpyDeviceToHost);
                    c2 = cudaMemcpy((float*)sk + hb, e.scale_k + row, n * 4, cudaMemcpyDeviceToHost);
                    c3 = cudaMemcpy((float*)sv + hb, e.scale_v + row, n * 4, cudaMemcpyDeviceToHost);
                }
                if (c0 != cudaSuccess || c1 != cudaSuccess || c2 != cudaSuccess || c3 != cudaSuccess)
                    throw std::runtime_error("KV copy failed");
            }
        }
        return TENZO_SUCCESS;
    });
}

tenzo_status_t tenzo_ext_kv_import(tenzo_engine_t engine, int seq, int layer, const int8_t* k, const int8_t* v,
                                   const float* sk, const float* sv, int len) {
    return kv_copy(engine, seq, layer, (void*)k, (void*)v, (void*)sk, (void*)sv, len, true);
}

tenzo_status_t tenzo_ext_kv_export(tenzo_engine_t engine, int seq, int layer, int8_t* k, int8_t* v, float* sk,
                                   float* sv, int len) {
    return kv_copy(engine, seq, layer, k, v, sk, sv, len, false);
}

tenzo_status_t tenzo_ext_kv_fill_random(tenzo_engine_t engine, int len, uint64_t seed) {
    if (!live(engine)) return TENZO_ERROR_INVALID_ARGUMENT;
    return guarded([&]() -> tenzo_status_t {
        tz::Engine& e = *engine->impl;
        if (len < 0 || len > e.cfg.max_seq_len) throw std::out_of_range("length outside [0, max_seq_len]");
        e.kv_fill(len, (unsigned long long)seed);
        return TENZO_SUCCESS;
    });
}

tenzo_status_t tenzo_ext_set_seq_len(tenzo_engine_t engine, int seq, int len) {
    if (!live(engine)) return TENZO_ERROR_INVALID_ARGUMENT;
    tz::Engine& e = *engine->impl;
    if (seq < 0 || seq >= e.batch || len < 0 || len > e.cfg.max_seq_len) return TENZO_ERROR_INVALID_ARGUMENT;
    return guarded([&]() -> tenzo_status_t {
        e.release_blocks(seq, len);                // block pools: the table follows the length
        e.reserve_blocks(seq, len);
        e.seq_len[seq] = len;
        return TENZO_SUCCESS;
    });
}

int tenzo_ext_get_seq_len(tenzo_engine_t engine, int seq) {
    if (!live(engine) || seq < 0 || seq >= engine->impl->batch) return 0;
    return engine->impl->seq_len[seq];
}

tenzo_status_t tenzo_ext_read_buffer(tenzo_engine_t engine, int which, int seq, float* dst, size_t count) {
    if (!live(engine) || !dst) return TENZO_ERROR_INVALID_ARGUMENT;
    return guarded([&]() -> tenzo_status_t {
        tz::Engine& e = *engine->impl;
        if (seq < 0 || seq >= e.batch) throw std::out_of_range("sequence index out of range");
        const float* src = nullptr;
        size_t n = 0;
        const size_t qkv = (size_t)e.qd + 2 * e.kvd;
        switch (which) {
            case TENZO_BUF_X: src = e.b_x + (size_t)seq * e.h; n = e.h; break;
            case TENZO_BUF_Q: src = e.b_qkv + seq * qkv; n = e.qd; break;
            case TENZO_BUF_K: src = e.b_qkv + seq * qkv + e.qd; n = e.kvd; break;
            case TENZO_BUF_V: src = e.b_qkv + seq * qkv + e.qd + e.kvd; n = e.kvd; break;
            case TENZO_BUF_ATTN_OUT: src = e.b_attn + (size_t)seq * e.qd; n = e.qd; break;
            case TENZO_BUF_H1: src = e.b_h1 + (size_t)seq * e.h; n = e.h; break;
            case TENZO_BUF_ACT: src = e.b_act + (size_t)seq * e.ffn; n = e.ffn; break;
            case TENZO_BUF_LOGITS: src = e.b_logits + (size_t)seq * e.V; n = e.V; break;
            default: throw std::invalid_argument("unknown buffer id");
        }
        if (count > n) throw std::out_of_range("count exceeds the buffer length");
        cudaStreamSynchronize(e.stream);
        if (cudaMemcpy(dst, src, count * 4, cudaMemcpyDeviceToHost) != cudaSuccess) throw std::runtime_error("read-back failed");
        return TENZO_SUCCESS;
    });
}

tenzo_status_t tenzo_ext_write_x(tenzo_engine_t engine, int seq, const float* x) {
    if (!live(engine) || !x) return TENZO_ERROR_INVALID_ARGUMENT;
    tz::Engine& e = *engine->impl;
    if (seq < 0 || seq >= e.batch) return TENZO_ERROR_INVALID_ARGUMENT;
    cudaStreamSynchronize(e.stream);
    return cudaMemcpy(e.b_x + (size_t)seq * e.h, x, (size_t)e.h * 4, cudaMemcpyHostToDevice) == cudaSuccess
               ? TENZO_SUCCESS : TENZO_ERROR_UNSUPPORTED;
}

tenzo_status_t tenzo_ext_run_layer(tenzo_engine_t engine, int layer) {
    if (!live(engine)) return TENZO_ERROR_INVALID_ARGUMENT;
    return guarded([&]() -> tenzo_status_t {
        tz::Engine& e = *engine->impl;
        if (layer < 0 || layer >= e.L) throw std::out_of_range("layer index outside [0, num_layers)");
        int longest = 1;
        for (int s = 0; s < e.batch; ++s) {
            if (e.seq_len[s] + 1 > e.cfg.max_seq_len) throw std::out_of_range("KV cache is full");
            longest = e.seq_len[s] + 1 > longest ? e.seq_len[s] + 1 : longest;
        }
        e.push_state(nullptr);
        e.prepare_kv(1);
        e.enqueue_layer(layer, longest);
        if (cudaStreamSynchronize(e.stream) != cudaSuccess) throw std::runtime_error("layer execution failed");
        return TENZO_SUCCESS;
    });
}

tenzo_status_t tenzo_ext_synchronize(tenzo_engine_t engine) {
    if (!live(engine)) return TENZO_ERROR_INVALID_ARGUMENT;
    return cudaStreamSynchronize(engine->impl->stream) == cudaSuccess ? TENZO_SUCCESS : TENZO_ERROR_UNSUPPORTED;
}

float tenzo_ext_last_device_ms(tenzo_engine_t engine) { return live(engine) ? engine->impl->last_ms() : -1.0f; }

float tenzo_ext_bench_gemv_stack(tenzo_engine_t engine, int iters, unsigned long long* launches) {
    if (!live(engine) || iters <= 0) return -1.0f;
    float ms = -1.0f;
    guarded([&]() -> tenzo_status_t {
        ms = engine->impl->bench_gemv_stack(iters, launches);
        return TENZO_SUCCESS;
    });
    return ms;
}

unsigned long long tenzo_ext_kernel_launches(tenzo_engine_t engine) { return live(engine) ? engine->impl->launches : 0ull; }

int tenzo_ext_persistent_phase_ns(tenzo_engine_t engine, unsigned long long* out8, int reset) {
    if (!live(engine) || !out8) return -1;
    tz::Engine& e = *engine->impl;
    if (!e.pc_usable() || !e.pc_phase_ns) return 0;
    cudaStreamSynchronize(e.stream);
    if (cudaMemcpy(out8, e.pc_phase_ns, 8 * sizeof(unsigned long long), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    if (reset == 2) {                      // experiments: out8 has room for 72 values, the optional timeline follows the sums
        if (cudaMemcpy(out8, e.pc_phase_ns, 72 * sizeof(unsigned long long), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    } else if (reset) {
        cudaMemset(e.pc_phase_ns, 0, 8 * sizeof(unsigned long long));
    }
    return 1;
}


tenzo_status_t tenzo_ext_prefill_chunk(tenzo_engine_t engine, const int* tokens, int n) {
    if (!live(engine) || !tokens || n < 0) return TENZO_ERROR_INVALID_ARGUMENT;
    return guarded([&]() -> tenzo_status_t {
        engine->impl->prefill_chunk(tokens, n);
        return TENZO_SUCCESS;
    });
}

tenzo_status_t tenzo_ext_rope_tables(int max_seq, int head_dim, float rope_theta, float* cos_host, float* sin_host) {
    if (max_seq <= 0 || head_dim <= 0 || (head_dim & 1) || !cos_host || !sin_host) return TENZO_ERROR_INVALID_ARGUMENT;
    tz::rope_tables_host(max_seq, head_dim, rope_theta > 0.0f ? rope_theta : 10000.0f, cos_host, sin_host);
    return TENZO_SUCCESS;
}

int tenzo_ext_sample_pairs(const float* values, const int* indices, int n, const tenzo_sampling_params_t* params, float r) {
    if (!values || n <= 0) return -1;
    const tenzo_sampling_params_t p = params ? *params : tenzo_default_sampling_params();
    return tz::sample_pairs(values, indices, n, p, r);
}

const char* tenzo_ext_last_error(void) { return tz::g_last_error.c_str(); }

}  // extern "C"
