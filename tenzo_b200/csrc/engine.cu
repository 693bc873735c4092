// Resident decode engine behind the tenzo.h ABI (and its additive extension, tenzo_ext.h).
//
// Mirrors TenzoEngineImpl of the reference (src/runtime/TenzoEngine.cpp:1215-1838): embedding ->
// num_layers x forward_layer -> (generate only) logits + sampler, with the sequence length
// advanced once per token after all layers. The differences are structural: weights, KV cache
// and every intermediate stay in device memory, a decode step is a fixed kernel sequence replayed
// as a CUDA graph (token ids and positions are read from device memory so the graph never
// changes), and `batch` independent sequences advance together.
//
// Per layer (reference lines in brackets):
//   tl1_gemv  in_norm + quant + [q|k|v] rows, store                     [:1542-1572]
//   attention RoPE, int8 append, softmax(QK)V                           [:1578]
//   tl1_gemv  attn_sub_norm + quant + out rows, h1 = x + .              [:1582-1590]
//   tl1_gemv  post_norm + quant + [gate|up] rows, relu(g)^2*u           [:1594-1620]
//   tl1_gemv  ffn_sub_norm + quant + down rows, x = h1 + .              [:1622-1628]
#include <cuda_runtime.h>
#include <nvtx3/nvToolsExt.h>

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <new>
#include <stdexcept>
#include <string>
#include <vector>

#include "../../include/tenzo.h"
#include "../../include/tenzo_ext.h"
#include "common.cuh"
#include "../../include/tenzo_kernels.h"
#include "engine.h"
#include "sampler.h"

namespace tz {

// cos/sin [max_seq][head_dim/2] with the reference's float expressions (TenzoEngine.cpp:466-469).
void rope_tables_host(int max_seq, int head_dim, float theta, float* cs, float* sn) {
    const int half = head_dim / 2;
    std::vector<float> freq(half);
    for (int i = 0; i < half; ++i) freq[i] = 1.0f / std::pow(theta, static_cast<float>(2 * i) / head_dim);
    for (int p = 0; p < max_seq; ++p)
        for (int i = 0; i < half; ++i) {
            const float ang = static_cast<float>(p) * freq[i];
            cs[(size_t)p * half + i] = std::cos(ang);
            sn[(size_t)p * half + i] = std::sin(ang);
        }
}


thread_local std::string g_last_error;
void set_error(const std::string& m) { g_last_error = m; }

#define TZ_KERNEL(expr)                                                                         \
    do {                                                                                        \
        int _r = (expr);                                                                        \
        if (_r > 0) throw CudaError((cudaError_t)_r, #expr);                                    \
        if (_r < 0) throw std::runtime_error(std::string(#expr) + " rejected its arguments");   \
    } while (0)

__global__ void advance_kernel(int* pos, int* tokens, const int* next, int batch, int feed_back, int vocab) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < batch) {
        pos[i] += 1;
        if (feed_back) {
            const int t = next[i];
            tokens[i] = (t >= 0 && t < vocab) ? t : 0;
        }
    }
}

__global__ void record_tokens_kernel(const int* next, int* history, int step, int batch) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < batch) history[(size_t)step * batch + i] = next[i];
}

// Chunked prefill: rotate and quantise the K rows, quantise the V rows of M consecutive tokens of one sequence and
// append them at positions pos0.. (the same arithmetic as the attention kernel's own append, TenzoEngine.cpp:459-533).
// One warp per (token, kv head, K|V); lane l holds elements 4l..4l+3.
// With a block table (kv_mode "paged_int8") the row goes to block table[pos / 16], slot pos % 16 of the pools
// [block][n_layers][kv_head][16][128] (TenzoEngine.cpp:322-323).
__global__ void __launch_bounds__(64) kv_append_rows_kernel(const float* qkv, int row_stride, int q_dim, int kv_dim, int n_kv, int pos0,
                                                            const float* rope_cos, const float* rope_sin, int8_t* cache_k, int8_t* cache_v,
                                                            float* scale_k, float* scale_v, size_t layer_row_base, int max_seq,
                                                            const int* table, int n_layers, int layer) {
    const int token = blockIdx.x, kvh = blockIdx.y, is_v = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int pos = pos0 + token;
    const float* src = qkv + (size_t)token * row_stride + q_dim + (is_v ? kv_dim : 0) + kvh * 128;
    float x[4];
    if (is_v) {
#pragma unroll
        for (int j = 0; j < 4; ++j) x[j] = __ldcg(src + lane * 4 + j);
    } else {
        const float* cs = rope_cos + (size_t)pos * 64;
        const float* sn = rope_sin + (size_t)pos * 64;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int e = lane * 4 + j, i = e & 63;
            const float x0 = __ldcg(src + i), x1 = __ldcg(src + i + 64), c = cs[i], sgn = sn[i];
            x[j] = e < 64 ? __fmaf_rn(x0, c, -(x1 * sgn)) : __fmaf_rn(x0, sgn, x1 * c);      // :475-476
        }
    }
    float amax = 1e-8f;
#pragma unroll
    for (int j = 0; j < 4; ++j) amax = fmaxf(amax, fabsf(x[j]));
    amax = tz::warp_max(amax);
    const float sc = amax / 127.0f;           // :522
    const float inv = 1.0f / sc;              // :527
    uint32_t packed = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float qf = fminf(fmaxf(roundf(x[j] * inv), -128.0f), 127.0f);   // :530
        packed |= ((uint32_t)(uint8_t)(int8_t)(int)qf) << (8 * j);
    }
    const size_t row = table ? (((size_t)table[pos >> 4] * n_layers + layer) * n_kv + kvh) * 16 + (size_t)(pos & 15)
                             : layer_row_base + (size_t)kvh * max_seq + pos;
    reinterpret_cast<uint32_t*>((is_v ? cache_v : cache_k) + row * 128)[lane] = packed;
    if (lane == 0) (is_v ? scale_v : scale_k)[row] = sc;
}

// Deterministic stand-in KV: int8 rows and positive scales from a counter hash.
__global__ void kv_fill_kernel(int8_t* k, int8_t* v, float* sk, float* sv, size_t rows_total, int max_seq, int len,
                               unsigned long long seed) {
    const size_t n = rows_total * 128;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const size_t row = i >> 7;
        if ((int)(row % max_seq) >= len) continue;
        unsigned long long z = (i + 1) * 0x9E3779B97F4A7C15ull + seed;
        z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
        z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
        z ^= z >> 31;
        // roughly N(0,1)/amax*127 shaped: sum of four uniform bytes, centred
        const int a = (int)(z & 255) + (int)((z >> 8) & 255) + (int)((z >> 16) & 255) + (int)((z >> 24) & 255) - 510;
        const int b = (int)((z >> 32) & 255) + (int)((z >> 40) & 255) + (int)((z >> 48) & 255) + (int)((z >> 56) & 255) - 510;
        k[i] = (int8_t)max(-127, min(127, a / 4));
        v[i] = (int8_t)max(-127, min(127, b / 4));
        if ((i & 127) == 0) {
            sk[row] = 0.02f + 0.00001f * (float)((z >> 20) & 1023);
            sv[row] = 0.02f + 0.00001f * (float)((z >> 44) & 1023);
        }
    }
}

static int env_flag(const char* name, int dflt) {
    const char* s = std::getenv(name);
    return s ? std::atoi(s) : dflt;
}

// Named ranges around the engine's public operations for timeline tools (the reference marks nothing; its only
// instrumentation is the wall-clock tok/s of its CLI). Off unless TENZO_NVTX=1: a range push is a call into the tools
// interface on every token.
struct NvtxRange {
    bool on;
    explicit NvtxRange(const char* name) : on(env_flag("TENZO_NVTX", 0) != 0) { if (on) nvtxRangePushA(name); }
    ~NvtxRange() { if (on) nvtxRangePop(); }
};

// A constructor that throws never runs the destructor, so what it had acquired by then (stream, events, device and
// pinned memory) is released here before the exception leaves.
Engine::Engine(const tenzo_config_t& c, const tenzo_ext_options_t& o) : cfg(c) {
    try {
        init(c, o);
    } catch (...) {
        release_all();
        throw;
    }
}

void Engine::init(const tenzo_config_t& c, const tenzo_ext_options_t& o) {
    batch = o.batch > 0 ? o.batch : 1;
    rope_theta = o.rope_theta > 0.0f ? o.rope_theta : 10000.0f;   // TenzoEngine.cpp:456
    use_graph = o.use_graph >= 0 ? o.use_graph : env_flag("TENZO_CUDA_GRAPH", 1);
    use_pdl = o.use_pdl >= 0 ? o.use_pdl : env_flag("TENZO_CUDA_PDL", 1);
    persistent = o.persistent >= 0 ? o.persistent : env_flag("TENZO_PERSISTENT", 0);
    attention_mode = o.attention_mode >= 0 ? o.attention_mode : env_flag("TENZO_ATTENTION_MODE", 0);
    if (attention_mode != 0 && attention_mode != 1) throw std::invalid_argument("attention_mode must be 0 or 1");
    paged = c.kv_mode && std::strcmp(c.kv_mode, "paged_int8") == 0;       // TenzoEngine.cpp:1220
    cfg.kv_mode = paged ? "paged_int8" : "int8_fused";
    cfg.device = "cuda";
    h = cfg.hidden_size;
    qd = cfg.num_q_heads * cfg.head_dim;
    kvd = cfg.num_kv_heads * cfg.head_dim;
    ffn = cfg.ffn_dim;
    L = cfg.num_layers;
    V = cfg.vocab_size;
    if (cfg.head_dim != 128) throw std::invalid_argument("head_dim must be 128");
    if (h <= 0 || ffn <= 0 || L <= 0 || V <= 0 || cfg.max_seq_len <= 0) throw std::invalid_argument("non-positive dimension");
    if (h % 64 || qd % 64 || kvd % 64 || ffn % 64) throw std::invalid_argument("hidden, q_dim, kv_dim and ffn_dim must be multiples of 64");
    if (qd != h) throw std::invalid_argument("num_q_heads*head_dim must equal hidden_size (the reference assumes it, TenzoEngine.cpp:1582)");
    if (cfg.num_q_heads % cfg.num_kv_heads) throw std::invalid_argument("num_q_heads must be a multiple of num_kv_heads");
    const int g = cfg.num_q_heads / cfg.num_kv_heads;
    if (g != 1 && g != 2 && g != 4 && g != 8) throw std::invalid_argument("query group size must be 1, 2, 4 or 8");
    if (h > 16384 || ffn > 16384) throw std::invalid_argument("hidden_size and ffn_dim are limited to 16384");

    TZ_CUDA(cudaGetDevice(&device));
    TZ_CUDA(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
    TZ_CUDA(cudaEventCreate(&ev0));
    TZ_CUDA(cudaEventCreate(&ev1));

    layers.resize(L);
    const size_t B = batch;
    auto dalloc = [&](size_t bytes) -> void* {
        void* p = nullptr;
        TZ_CUDA(cudaMalloc(&p, bytes ? bytes : 16));
        TZ_CUDA(cudaMemsetAsync(p, 0, bytes ? bytes : 16, stream));
        owned.push_back(p);
        return p;
    };
    d_tokens = (int*)dalloc(B * 4);
    d_pos = (int*)dalloc(B * 4);
    d_next = (int*)dalloc(B * 4);
    b_x = (float*)dalloc(B * h * 4);
    b_qkv = (float*)dalloc(B * (qd + 2 * kvd) * 4);
    b_attn = (float*)dalloc(B * qd * 4);
    b_h1 = (float*)dalloc(B * h * 4);
    b_act = (float*)dalloc(B * ffn * 4);
    b_logits = (float*)dalloc(B * V * 4);

    kv_rows_per_seq = (size_t)L * cfg.num_kv_heads * cfg.max_seq_len;
    if (paged) {
        // (max_seq_len + 15) / 16 blocks per sequence as the reference sizes its pool (:1218), for every sequence
        table_stride = (cfg.max_seq_len + kBlock - 1) / kBlock;
        total_blocks = batch * table_stride;
        kv_rows_per_seq = (size_t)table_stride * L * cfg.num_kv_heads * kBlock;
        d_table = (int*)dalloc(B * table_stride * 4);
        TZ_CUDA(cudaMallocHost(&h_table, B * table_stride * sizeof(int)));
        std::memset(h_table, 0, B * table_stride * sizeof(int));
        n_blocks.assign(batch, 0);
        for (int i = total_blocks - 1; i >= 0; --i) free_blocks.push_back(i);     // TenzoEngine.h:128-134
    }
    cache_k = (int8_t*)dalloc(B * kv_rows_per_seq * 128);
    cache_v = (int8_t*)dalloc(B * kv_rows_per_seq * 128);
    scale_k = (float*)dalloc(B * kv_rows_per_seq * 4);
    scale_v = (float*)dalloc(B * kv_rows_per_seq * 4);

    // RoPE tables, computed on the host with the reference's float expressions (:466-469) so the
    // rotation is bit-identical to a CPU run.
    {
        const int half = cfg.head_dim / 2;
        std::vector<float> cs((size_t)cfg.max_seq_len * half), sn(cs.size());
        rope_tables_host(cfg.max_seq_len, cfg.head_dim, rope_theta, cs.data(), sn.data());
        rope_cos = (float*)dalloc(cs.size() * 4);
        rope_sin = (float*)dalloc(sn.size() * 4);
        TZ_CUDA(cudaMemcpyAsync(rope_cos, cs.data(), cs.size() * 4, cudaMemcpyHostToDevice, stream));
        TZ_CUDA(cudaMemcpyAsync(rope_sin, sn.data(), sn.size() * 4, cudaMemcpyHostToDevice, stream));
        TZ_CUDA(cudaStreamSynchronize(stream));
    }

    lm_scratch = dalloc(tenzo_cuda_lm_head_scratch_bytes(batch));
    gemv_ws = dalloc(tenzo_cuda_tl1_gemv_workspace_bytes(batch, h > ffn ? h : ffn));
    if (attention_mode == 1) {
        if (paged) throw std::invalid_argument("attention_mode 1 needs the contiguous KV cache (kv_mode int8_fused)");
        if (cfg.max_seq_len % 4) throw std::invalid_argument("attention_mode 1 needs max_seq_len to be a multiple of 4 (16-byte rows of scales)");
        attn_ws_bytes = tenzo_cuda_attention_workspace_bytes(batch, cfg.num_q_heads, cfg.num_kv_heads, cfg.max_seq_len);
        attn_ws = dalloc(attn_ws_bytes);
        persistent = 0;                                   // the one-kernel form has only the exact-order attention
    }

    TZ_CUDA(cudaMallocHost(&h_pin, (3 * B + 16) * sizeof(int)));
    h_tokens = h_pin;
    h_pos = h_pin + B;
    h_next = h_pin + 2 * B;
    seq_len.assign(batch, 0);
    TZ_CUDA(cudaStreamSynchronize(stream));
}

// Everything the engine owns, safe to call on a partly constructed object (the constructor calls it when it throws).
void Engine::release_all() {
    if (stream) cudaStreamSynchronize(stream);
    for (auto& kv : graphs) cudaGraphExecDestroy(kv.second);
    graphs.clear();
    for (void* p : owned) cudaFree(p);
    owned.clear();
    if (h_pin) cudaFreeHost(h_pin);
    if (h_table) cudaFreeHost(h_table);
    if (h_cand) cudaFreeHost(h_cand);
    if (pc_host) cudaFreeHost(pc_host);
    h_pin = nullptr; h_table = nullptr; h_cand = nullptr; pc_host = nullptr;
    free_prefill_rows();
    if (d_sample_past) cudaFree(d_sample_past);
    if (d_history) cudaFree(d_history);
    d_sample_past = nullptr; d_history = nullptr;
    if (ev0) cudaEventDestroy(ev0);
    if (ev1) cudaEventDestroy(ev1);
    if (stream) cudaStreamDestroy(stream);
    ev0 = ev1 = nullptr;
    stream = nullptr;
}

Engine::~Engine() { release_all(); }

void Engine::free_prefill_rows() {
    void** ptrs[] = {(void**)&pf_x, (void**)&pf_qkv, (void**)&pf_attn, (void**)&pf_h1, (void**)&pf_act, (void**)&pf_tokens, (void**)&pf_pos, &pf_ws};
    for (void** p : ptrs) {
        if (*p) cudaFree(*p);
        *p = nullptr;
    }
    pf_cap = 0;
}

void Engine::reserve_blocks(int s, int len) {
    if (!paged) return;
    while (n_blocks[s] * kBlock < len) {
        if (free_blocks.empty()) throw std::out_of_range("the KV block pool is exhausted");   // the reference would reuse block 0 (:302)
        h_table[(size_t)s * table_stride + n_blocks[s]] = free_blocks.back();   // TenzoEngine.h:136-141
        free_blocks.pop_back();
        n_blocks[s] += 1;
        table_dirty = true;
    }
}

void Engine::release_blocks(int s, int len) {
    if (!paged) return;
    const int keep = (len + kBlock - 1) / kBlock;
    if (n_blocks[s] <= keep) return;
    TZ_CUDA(cudaStreamSynchronize(stream));               // no step in flight may still read the entries given back
    while (n_blocks[s] > keep) {
        n_blocks[s] -= 1;
        free_blocks.push_back(h_table[(size_t)s * table_stride + n_blocks[s]]);   // TenzoEngine.h:143-147
    }
}

// Entries are only ever added between two synchronising calls (reset_kv, release_blocks), so a copy still queued
// behind earlier steps may carry newer entries without harm: those steps do not read them.
void Engine::prepare_kv(int extra) {
    if (!paged) return;
    for (int s = 0; s < batch; ++s) reserve_blocks(s, seq_len[s] + extra);
    if (table_dirty) {
        TZ_CUDA(cudaMemcpyAsync(d_table, h_table, (size_t)batch * table_stride * sizeof(int), cudaMemcpyHostToDevice, stream));
        table_dirty = false;
    }
}

void Engine::reset_kv() {                                  // TenzoEngine.cpp:242-246
    for (auto& n : seq_len) n = 0;
    if (!paged) return;
    TZ_CUDA(cudaStreamSynchronize(stream));
    free_blocks.clear();
    for (int i = total_blocks - 1; i >= 0; --i) free_blocks.push_back(i);
    n_blocks.assign(batch, 0);
}

size_t Engine::kv_row(int s, int layer, int kvh, int t) const {
    if (paged) {
        const size_t blk = (size_t)h_table[(size_t)s * table_stride + t / kBlock];
        return ((blk * L + layer) * cfg.num_kv_heads + kvh) * kBlock + (size_t)(t % kBlock);
    }
    return (size_t)s * kv_rows_per_seq + ((size_t)layer * cfg.num_kv_heads + kvh) * cfg.max_seq_len + t;
}

void* Engine::upload(const void* host, size_t bytes) {
    void* p = nullptr;
    TZ_CUDA(cudaMalloc(&p, bytes));
    owned.push_back(p);
    TZ_CUDA(cudaMemcpy(p, host, bytes, cudaMemcpyHostToDevice));
    return p;
}

void Engine::set_layer(int l, const tenzo_layer_weights_t& w) {
    if (!w.q_w || !w.k_w || !w.v_w || !w.out_w) throw std::invalid_argument("q/k/v/out weights are required");
    LayerDev& d = layers[l];
    const size_t kb = (size_t)h / 4;                 // bytes per output row at K = hidden
    const size_t q_bytes = (size_t)qd * kb, kv_bytes = (size_t)kvd * kb;
    // q, k, v row blocks are laid back to back: blocks are self-contained in the TL1 layout, so
    // the concatenation is itself a valid [60 blocks][K/2][32] matrix (one launch, one LUT, :1547).
    if (!d.qkv) { TZ_CUDA(cudaMalloc((void**)&d.qkv, q_bytes + 2 * kv_bytes)); owned.push_back(d.qkv); }
    TZ_CUDA(cudaMemcpy(d.qkv, w.q_w, q_bytes, cudaMemcpyHostToDevice));
    TZ_CUDA(cudaMemcpy(d.qkv + q_bytes, w.k_w, kv_bytes, cudaMemcpyHostToDevice));
    TZ_CUDA(cudaMemcpy(d.qkv + q_bytes + kv_bytes, w.v_w, kv_bytes, cudaMemcpyHostToDevice));
    if (!d.o) { TZ_CUDA(cudaMalloc((void**)&d.o, (size_t)h * kb)); owned.push_back(d.o); }
    TZ_CUDA(cudaMemcpy(d.o, w.out_w, (size_t)h * kb, cudaMemcpyHostToDevice));
    d.has_mlp = w.gate_w && w.up_w && w.down_w;      // :1593
    if (d.has_mlp) {
        const size_t f_bytes = (size_t)ffn * kb, down_bytes = (size_t)h * ffn / 4;
        if (!d.gateup) { TZ_CUDA(cudaMalloc((void**)&d.gateup, 2 * f_bytes)); owned.push_back(d.gateup); }
        TZ_CUDA(cudaMemcpy(d.gateup, w.gate_w, f_bytes, cudaMemcpyHostToDevice));
        TZ_CUDA(cudaMemcpy(d.gateup + f_bytes, w.up_w, f_bytes, cudaMemcpyHostToDevice));
        if (!d.down) { TZ_CUDA(cudaMalloc((void**)&d.down, down_bytes)); owned.push_back(d.down); }
        TZ_CUDA(cudaMemcpy(d.down, w.down_w, down_bytes, cudaMemcpyHostToDevice));
    }
    d.s_q = w.q_scale; d.s_k = w.k_scale; d.s_v = w.v_scale; d.s_o = w.out_scale;
    d.s_gate = w.gate_scale; d.s_up = w.up_scale; d.s_down = w.down_scale;
    auto norm = [&](float*& dst, const float* src, int n) {
        if (!src) { dst = nullptr; return; }
        if (!dst) { TZ_CUDA(cudaMalloc((void**)&dst, (size_t)n * 4)); owned.push_back(dst); }
        TZ_CUDA(cudaMemcpy(dst, src, (size_t)n * 4, cudaMemcpyHostToDevice));
    };
    norm(d.in_norm, w.in_norm, h);
    norm(d.attn_sub_norm, w.attn_sub_norm, h);
    norm(d.post_norm, w.post_norm, h);
    norm(d.ffn_sub_norm, w.ffn_sub_norm, ffn);
    d.set = true;
    invalidate_graphs();
}

void Engine::set_final_norm(const float* w) {
    if (!final_norm) final_norm = (float*)upload(w, (size_t)h * 4);
    else TZ_CUDA(cudaMemcpy(final_norm, w, (size_t)h * 4, cudaMemcpyHostToDevice));
    invalidate_graphs();
}

void Engine::set_lm_head(const int8_t* w, const float* scales) {
    if (!lm_w) {
        lm_w = (int8_t*)upload(w, (size_t)V * h);
        lm_scales = (float*)upload(scales, (size_t)V * 4);
    } else {
        TZ_CUDA(cudaMemcpy(lm_w, w, (size_t)V * h, cudaMemcpyHostToDevice));
        TZ_CUDA(cudaMemcpy(lm_scales, scales, (size_t)V * 4, cudaMemcpyHostToDevice));
    }
    invalidate_graphs();
}

void Engine::invalidate_graphs() {
    pc_built = false;                      // the persistent kernel's layer table is rebuilt from the new pointers
    if (graphs.empty()) return;
    cudaStreamSynchronize(stream);
    for (auto& kv : graphs) cudaGraphExecDestroy(kv.second);
    graphs.clear();
}

void Engine::enqueue_layer(int l, int max_len, bool gemv_only) {
    const LayerDev& d = layers[l];
    if (!d.set) throw std::runtime_error("layer weights were never set");
    tenzo_tl1_gemv_args g;
    std::memset(&g, 0, sizeof g);
    g.eps = 1e-5f;
    g.do_norm = 1;
    g.batch = batch;
    g.use_pdl = use_pdl;
    g.workspace = gemv_ws;

    // q | k | v
    g.x = b_x; g.x_stride = h; g.norm_w = d.in_norm; g.w = d.qkv; g.K = h;
    g.n_blocks = (qd + 2 * kvd) / 64;
    g.seg_end[0] = qd / 64; g.seg_end[1] = (qd + kvd) / 64; g.seg_end[2] = g.n_blocks;
    g.seg_scale[0] = d.s_q; g.seg_scale[1] = d.s_k; g.seg_scale[2] = d.s_v;
    g.epilogue = TENZO_EPI_STORE; g.out = b_qkv; g.out_stride = qd + 2 * kvd;
    g.prefetch = d.o; g.prefetch_bytes = (size_t)h * h / 4;
    const int gemv_kernels = batch > 1 ? 2 : 1;      // several sequences: quantiser kernel + GEMM kernel
    TZ_KERNEL(tenzo_cuda_tl1_gemv(&g, stream));
    launches += gemv_kernels;

    tenzo_attention_args a;
    std::memset(&a, 0, sizeof a);
    a.q = b_qkv; a.k = b_qkv + qd; a.v = b_qkv + qd + kvd;
    a.out = b_attn;
    a.cache_k = cache_k; a.cache_v = cache_v; a.scale_k = scale_k; a.scale_v = scale_v;
    a.seq_stride_kv = kv_rows_per_seq * 128; a.seq_stride_sc = kv_rows_per_seq;
    a.pos = d_pos; a.rope_cos = rope_cos; a.rope_sin = rope_sin;
    a.layer = l; a.n_q = cfg.num_q_heads; a.n_kv = cfg.num_kv_heads; a.head_dim = 128;
    a.max_seq = cfg.max_seq_len; a.batch = batch; a.max_len = max_len; a.append = 1;
    a.use_pdl = use_pdl;
    a.q_stride = a.kv_stride = qd + 2 * kvd;
    if (paged) { a.block_table = d_table; a.table_stride = table_stride; a.n_layers = L; a.n_pool_blocks = total_blocks; }
    a.mode = attention_mode; a.workspace = attn_ws; a.workspace_bytes = attn_ws_bytes;
    if (!gemv_only) {
        TZ_KERNEL(tenzo_cuda_attention_int8(&a, stream));
        launches += attention_mode == 1 ? 3 : 1;          // tolerance mode: append, split kernel, merge
    }

    // out projection + residual
    g.x = b_attn; g.x_stride = qd; g.norm_w = d.attn_sub_norm; g.w = d.o; g.K = h;
    g.n_blocks = h / 64; g.seg_end[0] = g.seg_end[1] = g.seg_end[2] = g.n_blocks; g.seg_scale[0] = d.s_o;
    g.epilogue = TENZO_EPI_RESIDUAL; g.resid = b_x; g.out = b_h1; g.out_stride = h;
    const LayerDev* nxt = l + 1 < L ? &layers[l + 1] : nullptr;
    if (d.has_mlp) { g.prefetch = d.gateup; g.prefetch_bytes = (size_t)2 * ffn * h / 4; }
    else { g.prefetch = nxt ? nxt->qkv : nullptr; g.prefetch_bytes = (size_t)(qd + 2 * kvd) * h / 4; }
    TZ_KERNEL(tenzo_cuda_tl1_gemv(&g, stream));
    launches += gemv_kernels;

    if (d.has_mlp) {
        g.x = b_h1; g.x_stride = h; g.norm_w = d.post_norm; g.w = d.gateup; g.K = h;
        g.n_blocks = 2 * ffn / 64; g.seg_end[0] = ffn / 64; g.seg_end[1] = g.seg_end[2] = g.n_blocks;
        g.seg_scale[0] = d.s_gate; g.seg_scale[1] = d.s_up;
        g.epilogue = TENZO_EPI_RELU2_GLU; g.resid = nullptr; g.out = b_act; g.out_stride = ffn;
        g.prefetch = d.down; g.prefetch_bytes = (size_t)h * ffn / 4;
        TZ_KERNEL(tenzo_cuda_tl1_gemv(&g, stream));

        g.x = b_act; g.x_stride = ffn; g.norm_w = d.ffn_sub_norm; g.w = d.down; g.K = ffn;
        g.n_blocks = h / 64; g.seg_end[0] = g.seg_end[1] = g.seg_end[2] = g.n_blocks; g.seg_scale[0] = d.s_down;
        g.epilogue = TENZO_EPI_RESIDUAL; g.resid = b_h1; g.out = b_x; g.out_stride = h;
        if (nxt) { g.prefetch = nxt->qkv; g.prefetch_bytes = (size_t)(qd + 2 * kvd) * h / 4; }
        else { g.prefetch = lm_w; g.prefetch_bytes = (size_t)64 << 20; if ((size_t)V * h < g.prefetch_bytes) g.prefetch_bytes = (size_t)V * h; }
        TZ_KERNEL(tenzo_cuda_tl1_gemv(&g, stream));
        launches += 2 * gemv_kernels;
    } else {
        TZ_CUDA(cudaMemcpyAsync(b_x, b_h1, (size_t)batch * h * 4, cudaMemcpyDeviceToDevice, stream));   // :1630
    }
}

void Engine::enqueue_step(bool with_logits, bool feed_back, int max_len) {
    if (!lm_w) throw std::runtime_error("LM head / embedding was never set");
    TZ_KERNEL(tenzo_cuda_embedding_i8(lm_w, lm_scales, h, d_tokens, batch, b_x, h, V, stream));
    launches += 1;
    for (int l = 0; l < L; ++l) enqueue_layer(l, max_len);
    if (with_logits) {
        TZ_KERNEL(tenzo_cuda_lm_head_i8(b_x, final_norm, 1, 1e-5f, lm_w, lm_scales, V, h, batch, h, b_logits, nullptr,
                                        d_next, lm_scratch, use_pdl, stream));
        launches += batch >= 16 && h % 128 == 0 ? 3 : 2;   // (quantiser +) LM head + argmax finish
    }
    advance_kernel<<<(batch + 127) / 128, 128, 0, stream>>>(d_pos, d_tokens, d_next, batch, feed_back ? 1 : 0, V);
    TZ_CUDA(cudaGetLastError());
    launches += 1;
}

static int bucket_for(int len, int max_seq);

// Chunked prefill of one sequence: M prompt tokens go through every layer together - the TL1 layers as GEMMs over the
// M rows, the K/V rows appended first, then causal attention as M independent queries over the same cache (token i sees
// keys 0..pos0+i). Row i of every product is the same arithmetic as feeding token i alone, so the cache and the state
// after the chunk are bit-identical to M calls of prefill().
void Engine::prefill_chunk(const int* tokens, int M) {
    NvtxRange range("tenzo.prefill_chunk");
    if (batch != 1) throw std::invalid_argument("chunked prefill is for single-sequence engines");
    if (M <= 0) return;
    if (!lm_w) throw std::runtime_error("LM head / embedding was never set");
    if (seq_len[0] + M > cfg.max_seq_len) throw std::out_of_range("KV cache is full (max_seq_len reached)");
    for (int i = 0; i < M; ++i)
        if (tokens[i] < 0 || tokens[i] >= V) throw std::out_of_range("token id outside [0, vocab_size)");
    if (M > pf_cap) {
        // Free first, forget the old pointers, and claim the new capacity only once every allocation has succeeded: a
        // failed cudaMalloc must leave the engine with no rows rather than with freed ones.
        free_prefill_rows();
        const size_t m = (size_t)M;
        try {
            TZ_CUDA(cudaMalloc((void**)&pf_x, m * h * 4));
            TZ_CUDA(cudaMalloc((void**)&pf_qkv, m * (qd + 2 * kvd) * 4));
            TZ_CUDA(cudaMalloc((void**)&pf_attn, m * qd * 4));
            TZ_CUDA(cudaMalloc((void**)&pf_h1, m * h * 4));
            TZ_CUDA(cudaMalloc((void**)&pf_act, m * ffn * 4));
            TZ_CUDA(cudaMalloc((void**)&pf_tokens, m * 4));
            TZ_CUDA(cudaMalloc((void**)&pf_pos, m * 4));
            TZ_CUDA(cudaMalloc(&pf_ws, tenzo_cuda_tl1_gemv_workspace_bytes(M > 1 ? M : 2, h > ffn ? h : ffn)));
        } catch (...) {
            free_prefill_rows();
            throw;
        }
        pf_cap = M;
    }
    const int pos0 = seq_len[0];
    prepare_kv(M);
    std::vector<int> hp(M);
    for (int i = 0; i < M; ++i) hp[i] = pos0 + i;
    TZ_CUDA(cudaMemcpyAsync(pf_tokens, tokens, (size_t)M * 4, cudaMemcpyHostToDevice, stream));
    TZ_CUDA(cudaMemcpyAsync(pf_pos, hp.data(), (size_t)M * 4, cudaMemcpyHostToDevice, stream));
    TZ_CUDA(cudaEventRecord(ev0, stream));
    TZ_KERNEL(tenzo_cuda_embedding_i8(lm_w, lm_scales, h, pf_tokens, M, pf_x, h, V, stream));
    launches += 1;
    const int gemv_kernels = M > 1 ? 2 : 1;
    const int max_len = bucket_for(pos0 + M, cfg.max_seq_len);
    for (int l = 0; l < L; ++l) {
        const LayerDev& d = layers[l];
        if (!d.set) throw std::runtime_error("layer weights were never set");
        tenzo_tl1_gemv_args g;
        std::memset(&g, 0, sizeof g);
        g.do_norm = 1; g.eps = 1e-5f; g.batch = M; g.workspace = pf_ws; g.use_pdl = 0;
        g.x = pf_x; g.x_stride = h; g.norm_w = d.in_norm; g.w = d.qkv; g.K = h;
        g.n_blocks = (qd + 2 * kvd) / 64;
        g.seg_end[0] = qd / 64; g.seg_end[1] = (qd + kvd) / 64; g.seg_end[2] = g.n_blocks;
        g.seg_scale[0] = d.s_q; g.seg_scale[1] = d.s_k; g.seg_scale[2] = d.s_v;
        g.epilogue = TENZO_EPI_STORE; g.out = pf_qkv; g.out_stride = qd + 2 * kvd;
        TZ_KERNEL(tenzo_cuda_tl1_gemv(&g, stream));
        const size_t layer_row_base = (size_t)l * cfg.num_kv_heads * cfg.max_seq_len;
        kv_append_rows_kernel<<<dim3((unsigned)M, (unsigned)cfg.num_kv_heads), 64, 0, stream>>>(
            pf_qkv, qd + 2 * kvd, qd, kvd, cfg.num_kv_heads, pos0, rope_cos, rope_sin, cache_k, cache_v, scale_k, scale_v, layer_row_base,
            cfg.max_seq_len, paged ? d_table : nullptr, L, l);
        TZ_CUDA(cudaGetLastError());
        tenzo_attention_args a;
        std::memset(&a, 0, sizeof a);
        a.q = pf_qkv; a.out = pf_attn; a.q_stride = a.kv_stride = qd + 2 * kvd;
        a.cache_k = cache_k; a.cache_v = cache_v; a.scale_k = scale_k; a.scale_v = scale_v;
        a.seq_stride_kv = 0; a.seq_stride_sc = 0;          // every query row reads the one sequence's cache
        a.pos = pf_pos; a.rope_cos = rope_cos; a.rope_sin = rope_sin;
        a.layer = l; a.n_q = cfg.num_q_heads; a.n_kv = cfg.num_kv_heads; a.head_dim = 128;
        a.max_seq = cfg.max_seq_len; a.batch = M; a.max_len = max_len; a.append = 0; a.tiles = 2;
        if (paged) { a.block_table = d_table; a.table_stride = 0; a.n_layers = L; a.n_pool_blocks = total_blocks; }      // every query row reads sequence 0's table
        TZ_KERNEL(tenzo_cuda_attention_int8(&a, stream));
        g.x = pf_attn; g.x_stride = qd; g.norm_w = d.attn_sub_norm; g.w = d.o; g.K = h;
        g.n_blocks = h / 64; g.seg_end[0] = g.seg_end[1] = g.seg_end[2] = g.n_blocks; g.seg_scale[0] = d.s_o;
        g.epilogue = TENZO_EPI_RESIDUAL; g.resid = pf_x; g.out = pf_h1; g.out_stride = h;
        TZ_KERNEL(tenzo_cuda_tl1_gemv(&g, stream));
        launches += 2 * gemv_kernels + 2;
        if (d.has_mlp) {
            g.x = pf_h1; g.x_stride = h; g.norm_w = d.post_norm; g.w = d.gateup; g.K = h;
            g.n_blocks = 2 * ffn / 64; g.seg_end[0] = ffn / 64; g.seg_end[1] = g.seg_end[2] = g.n_blocks;
            g.seg_scale[0] = d.s_gate; g.seg_scale[1] = d.s_up;
            g.epilogue = TENZO_EPI_RELU2_GLU; g.resid = nullptr; g.out = pf_act; g.out_stride = ffn;
            TZ_KERNEL(tenzo_cuda_tl1_gemv(&g, stream));
            g.x = pf_act; g.x_stride = ffn; g.norm_w = d.ffn_sub_norm; g.w = d.down; g.K = ffn;
            g.n_blocks = h / 64; g.seg_end[0] = g.seg_end[1] = g.seg_end[2] = g.n_blocks; g.seg_scale[0] = d.s_down;
            g.epilogue = TENZO_EPI_RESIDUAL; g.resid = pf_h1; g.out = pf_x; g.out_stride = h;
            TZ_KERNEL(tenzo_cuda_tl1_gemv(&g, stream));
            launches += 2 * gemv_kernels;
        } else {
            TZ_CUDA(cudaMemcpyAsync(pf_x, pf_h1, (size_t)M * h * 4, cudaMemcpyDeviceToDevice, stream));   // :1630
        }
    }
    // the engine's single-token state after the chunk: residual stream of the last token, position
    TZ_CUDA(cudaMemcpyAsync(b_x, pf_x + (size_t)(M - 1) * h, (size_t)h * 4, cudaMemcpyDeviceToDevice, stream));
    TZ_CUDA(cudaEventRecord(ev1, stream));
    TZ_CUDA(cudaStreamSynchronize(stream));
    seq_len[0] += M;
    check_device_status(false);
}

static int bucket_for(int len, int max_seq) {
    int b = 256;
    while (b < len) b <<= 1;
    return b < max_seq ? b : max_seq;
}

// One step for all sequences. The graph key is (with_logits, feed_back, attention bucket).
void Engine::run_step(bool with_logits, bool feed_back) {
    int longest = 0;
    for (int s = 0; s < batch; ++s) {
        if (seq_len[s] + 1 > cfg.max_seq_len) throw std::out_of_range("KV cache is full (max_seq_len reached)");
        longest = seq_len[s] + 1 > longest ? seq_len[s] + 1 : longest;
    }
    const int max_len = bucket_for(longest, cfg.max_seq_len);
    prepare_kv(1);
    if (pc_usable() && longest <= pc_score_cap(max_len)) {
        pc_step(with_logits, feed_back, max_len);
    } else if (!use_graph) {
        enqueue_step(with_logits, feed_back, max_len);
    } else {
        const int key = (with_logits ? 1 : 0) | (feed_back ? 2 : 0) | (max_len << 2);
        auto it = graphs.find(key);
        if (it == graphs.end()) {
            const unsigned long long before = launches;
            cudaGraph_t graph = nullptr;
            TZ_CUDA(cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal));
            try {
                enqueue_step(with_logits, feed_back, max_len);
            } catch (...) {
                cudaStreamEndCapture(stream, &graph);
                if (graph) cudaGraphDestroy(graph);
                launches = before;
                throw;
            }
            TZ_CUDA(cudaStreamEndCapture(stream, &graph));
            cudaGraphExec_t exec = nullptr;
            cudaError_t e = cudaGraphInstantiate(&exec, graph, 0);
            cudaGraphDestroy(graph);
            if (e != cudaSuccess) throw CudaError(e, "cudaGraphInstantiate");
            graph_kernels[key] = launches - before;
            launches = before;
            it = graphs.emplace(key, exec).first;
        }
        TZ_CUDA(cudaGraphLaunch(it->second, stream));
        launches += graph_kernels[key];
    }
    for (int s = 0; s < batch; ++s) seq_len[s] += 1;   // :1831-1835, once per token
}

void Engine::push_state(const int* tokens) {
    for (int s = 0; s < batch; ++s) {
        if (tokens) {
            if (tokens[s] < 0 || tokens[s] >= V) throw std::out_of_range("token id outside [0, vocab_size)");
            h_tokens[s] = tokens[s];
        }
        h_pos[s] = seq_len[s];
    }
    if (tokens) TZ_CUDA(cudaMemcpyAsync(d_tokens, h_tokens, (size_t)batch * 4, cudaMemcpyHostToDevice, stream));
    TZ_CUDA(cudaMemcpyAsync(d_pos, h_pos, (size_t)batch * 4, cudaMemcpyHostToDevice, stream));
}

// The TL1 kernel's waits on asynchronous copies are bounded; a give-up is reported here instead of
// hanging the device. Polled sparsely on the per-token path (the query synchronises).
void Engine::check_device_status(bool force) {
    // The flags live in device memory, so reading them costs a few synchronising copies: every call for batched engines
    // (a step there is milliseconds), every 32nd token on the single-sequence kernel chain.
    if (!force && batch == 1 && (++status_poll & 31) != 0) return;
    if (tenzo_cuda_attention_take_timeouts() > 0)
        throw std::runtime_error("an attention kernel gave up waiting for a KV copy or refused a position outside its bound; results are invalid");
    if (tenzo_cuda_lm_head_take_timeouts() > 0) throw std::runtime_error("the LM head kernel gave up waiting for a tile copy; results are invalid");
    if (tenzo_cuda_tl1_gemv_take_timeouts() > 0) throw std::runtime_error("a TL1 kernel gave up waiting for its weight copy; results are invalid");
}

void Engine::prefill(const int* tokens) {
    NvtxRange range("tenzo.prefill_token");
    push_state(tokens);
    TZ_CUDA(cudaEventRecord(ev0, stream));
    run_step(false, false);
    TZ_CUDA(cudaEventRecord(ev1, stream));
    TZ_CUDA(cudaStreamSynchronize(stream));
    pc_check();
}

void Engine::generate(const int* cur, int* out) {
    NvtxRange range("tenzo.generate_step");
    if (pc_usable() && seq_len[0] + 1 <= pc_score_cap(bucket_for(seq_len[0] + 1, cfg.max_seq_len))) {
        // persistent kernel: token and position travel as kernel arguments, the result comes back through a mapped
        // host word - no copies in either direction
        if (!cur || cur[0] < 0 || cur[0] >= V) throw std::out_of_range("token id outside [0, vocab_size)");
        pc_token_arg = cur[0];
        pc_pos_arg = seq_len[0];
        TZ_CUDA(cudaEventRecord(ev0, stream));
        try {
            run_step(true, false);
        } catch (...) {
            pc_token_arg = pc_pos_arg = -1;
            throw;
        }
        pc_token_arg = pc_pos_arg = -1;
        TZ_CUDA(cudaEventRecord(ev1, stream));
        TZ_CUDA(cudaStreamSynchronize(stream));
        pc_check();
        out[0] = pc_host[1];
        return;
    }
    push_state(cur);
    TZ_CUDA(cudaEventRecord(ev0, stream));
    run_step(true, false);
    TZ_CUDA(cudaEventRecord(ev1, stream));
    TZ_CUDA(cudaMemcpyAsync(h_next, d_next, (size_t)batch * 4, cudaMemcpyDeviceToHost, stream));
    TZ_CUDA(cudaStreamSynchronize(stream));
    check_device_status(false);
    for (int s = 0; s < batch; ++s) out[s] = h_next[s];
}

void Engine::decode_greedy(const int* first, int n_steps, int* out) {
    NvtxRange range("tenzo.decode_greedy");
    if (n_steps <= 0) return;
    if ((size_t)n_steps * batch > history_cap) {
        if (d_history) cudaFree(d_history);
        d_history = nullptr;
        TZ_CUDA(cudaMalloc((void**)&d_history, (size_t)n_steps * batch * 4));
        history_cap = (size_t)n_steps * batch;
    }
    push_state(first);
    TZ_CUDA(cudaEventRecord(ev0, stream));
    for (int i = 0; i < n_steps; ++i) {
        run_step(true, true);
        record_tokens_kernel<<<(batch + 127) / 128, 128, 0, stream>>>(d_next, d_history, i, batch);
        launches += 1;
    }
    TZ_CUDA(cudaEventRecord(ev1, stream));
    TZ_CUDA(cudaMemcpyAsync(out, d_history, (size_t)n_steps * batch * 4, cudaMemcpyDeviceToHost, stream));
    TZ_CUDA(cudaStreamSynchronize(stream));
    pc_check();
    check_device_status(true);
}

void Engine::kv_fill(int len, unsigned long long seed) {
    const size_t rows = (size_t)batch * kv_rows_per_seq;
    // block pools: every row of every block is filled, then each sequence is given the blocks that hold `len` tokens
    kv_fill_kernel<<<148 * 16, 256, 0, stream>>>(cache_k, cache_v, scale_k, scale_v, rows, paged ? 1 : cfg.max_seq_len, paged ? 1 : len, seed);
    TZ_CUDA(cudaGetLastError());
    TZ_CUDA(cudaStreamSynchronize(stream));
    for (int s = 0; s < batch; ++s) {
        release_blocks(s, len);
        reserve_blocks(s, len);
        seq_len[s] = len;
    }
}

float Engine::bench_gemv_stack(int iters, unsigned long long* n_launches) {
    const unsigned long long before = launches;
    cudaGraph_t graph = nullptr;
    TZ_CUDA(cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal));
    try {
        for (int l = 0; l < L; ++l) enqueue_layer(l, 1, true);
    } catch (...) {
        cudaStreamEndCapture(stream, &graph);
        if (graph) cudaGraphDestroy(graph);
        launches = before;
        throw;
    }
    TZ_CUDA(cudaStreamEndCapture(stream, &graph));
    const unsigned long long per_iter = launches - before;
    launches = before;
    cudaGraphExec_t exec = nullptr;
    cudaError_t e = cudaGraphInstantiate(&exec, graph, 0);
    cudaGraphDestroy(graph);
    if (e != cudaSuccess) throw CudaError(e, "cudaGraphInstantiate");
    TZ_CUDA(cudaEventRecord(ev0, stream));
    for (int i = 0; i < iters; ++i) {
        e = cudaGraphLaunch(exec, stream);
        if (e != cudaSuccess) break;
    }
    cudaEventRecord(ev1, stream);
    cudaError_t es = cudaStreamSynchronize(stream);
    cudaGraphExecDestroy(exec);
    if (e != cudaSuccess) throw CudaError(e, "cudaGraphLaunch");
    if (es != cudaSuccess) throw CudaError(es, "cudaStreamSynchronize");
    launches += per_iter * iters;
    if (n_launches) *n_launches = per_iter * iters;
    return last_ms();
}


// ---- the persistent single-sequence kernel (decode_persistent.cu) ------------------------------------------------------
// Keys the kernel's attention phase has room for at this bucket (0 when the shapes do not fit it at all).
int Engine::pc_score_cap(int max_len) {
    PcSmemPlan pl;
    if (!pc_plan(h, qd, kvd, ffn, cfg.num_q_heads, cfg.num_kv_heads, V, L, max_len, pc_grid, &pl)) return 0;
    return pl.score_cap;
}

bool Engine::pc_usable() {
    if (!persistent || batch != 1 || paged) return false;
    if (pc_built) return pc_ok;
    pc_built = true;
    pc_ok = false;
    if (!lm_w) return false;
    for (const LayerDev& d : layers)
        if (!d.set || !d.has_mlp) return false;
    if (!pc_grid) pc_grid = pc_grid_size();
    PcSmemPlan pl;
    if (!pc_grid || !pc_plan(h, qd, kvd, ffn, cfg.num_q_heads, cfg.num_kv_heads, V, L, 256 < cfg.max_seq_len ? 256 : cfg.max_seq_len, pc_grid, &pl))
        return false;
    if (!pc_layers) {
        auto dalloc = [&](size_t bytes) -> void* {
            void* ptr = nullptr;
            TZ_CUDA(cudaMalloc(&ptr, bytes));
            owned.push_back(ptr);
            TZ_CUDA(cudaMemsetAsync(ptr, 0, bytes, stream));
            return ptr;
        };
        pc_layers = (PcLayer*)dalloc((size_t)L * sizeof(PcLayer));
        pc_acc = (int32_t*)dalloc(pc_acc_ints(h, qd, kvd, ffn) * sizeof(int32_t));
        pc_bar = (unsigned*)dalloc(256);
        pc_status = (int*)dalloc(256);
        pc_best = (LmBest*)dalloc((size_t)pc_grid * sizeof(LmBest));
        pc_phase_ns = (unsigned long long*)dalloc(72 * sizeof(unsigned long long));
        TZ_CUDA(cudaHostAlloc((void**)&pc_host, 64, cudaHostAllocMapped));
        std::memset(pc_host, 0, 64);
        TZ_CUDA(cudaHostGetDevicePointer((void**)&pc_host_dev, pc_host, 0));
        pc_bar_base = 0;
    }
    std::vector<PcLayer> tab(L);
    for (int l = 0; l < L; ++l) {
        const LayerDev& d = layers[l];
        PcLayer& t = tab[l];
        t.qkv = d.qkv; t.o = d.o; t.gu = d.gateup; t.down = d.down;
        t.in_norm = d.in_norm; t.attn_sub_norm = d.attn_sub_norm; t.post_norm = d.post_norm; t.ffn_sub_norm = d.ffn_sub_norm;
        t.s_q = d.s_q; t.s_k = d.s_k; t.s_v = d.s_v; t.s_o = d.s_o; t.s_gate = d.s_gate; t.s_up = d.s_up; t.s_down = d.s_down;
    }
    TZ_CUDA(cudaStreamSynchronize(stream));
    TZ_CUDA(cudaMemcpy(pc_layers, tab.data(), (size_t)L * sizeof(PcLayer), cudaMemcpyHostToDevice));
    pc_ok = true;
    return true;
}

void Engine::pc_step(bool with_logits, bool feed_back, int max_len) {
    PcParams p;
    std::memset(&p, 0, sizeof p);
    if (!pc_plan(h, qd, kvd, ffn, cfg.num_q_heads, cfg.num_kv_heads, V, L, max_len, pc_grid, &p.plan))
        throw std::runtime_error("the persistent decode kernel does not fit this context length");
    p.layers = pc_layers;
    p.n_layers = L; p.h = h; p.qd = qd; p.kvd = kvd; p.ffn = ffn; p.V = V;
    p.n_q = cfg.num_q_heads; p.n_kv = cfg.num_kv_heads; p.max_seq = cfg.max_seq_len;
    p.lm_w = lm_w; p.lm_scales = lm_scales; p.final_norm = final_norm;
    p.tokens = d_tokens; p.pos = d_pos; p.token_arg = pc_token_arg; p.pos_arg = pc_pos_arg;
    p.next = d_next; p.host_next = pc_host_dev + 1;
    p.cache_k = cache_k; p.cache_v = cache_v; p.scale_k = scale_k; p.scale_v = scale_v;
    p.rope_cos = rope_cos; p.rope_sin = rope_sin;
    p.acc = pc_acc; p.attn_out = b_attn;
    p.b_x = b_x; p.b_qkv = b_qkv; p.b_h1 = b_h1; p.b_act = b_act; p.b_logits = b_logits;
    p.cta_best = pc_best;
    p.bar_counter = pc_bar; p.bar_base = pc_bar_base;
    p.status = pc_status; p.host_status = pc_host_dev;
    p.phase_ns = pc_phase_ns;
    p.with_logits = with_logits ? 1 : 0;
    p.feed_back = feed_back ? 1 : 0;
    p.eps = 1e-5f;
    TZ_CUDA(pc_launch(p, pc_grid, stream));
    pc_bar_base += (unsigned)pc_barriers_per_launch(L) * (unsigned)pc_grid;
    launches += 1;
}

// The barrier word and the accumulators are only consistent after a launch that ran to its end: start over.
void Engine::pc_reset_scratch() {
    if (!pc_layers) return;
    cudaStreamSynchronize(stream);
    cudaMemset(pc_bar, 0, 256);
    cudaMemset(pc_status, 0, 256);
    cudaMemset(pc_acc, 0, pc_acc_ints(h, qd, kvd, ffn) * sizeof(int32_t));
    pc_host[0] = 0;
    pc_bar_base = 0;
}

void Engine::pc_check() {
    if (!pc_host || pc_host[0] == 0) return;
    const int code = pc_host[0];
    pc_reset_scratch();
    static const char* what[] = {"", "a grid-wide barrier", "a weight copy", "a value-cache copy", "a position inside its bounds"};
    throw std::runtime_error(std::string("the persistent decode kernel gave up waiting for ") + (code >= 1 && code <= 4 ? what[code] : "something") +
                             "; results of that step are invalid");
}

float Engine::last_ms() {
    float ms = 0.0f;
    if (cudaEventElapsedTime(&ms, ev0, ev1) != cudaSuccess) return -1.0f;
    return ms;
}

// The reference sampler (TenzoEngine.cpp:1722-1807) on host logits, for the stochastic path and
// for greedy decoding with a repetition penalty. Candidate order follows std::pair<float,int>.
// The reference's streaming top-k, softmax, top-p and draw (TenzoEngine.cpp:1745-1806) over pairs in ascending index order.
int sample_pairs(const float* vals, const int* idxs, int n_in, const tenzo_sampling_params_t& p, float r_in) {
    if (n_in <= 0) return 0;
    if (p.temperature <= 0.0f) {                          // first maximum (:1746-1755)
        int best = 0;
        for (int i = 1; i < n_in; ++i)
            if (vals[i] > vals[best]) best = i;
        return idxs ? idxs[best] : best;
    }
    const int top_k = p.top_k < 1 ? 1 : (p.top_k > 64 ? 64 : p.top_k);
    float cl[64];
    int ci[64], n = 0;
    for (int j = 0; j < n_in; ++j) {                      // sorted insert = the min-heap of (value, index) pairs, :1760-1768
        const float l = vals[j];
        const int i = idxs ? idxs[j] : j;
        if (n == top_k) {
            if (!(l > cl[n - 1])) continue;
            --n;
        }
        int q = n;
        while (q > 0 && (cl[q - 1] < l || (!(l < cl[q - 1]) && ci[q - 1] < i))) { cl[q] = cl[q - 1]; ci[q] = ci[q - 1]; --q; }
        cl[q] = l; ci[q] = i; ++n;
    }
    float probs[64], sum = 0.0f;
    for (int i = 0; i < n; ++i) { probs[i] = std::exp((cl[i] - cl[0]) / p.temperature); sum += probs[i]; }
    for (int i = 0; i < n; ++i) probs[i] /= sum;
    float cum = 0.0f;
    int cut = n;
    for (int i = 0; i < n; ++i) { cum += probs[i]; if (cum >= p.top_p) { cut = i + 1; break; } }
    float sub = 0.0f;
    for (int i = 0; i < cut; ++i) sub += probs[i];
    for (int i = 0; i < cut; ++i) probs[i] /= sub;
    const float r = r_in >= 0.0f ? r_in : static_cast<float>(std::rand()) / static_cast<float>(RAND_MAX);   // :1800, process-global rand()
    float acc = 0.0f;
    for (int i = 0; i < cut; ++i) { acc += probs[i]; if (r <= acc) return ci[i]; }
    return ci[0];
}

// Penalty, k-th-largest selection and candidate compaction on the device (sampler.cu), the rest on the host.
int Engine::sample(const tenzo_sampling_params_t& p, const int* past, int n_past) {
    if (batch != 1) throw std::invalid_argument("sampling with parameters is per sequence");
    if (p.repetition_penalty != 1.0f && past && n_past > 0) {
        std::map<int, int> mult;                          // once per occurrence (:1736-1742)
        for (int i = 0; i < n_past; ++i) ++mult[past[i]];
        std::vector<int> toks, cnts;
        for (auto& kv : mult) { toks.push_back(kv.first); cnts.push_back(kv.second); }
        const size_t n = toks.size();
        if (n > sample_past_cap) {
            if (d_sample_past) cudaFree(d_sample_past);
            sample_past_cap = n * 2;
            TZ_CUDA(cudaMalloc((void**)&d_sample_past, sample_past_cap * 2 * sizeof(int)));
        }
        TZ_CUDA(cudaMemcpyAsync(d_sample_past, toks.data(), n * 4, cudaMemcpyHostToDevice, stream));
        TZ_CUDA(cudaMemcpyAsync(d_sample_past + sample_past_cap, cnts.data(), n * 4, cudaMemcpyHostToDevice, stream));
        TZ_CUDA(launch_penalty(b_logits, V, d_sample_past, d_sample_past + sample_past_cap, (int)n, p.repetition_penalty, stream));
        launches += 1;
    }
    const int k = p.temperature <= 0.0f ? 1 : (p.top_k < 1 ? 1 : (p.top_k > 64 ? 64 : p.top_k));
    if (!d_cand) {
        TZ_CUDA(cudaMalloc((void**)&d_cand, 16 + (size_t)kMaxCandidates * 8));
        owned.push_back(d_cand);
        TZ_CUDA(cudaMallocHost((void**)&h_cand, 16 + (size_t)kMaxCandidates * 8));
    }
    int* d_count = reinterpret_cast<int*>(d_cand);
    float* d_val = reinterpret_cast<float*>(static_cast<unsigned char*>(d_cand) + 16);
    int* d_idx = reinterpret_cast<int*>(d_val + kMaxCandidates);
    TZ_CUDA(launch_select_candidates(b_logits, V, k, d_count, d_val, d_idx, stream));
    launches += 1;
    TZ_CUDA(cudaMemcpyAsync(h_cand, d_cand, 16 + (size_t)kMaxCandidates * 8, cudaMemcpyDeviceToHost, stream));
    TZ_CUDA(cudaStreamSynchronize(stream));
    const int count = *reinterpret_cast<const int*>(h_cand);
    const float* hv = reinterpret_cast<const float*>(static_cast<unsigned char*>(h_cand) + 16);
    const int* hi = reinterpret_cast<const int*>(hv + kMaxCandidates);
    if (count > kMaxCandidates) {                         // a huge tie at the threshold: take the whole vector
        std::vector<float> lg((size_t)V);
        TZ_CUDA(cudaMemcpy(lg.data(), b_logits, lg.size() * 4, cudaMemcpyDeviceToHost));
        return sample_pairs(lg.data(), nullptr, V, p, -1.0f);
    }
    return sample_pairs(hv, hi, count, p, -1.0f);
}

}  // namespace tz
