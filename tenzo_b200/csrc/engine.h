// Engine state shared between engine.cu (behaviour) and capi.cu (the extern "C" boundary).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <map>
#include <string>
#include <vector>

#include "../../include/tenzo.h"
#include "../../include/tenzo_ext.h"
#include "decode_persistent.h"

namespace tz {

void rope_tables_host(int max_seq, int head_dim, float theta, float* cs, float* sn);


extern thread_local std::string g_last_error;
void set_error(const std::string& m);

struct CudaError : std::runtime_error {
    cudaError_t code;
    CudaError(cudaError_t c, const char* what) : std::runtime_error(std::string(what) + ": " + cudaGetErrorString(c)), code(c) {}
};
#define TZ_CUDA(expr)                                            \
    do {                                                         \
        cudaError_t _e = (expr);                                 \
        if (_e != cudaSuccess) throw tz::CudaError(_e, #expr);   \
    } while (0)


struct LayerDev {
    uint8_t* qkv = nullptr;      // q|k|v row blocks back to back, TL1 layout
    uint8_t* o = nullptr;
    uint8_t* gateup = nullptr;   // gate|up
    uint8_t* down = nullptr;
    float s_q = 1, s_k = 1, s_v = 1, s_o = 1, s_gate = 1, s_up = 1, s_down = 1;
    float *in_norm = nullptr, *attn_sub_norm = nullptr, *post_norm = nullptr, *ffn_sub_norm = nullptr;
    bool has_mlp = false, set = false;
};

class Engine {
public:
    Engine(const tenzo_config_t& cfg, const tenzo_ext_options_t& opt);
    ~Engine();
    void init(const tenzo_config_t& cfg, const tenzo_ext_options_t& opt);
    Engine(const Engine&) = delete;
    Engine& operator=(const Engine&) = delete;

    void set_layer(int l, const tenzo_layer_weights_t& w);
    void set_final_norm(const float* w);
    void set_lm_head(const int8_t* w, const float* scales);

    void prefill(const int* tokens);                       // one token per sequence, no logits
    void prefill_chunk(const int* tokens, int n);          // n consecutive tokens of the one sequence, together
    void generate(const int* cur, int* out);               // device argmax
    void decode_greedy(const int* first, int n_steps, int* out);
    int sample(const tenzo_sampling_params_t& p, const int* past, int n_past);   // on the logits of the last step

    void push_state(const int* tokens);
    void run_step(bool with_logits, bool feed_back);
    void enqueue_step(bool with_logits, bool feed_back, int max_len);
    void enqueue_layer(int l, int max_len, bool gemv_only = false);
    float bench_gemv_stack(int iters, unsigned long long* n_launches);
    void invalidate_graphs();
    void free_prefill_rows();
    void release_all();
    void* upload(const void* host, size_t bytes);
    float last_ms();
    void check_device_status(bool force);
    unsigned status_poll = 0;
    void kv_fill(int len, unsigned long long seed);

    // kv_mode "paged_int8" (PagedKVCache + PagedBlockManager of the reference, TenzoEngine.h:117-193): the caches are pools
    // of 16-token blocks [block][layer][kv_head][16][128]; every sequence has a row of the block table. Blocks are taken
    // from the free list on the host before the step that first writes into them (the reference does it inside layer 0,
    // TenzoEngine.cpp:294-300) and the table row is copied to the device ahead of the launch.
    static constexpr int kBlock = 16;
    bool paged = false;
    int total_blocks = 0, table_stride = 0;
    int *d_table = nullptr, *h_table = nullptr;          // [batch][table_stride]; h_table is the pinned master copy
    std::vector<int> free_blocks, n_blocks;              // free list (taken from the back: 0, 1, 2, ... as the reference's)
    bool table_dirty = false;
    void reserve_blocks(int seq, int len);               // the table of `seq` covers tokens [0, len)
    void release_blocks(int seq, int len);               // blocks past token len go back to the free list
    void prepare_kv(int extra);                          // before a step that appends `extra` tokens to every sequence
    void reset_kv();
    size_t kv_row(int seq, int layer, int kvh, int t) const;   // row of a cached token in cache_k/v (x128) and scale_k/v

    tenzo_config_t cfg;
    int batch = 1, device = 0, use_graph = 1, use_pdl = 1;
    float rope_theta = 10000.0f;
    int h = 0, qd = 0, kvd = 0, ffn = 0, L = 0, V = 0;
    cudaStream_t stream = nullptr;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    std::vector<LayerDev> layers;
    float* final_norm = nullptr;
    int8_t* lm_w = nullptr;
    float* lm_scales = nullptr;

    int *d_tokens = nullptr, *d_pos = nullptr, *d_next = nullptr, *d_history = nullptr;
    size_t history_cap = 0;
    float *b_x = nullptr, *b_qkv = nullptr, *b_attn = nullptr, *b_h1 = nullptr, *b_act = nullptr, *b_logits = nullptr;
    int8_t *cache_k = nullptr, *cache_v = nullptr;
    float *scale_k = nullptr, *scale_v = nullptr;
    size_t kv_rows_per_seq = 0;
    float *rope_cos = nullptr, *rope_sin = nullptr;
    void *lm_scratch = nullptr, *gemv_ws = nullptr;
    int attention_mode = 0;              // 1: tolerance-mode attention (attention_fast.cu) in the kernel chain
    void* attn_ws = nullptr;
    size_t attn_ws_bytes = 0;
    float *pf_x = nullptr, *pf_qkv = nullptr, *pf_attn = nullptr, *pf_h1 = nullptr, *pf_act = nullptr;   // chunked prefill rows
    int *pf_tokens = nullptr, *pf_pos = nullptr, pf_cap = 0;
    void* pf_ws = nullptr;
    void *d_cand = nullptr, *h_cand = nullptr;           // sampler: candidate count + (value, index) pairs
    int* d_sample_past = nullptr;
    size_t sample_past_cap = 0;
    int *h_pin = nullptr, *h_tokens = nullptr, *h_pos = nullptr, *h_next = nullptr;
    std::vector<int> seq_len;
    std::vector<void*> owned;
    std::map<int, cudaGraphExec_t> graphs;
    std::map<int, unsigned long long> graph_kernels;
    unsigned long long launches = 0;

    // Single-sequence engines: the whole token as one persistent cooperative kernel (decode_persistent.cu) instead of the
    // kernel chain, whenever the shapes fit it (pc_usable). Its scratch is owned here: zeroed accumulators, the barrier
    // word (only ever grows; pc_bar_base tracks it), status and result words the host can read without a copy.
    int persistent = 0;                  // option / TENZO_PERSISTENT (off unless asked for: measured slower than the kernel chain)
    bool pc_built = false, pc_ok = false;
    int pc_grid = 0;
    PcLayer* pc_layers = nullptr;
    int32_t* pc_acc = nullptr;
    unsigned* pc_bar = nullptr;
    unsigned pc_bar_base = 0;
    int* pc_status = nullptr;
    int* pc_host = nullptr;              // mapped pinned: [0] status mirror, [1] next token
    int* pc_host_dev = nullptr;          // the device's view of it
    LmBest* pc_best = nullptr;
    unsigned long long* pc_phase_ns = nullptr;
    int pc_token_arg = -1, pc_pos_arg = -1;
    int pc_score_cap(int max_len);
    bool pc_usable();                    // builds the layer table on first use; false = use the kernel chain
    void pc_step(bool with_logits, bool feed_back, int max_len);
    void pc_check();                     // after a synchronisation: throws (and re-arms the scratch) if a launch gave up
    void pc_reset_scratch();
};

}  // namespace tz

struct tenzo_engine_opaque {
    tz::Engine* impl;
};
