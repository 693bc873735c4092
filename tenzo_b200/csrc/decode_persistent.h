// Single-sequence decode as ONE persistent cooperative kernel per token (decode_persistent.cu), shared with engine.cu.
//
// The kernel replaces, for batch 1, the chain of ~150 dependent launches per token (embedding, then per layer
// q|k|v GEMV, attention, out GEMV, gate|up GEMV, down GEMV, then LM head and argmax): the sequencing of
// TenzoEngineImpl::forward_layer_raw / generate_step in the reference (src/runtime/TenzoEngine.cpp:1538-1632,
// :1809-1838). Arithmetic and results are those of the per-operator kernels, bit for bit.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "lm_head.cuh"

namespace tz {

struct PcLayer {                      // one per layer, in device memory
    const uint8_t *qkv, *o, *gu, *down;                      // TL1 layouts [N/64][K/2][32]; q|k|v and gate|up back to back
    const float *in_norm, *attn_sub_norm, *post_norm, *ffn_sub_norm;   // may be null
    float s_q, s_k, s_v, s_o, s_gate, s_up, s_down;
};

struct PcSmemPlan {
    int off_sd, off_red, off_suma, off_layers, off_x, off_h1, off_sq, off_scratch, off_ring;   // byte offsets from the dynamic shared base
    int scratch_bytes, n_stages, total_bytes;
    int score_cap;                    // keys the attention phase has room for
};

struct PcParams {
    const PcLayer* layers;
    int n_layers, h, qd, kvd, ffn, V, n_q, n_kv, max_seq;
    const int8_t* lm_w;
    const float* lm_scales;
    const float* final_norm;          // may be null
    int* tokens;                      // device [1]: token to run when token_arg < 0; receives the next token when feed_back
    int* pos;                         // device [1]: position (tokens already cached); incremented by the kernel
    int token_arg;                    // >= 0: run this token (no copy into *tokens needed)
    int pos_arg;                      // >= 0: use this position instead of *pos (*pos is still set to pos_arg + 1)
    int* next;                        // device [1]: argmax of the logits (with_logits)
    int* host_next;                   // optional mapped host word receiving the same
    int8_t *cache_k, *cache_v;        // this sequence's cache: [layer][kv_head][max_seq][128]
    float *scale_k, *scale_v;         // [layer][kv_head][max_seq]
    const float *rope_cos, *rope_sin; // [max_seq][64]
    int32_t* acc;                     // zeroed scratch: q|k|v, out, gate|up, down accumulators back to back
    float* attn_out;                  // [qd] attention output of the current layer
    float *b_x, *b_qkv, *b_h1, *b_act, *b_logits;   // read-back copies of the last layer's vectors; logits [V]
    LmBest* cta_best;                 // [grid]
    unsigned* bar_counter;            // grid barrier arrivals, monotonic across launches
    unsigned bar_base;                // its value when this launch starts
    int* status;                      // device word, 0 = fine (see PC_ERR_*)
    int* host_status;                 // optional mapped host word mirroring it
    unsigned long long* phase_ns;     // optional [8]: time per phase kind summed by CTA 0 (measurement)
    int with_logits, feed_back;
    float eps;
    PcSmemPlan plan;
};

enum { PC_ERR_BARRIER = 1, PC_ERR_WEIGHT_COPY = 2, PC_ERR_VALUE_COPY = 3, PC_ERR_POSITION = 4 };

// Barriers one launch performs (the host advances bar_base by this times the grid size).
inline int pc_barriers_per_launch(int n_layers) { return 5 * n_layers + 1; }

// Ints in PcParams::acc.
inline size_t pc_acc_ints(int h, int qd, int kvd, int ffn) { return (size_t)(qd + 2 * kvd) + h + 2 * (size_t)ffn + h; }

// CTAs of the launch (one per SM) or 0 when the device cannot run the kernel (no cooperative launch).
int pc_grid_size();
// Shared-memory layout for these shapes with room for `max_len` keys; false when the shapes do not fit the kernel
// (K not a multiple of 32, hidden not a multiple of 16, too many row blocks per CTA, too little room for the weight ring).
bool pc_plan(int h, int qd, int kvd, int ffn, int n_q, int n_kv, int V, int n_layers, int max_len, int grid, PcSmemPlan* out);
cudaError_t pc_launch(const PcParams& p, int grid, cudaStream_t st);

}  // namespace tz
