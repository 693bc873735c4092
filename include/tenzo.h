/* tenzo.h — engine C ABI of the B200 (sm_100a) decode runtime.
 *
 * Binary- and source-compatible with the C interface catdlia/tenzo declares in its own
 * include/tenzo.h (:39-193): the same fourteen entry points, the same three plain structs with
 * the same field order, the same status values, so a program built against the reference header
 * (or its C++ wrapper include/tenzo.hpp) links against libtenzo_runtime.so from this repository
 * unchanged. tests/test_abi.py checks sizes and field offsets against the reference layout.
 *
 * Differences in behaviour, all on the strict side:
 *   - the engine always runs on the CUDA device; `device` in the config is accepted and ignored;
 *   - kv_mode "int8_fused" (or NULL) and "paged_int8" are implemented, other modes fail engine creation;
 *   - setters copy to device memory at once, so callers may free their buffers afterwards;
 *   - out-of-range layer indices, token ids and a full KV cache are reported instead of ignored.
 */
#ifndef TENZO_H
#define TENZO_H

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#ifndef TENZO_API
#if defined(__GNUC__) && __GNUC__ >= 4
#define TENZO_API __attribute__((visibility("default")))
#else
#define TENZO_API
#endif
#endif

#define TENZO_VERSION_MAJOR 1
#define TENZO_VERSION_MINOR 0
#define TENZO_VERSION_PATCH 0
#define TENZO_VERSION_STRING "1.0.0-beta.1" /* reference tenzo.h:37 */

typedef struct tenzo_engine_opaque* tenzo_engine_t; /* reference tenzo.h:40 */

typedef enum { /* reference tenzo.h:43-50 */
    TENZO_SUCCESS = 0,
    TENZO_ERROR_INVALID_ARGUMENT = -1,
    TENZO_ERROR_OUT_OF_MEMORY = -2,
    TENZO_ERROR_IO = -3,
    TENZO_ERROR_MODEL_PARSE = -4,
    TENZO_ERROR_UNSUPPORTED = -5
} tenzo_status_t;

typedef struct { /* reference tenzo.h:53-64; defaults are BitNet-b1.58-2B-4T */
    int hidden_size;     /* 2560   */
    int num_q_heads;     /* 20     */
    int num_kv_heads;    /* 5      */
    int head_dim;        /* 128 (the only supported value) */
    int num_layers;      /* 30     */
    int ffn_dim;         /* 6912   */
    int vocab_size;      /* 128256 */
    int max_seq_len;     /* 8192   */
    const char* kv_mode; /* "int8_fused" (or NULL) or "paged_int8" */
    const char* device;  /* ignored: always the current CUDA device */
} tenzo_config_t;

typedef struct { /* reference tenzo.h:67-72 */
    float temperature;        /* 0.7; <= 0 selects greedy argmax */
    float top_p;              /* 0.9  */
    int top_k;                /* 40, clamped to 1..64 */
    float repetition_penalty; /* 1.15; applied before the argmax in greedy mode too */
} tenzo_sampling_params_t;

typedef struct { /* reference tenzo.h:75-87; *_w are HOST pointers to TL1-packed weights */
    const int8_t* q_w;    float q_scale;
    const int8_t* k_w;    float k_scale;
    const int8_t* v_w;    float v_scale;
    const int8_t* out_w;  float out_scale;
    const int8_t* gate_w; float gate_scale;
    const int8_t* up_w;   float up_scale;
    const int8_t* down_w; float down_scale;
    const float* in_norm;       /* [hidden] */
    const float* attn_sub_norm; /* [hidden] */
    const float* post_norm;     /* [hidden] */
    const float* ffn_sub_norm;  /* [ffn]    */
} tenzo_layer_weights_t;

/* reference tenzo.h:92 / TenzoEngine.cpp:2088 */
TENZO_API const char* tenzo_get_version(void);
/* reference tenzo.h:97 / TenzoEngine.cpp:2092-2105 */
TENZO_API tenzo_config_t tenzo_default_config(void);
/* reference tenzo.h:102 / TenzoEngine.cpp:2107-2114 */
TENZO_API tenzo_sampling_params_t tenzo_default_sampling_params(void);
/* reference tenzo.h:109 / TenzoEngine.cpp:2116-2121. NULL config = defaults. Returns NULL on
 * unsupported configuration or allocation failure (tenzo_ext_last_error() says which). */
TENZO_API tenzo_engine_t tenzo_create_engine(const tenzo_config_t* config);
/* reference tenzo.h:114 */
TENZO_API void tenzo_destroy_engine(tenzo_engine_t engine);
/* reference tenzo.h:119: sequence length back to 0, cache contents kept */
TENZO_API void tenzo_reset(tenzo_engine_t engine);
/* reference tenzo.h:124: 0 for a NULL engine */
TENZO_API int tenzo_get_seq_len(tenzo_engine_t engine);
/* reference tenzo.h:129-133 / TenzoEngine.cpp:1257-1277, :2139-2147 */
TENZO_API tenzo_status_t tenzo_set_layer_weights(tenzo_engine_t engine, int layer_idx,
                                                 const tenzo_layer_weights_t* weights);
/* reference tenzo.h:138 */
TENZO_API tenzo_status_t tenzo_set_final_norm(tenzo_engine_t engine, const float* norm_w);
/* reference tenzo.h:143-148: the fp32 LM head is outside the quantized path -> TENZO_ERROR_UNSUPPORTED */
TENZO_API tenzo_status_t tenzo_set_lm_head_f32(tenzo_engine_t engine, const float* embed_w,
                                               int vocab_size, int hidden_size);
/* reference tenzo.h:153-159 / TenzoEngine.cpp:1288-1292: tied INT8 embedding / LM head */
TENZO_API tenzo_status_t tenzo_set_lm_head_i8(tenzo_engine_t engine, const int8_t* embed_w,
                                              const float* embed_scales, int vocab_size, int hidden_size);
/* reference tenzo.h:167-171 / TenzoEngine.cpp:1887-2078 */
TENZO_API tenzo_status_t tenzo_load_model(tenzo_engine_t engine, const char* weights_path,
                                          const char* mlir_path);
/* reference tenzo.h:176 / TenzoEngine.cpp:1809-1819 */
TENZO_API tenzo_status_t tenzo_prefill_token(tenzo_engine_t engine, int token_id);
/* reference tenzo.h:187-193 / TenzoEngine.cpp:1821-1838: returns the next token or -1 */
TENZO_API int tenzo_generate_step(tenzo_engine_t engine, int cur_token,
                                  const tenzo_sampling_params_t* params, const int* past_tokens,
                                  int past_tokens_len);

#ifdef __cplusplus
}
#endif
#endif /* TENZO_H */
