"""ctypes mirror of the engine C ABI (include/tenzo.h, include/tenzo_ext.h, include/tenzo_kernels.h).

Struct layouts follow the reference's include/tenzo.h:53-87 field for field; the same classes are
used to drive this repository's library and, in tests, the compiled reference.
"""
from __future__ import annotations

import ctypes as C

c_f32p = C.POINTER(C.c_float)
c_i8p = C.POINTER(C.c_int8)
c_u8p = C.POINTER(C.c_uint8)
c_i32p = C.POINTER(C.c_int32)
c_u32p = C.POINTER(C.c_uint32)

SUCCESS, ERR_INVALID, ERR_OOM, ERR_IO, ERR_PARSE, ERR_UNSUPPORTED = 0, -1, -2, -3, -4, -5


class TenzoConfig(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("hidden_size", "num_q_heads", "num_kv_heads", "head_dim", "num_layers",
                                       "ffn_dim", "vocab_size", "max_seq_len")] + [
        ("kv_mode", C.c_char_p), ("device", C.c_char_p)]


class TenzoSampling(C.Structure):
    _fields_ = [("temperature", C.c_float), ("top_p", C.c_float), ("top_k", C.c_int),
                ("repetition_penalty", C.c_float)]


def _layer_fields():
    f = []
    for n in ("q", "k", "v", "out", "gate", "up", "down"):
        f += [(f"{n}_w", c_i8p), (f"{n}_scale", C.c_float)]
    return f + [(n, c_f32p) for n in ("in_norm", "attn_sub_norm", "post_norm", "ffn_sub_norm")]


class TenzoLayerWeights(C.Structure):
    _fields_ = _layer_fields()


class TenzoExtOptions(C.Structure):
    _fields_ = [("batch", C.c_int), ("rope_theta", C.c_float), ("use_graph", C.c_int), ("use_pdl", C.c_int), ("persistent", C.c_int), ("attention_mode", C.c_int)]


class Tl1GemvArgs(C.Structure):
    _fields_ = [
        ("x", C.c_void_p), ("norm_w", C.c_void_p), ("do_norm", C.c_int), ("eps", C.c_float),
        ("w", C.c_void_p), ("n_blocks", C.c_int), ("K", C.c_int),
        ("seg_end", C.c_int * 3), ("seg_scale", C.c_float * 3),
        ("epilogue", C.c_int), ("resid", C.c_void_p), ("out", C.c_void_p),
        ("acc_out", C.c_void_p), ("a_out", C.c_void_p), ("inv_out", C.c_void_p),
        ("batch", C.c_int), ("x_stride", C.c_int), ("out_stride", C.c_int),
        ("prefetch", C.c_void_p), ("prefetch_bytes", C.c_size_t), ("workspace", C.c_void_p), ("use_pdl", C.c_int),
    ]


class AttentionArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("out", C.c_void_p),
        ("q_stride", C.c_int), ("kv_stride", C.c_int),
        ("cache_k", C.c_void_p), ("cache_v", C.c_void_p), ("scale_k", C.c_void_p), ("scale_v", C.c_void_p),
        ("seq_stride_kv", C.c_size_t), ("seq_stride_sc", C.c_size_t),
        ("pos", C.c_void_p), ("rope_cos", C.c_void_p), ("rope_sin", C.c_void_p),
        ("layer", C.c_int), ("n_q", C.c_int), ("n_kv", C.c_int), ("head_dim", C.c_int), ("max_seq", C.c_int),
        ("batch", C.c_int), ("max_len", C.c_int), ("append", C.c_int),
        ("heads_per_cta", C.c_int), ("use_pdl", C.c_int), ("tiles", C.c_int),
        ("block_table", C.c_void_p), ("table_stride", C.c_int), ("n_layers", C.c_int), ("n_pool_blocks", C.c_int),
        ("mode", C.c_int), ("split_keys", C.c_int), ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
    ]


ENGINE_SYMBOLS = [
    "tenzo_get_version", "tenzo_default_config", "tenzo_default_sampling_params", "tenzo_create_engine",
    "tenzo_destroy_engine", "tenzo_reset", "tenzo_get_seq_len", "tenzo_set_layer_weights", "tenzo_set_final_norm",
    "tenzo_set_lm_head_f32", "tenzo_set_lm_head_i8", "tenzo_load_model", "tenzo_prefill_token", "tenzo_generate_step",
]
EXT_SYMBOLS = [
    "tenzo_ext_default_options", "tenzo_ext_create_engine", "tenzo_ext_batch", "tenzo_ext_prefill_tokens",
    "tenzo_ext_generate_step", "tenzo_ext_decode_greedy", "tenzo_ext_kv_import", "tenzo_ext_kv_export",
    "tenzo_ext_kv_fill_random", "tenzo_ext_set_seq_len", "tenzo_ext_get_seq_len", "tenzo_ext_read_buffer",
    "tenzo_ext_write_x", "tenzo_ext_run_layer", "tenzo_ext_synchronize", "tenzo_ext_last_device_ms",
    "tenzo_ext_kernel_launches", "tenzo_ext_last_error", "tenzo_ext_bench_gemv_stack", "tenzo_ext_rope_tables", "tenzo_ext_parse_manifest", "tenzo_ext_sample_pairs", "tenzo_ext_prefill_chunk",
    "tenzo_ext_persistent_phase_ns",
]
KERNEL_SYMBOLS = [
    "tenzo_cuda_tl1_gemv", "tenzo_cuda_tl1_gemv_ksplit", "tenzo_cuda_tl1_gemm_ksplit", "tenzo_cuda_tl1_gemm_layout", "tenzo_cuda_tl1_gemv_workspace_bytes", "tenzo_cuda_tl1_gemv_take_timeouts", "tenzo_cuda_selftest_wait_expiry", "tenzo_cuda_rmsnorm_quant", "tenzo_cuda_attention_int8",
    "tenzo_cuda_attention_heads_per_cta", "tenzo_cuda_attention_take_timeouts", "tenzo_cuda_attention_workspace_bytes", "tenzo_cuda_lm_head_i8", "tenzo_cuda_lm_head_scratch_bytes",
    "tenzo_cuda_embedding_i8", "tenzo_cuda_tl1_pack_rows2bit", "tenzo_cuda_lm_head_i8_static",
    "tenzo_cuda_lm_head_static_max_batch", "tenzo_cuda_lm_head_take_timeouts", "tenzo_cuda_repetition_penalty",
    "tenzo_cuda_topk_candidates", "tenzo_cuda_topk_max_candidates",
]
HAL_SYMBOLS = ["tenzo_hal_initialize", "tenzo_hal_bitlinear_tl1_host", "tenzo_hal_rmsnorm_host", "tenzo_hal_gemm_f32_host", "tenzo_hal_call_count"]


def declare_tenzo_abi(L):
    """Attach prototypes for the 14 tenzo.h entry points to a loaded library."""
    vp, i32 = C.c_void_p, C.c_int
    L.tenzo_get_version.restype, L.tenzo_get_version.argtypes = C.c_char_p, []
    L.tenzo_default_config.restype, L.tenzo_default_config.argtypes = TenzoConfig, []
    L.tenzo_default_sampling_params.restype, L.tenzo_default_sampling_params.argtypes = TenzoSampling, []
    L.tenzo_create_engine.restype, L.tenzo_create_engine.argtypes = vp, [C.POINTER(TenzoConfig)]
    L.tenzo_destroy_engine.restype, L.tenzo_destroy_engine.argtypes = None, [vp]
    L.tenzo_reset.restype, L.tenzo_reset.argtypes = None, [vp]
    L.tenzo_get_seq_len.restype, L.tenzo_get_seq_len.argtypes = i32, [vp]
    L.tenzo_set_layer_weights.restype = i32
    L.tenzo_set_layer_weights.argtypes = [vp, i32, C.POINTER(TenzoLayerWeights)]
    L.tenzo_set_final_norm.restype, L.tenzo_set_final_norm.argtypes = i32, [vp, c_f32p]
    L.tenzo_set_lm_head_f32.restype, L.tenzo_set_lm_head_f32.argtypes = i32, [vp, c_f32p, i32, i32]
    L.tenzo_set_lm_head_i8.restype, L.tenzo_set_lm_head_i8.argtypes = i32, [vp, c_i8p, c_f32p, i32, i32]
    L.tenzo_load_model.restype, L.tenzo_load_model.argtypes = i32, [vp, C.c_char_p, C.c_char_p]
    L.tenzo_prefill_token.restype, L.tenzo_prefill_token.argtypes = i32, [vp, i32]
    L.tenzo_generate_step.restype = i32
    L.tenzo_generate_step.argtypes = [vp, i32, C.POINTER(TenzoSampling), c_i32p, i32]
    return L


def declare_ext_abi(L):
    vp, i32, f32 = C.c_void_p, C.c_int, C.c_float
    L.tenzo_ext_default_options.restype, L.tenzo_ext_default_options.argtypes = TenzoExtOptions, []
    L.tenzo_ext_create_engine.restype = vp
    L.tenzo_ext_create_engine.argtypes = [C.POINTER(TenzoConfig), C.POINTER(TenzoExtOptions)]
    L.tenzo_ext_batch.restype, L.tenzo_ext_batch.argtypes = i32, [vp]
    L.tenzo_ext_prefill_tokens.restype, L.tenzo_ext_prefill_tokens.argtypes = i32, [vp, c_i32p]
    L.tenzo_ext_generate_step.restype = i32
    L.tenzo_ext_generate_step.argtypes = [vp, c_i32p, C.POINTER(TenzoSampling), c_i32p]
    L.tenzo_ext_decode_greedy.restype, L.tenzo_ext_decode_greedy.argtypes = i32, [vp, c_i32p, i32, c_i32p]
    L.tenzo_ext_kv_import.restype = i32
    L.tenzo_ext_kv_import.argtypes = [vp, i32, i32, c_i8p, c_i8p, c_f32p, c_f32p, i32]
    L.tenzo_ext_kv_export.restype = i32
    L.tenzo_ext_kv_export.argtypes = [vp, i32, i32, c_i8p, c_i8p, c_f32p, c_f32p, i32]
    L.tenzo_ext_kv_fill_random.restype, L.tenzo_ext_kv_fill_random.argtypes = i32, [vp, i32, C.c_uint64]
    L.tenzo_ext_set_seq_len.restype, L.tenzo_ext_set_seq_len.argtypes = i32, [vp, i32, i32]
    L.tenzo_ext_get_seq_len.restype, L.tenzo_ext_get_seq_len.argtypes = i32, [vp, i32]
    L.tenzo_ext_read_buffer.restype, L.tenzo_ext_read_buffer.argtypes = i32, [vp, i32, i32, c_f32p, C.c_size_t]
    L.tenzo_ext_write_x.restype, L.tenzo_ext_write_x.argtypes = i32, [vp, i32, c_f32p]
    L.tenzo_ext_run_layer.restype, L.tenzo_ext_run_layer.argtypes = i32, [vp, i32]
    L.tenzo_ext_synchronize.restype, L.tenzo_ext_synchronize.argtypes = i32, [vp]
    L.tenzo_ext_last_device_ms.restype, L.tenzo_ext_last_device_ms.argtypes = f32, [vp]
    L.tenzo_ext_kernel_launches.restype, L.tenzo_ext_kernel_launches.argtypes = C.c_ulonglong, [vp]
    L.tenzo_ext_last_error.restype, L.tenzo_ext_last_error.argtypes = C.c_char_p, []
    L.tenzo_ext_bench_gemv_stack.restype = f32
    L.tenzo_ext_bench_gemv_stack.argtypes = [vp, i32, C.POINTER(C.c_ulonglong)]
    L.tenzo_ext_rope_tables.restype, L.tenzo_ext_rope_tables.argtypes = i32, [i32, i32, f32, c_f32p, c_f32p]
    L.tenzo_ext_sample_pairs.restype, L.tenzo_ext_sample_pairs.argtypes = i32, [c_f32p, c_i32p, i32, C.POINTER(TenzoSampling), f32]
    L.tenzo_ext_prefill_chunk.restype, L.tenzo_ext_prefill_chunk.argtypes = i32, [vp, c_i32p, i32]
    L.tenzo_ext_parse_manifest.restype = i32
    L.tenzo_ext_parse_manifest.argtypes = [C.c_char_p, C.POINTER(C.c_ulonglong), i32, C.POINTER(i32), c_f32p, i32, C.POINTER(i32)]
    return L


def declare_kernel_abi(L):
    vp, i32, f32, sz = C.c_void_p, C.c_int, C.c_float, C.c_size_t
    L.tenzo_cuda_tl1_gemv.restype, L.tenzo_cuda_tl1_gemv.argtypes = i32, [C.POINTER(Tl1GemvArgs), vp]
    L.tenzo_cuda_tl1_gemv_ksplit.restype, L.tenzo_cuda_tl1_gemv_ksplit.argtypes = i32, [i32, i32, i32]
    L.tenzo_cuda_tl1_gemm_ksplit.restype, L.tenzo_cuda_tl1_gemm_ksplit.argtypes = i32, [i32, i32, i32, i32]
    L.tenzo_cuda_tl1_gemm_layout.restype = i32
    L.tenzo_cuda_tl1_gemm_layout.argtypes = [i32, C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_size_t), C.POINTER(C.c_size_t)]
    L.tenzo_cuda_tl1_gemv_workspace_bytes.restype, L.tenzo_cuda_tl1_gemv_workspace_bytes.argtypes = sz, [i32, i32]
    L.tenzo_cuda_tl1_gemv_take_timeouts.restype, L.tenzo_cuda_tl1_gemv_take_timeouts.argtypes = i32, []
    L.tenzo_cuda_rmsnorm_quant.restype = i32
    L.tenzo_cuda_rmsnorm_quant.argtypes = [vp, vp, i32, f32, i32, i32, i32, i32, vp, vp, vp, vp]
    L.tenzo_cuda_attention_int8.restype, L.tenzo_cuda_attention_int8.argtypes = i32, [C.POINTER(AttentionArgs), vp]
    L.tenzo_cuda_attention_take_timeouts.restype, L.tenzo_cuda_attention_take_timeouts.argtypes = i32, []
    L.tenzo_cuda_attention_heads_per_cta.restype, L.tenzo_cuda_attention_heads_per_cta.argtypes = i32, [i32, i32, i32, i32]
    L.tenzo_cuda_lm_head_i8.restype = i32
    L.tenzo_cuda_lm_head_i8.argtypes = [vp, vp, i32, f32, vp, vp, i32, i32, i32, i32, vp, vp, vp, vp, i32, vp]
    L.tenzo_cuda_lm_head_i8_static.restype = i32
    L.tenzo_cuda_lm_head_i8_static.argtypes = [vp, vp, i32, f32, vp, vp, i32, i32, i32, i32, vp, vp, vp, i32, vp]
    L.tenzo_cuda_lm_head_static_max_batch.restype, L.tenzo_cuda_lm_head_static_max_batch.argtypes = i32, []
    L.tenzo_cuda_lm_head_take_timeouts.restype, L.tenzo_cuda_lm_head_take_timeouts.argtypes = i32, []
    L.tenzo_cuda_repetition_penalty.restype, L.tenzo_cuda_repetition_penalty.argtypes = i32, [vp, i32, vp, vp, i32, f32, vp]
    L.tenzo_cuda_topk_candidates.restype, L.tenzo_cuda_topk_candidates.argtypes = i32, [vp, i32, i32, vp, vp, vp, vp]
    L.tenzo_cuda_topk_max_candidates.restype, L.tenzo_cuda_topk_max_candidates.argtypes = i32, []
    L.tenzo_cuda_lm_head_scratch_bytes.restype, L.tenzo_cuda_lm_head_scratch_bytes.argtypes = sz, [i32]
    L.tenzo_cuda_embedding_i8.restype, L.tenzo_cuda_embedding_i8.argtypes = i32, [vp, vp, i32, vp, i32, vp, i32, i32, vp]
    L.tenzo_cuda_tl1_pack_rows2bit.restype, L.tenzo_cuda_tl1_pack_rows2bit.argtypes = i32, [vp, i32, i32, vp, vp]
    L.tenzo_hal_initialize.restype, L.tenzo_hal_initialize.argtypes = i32, []
    L.tenzo_hal_bitlinear_tl1_host.restype = i32
    L.tenzo_hal_bitlinear_tl1_host.argtypes = [c_f32p, c_u8p, c_f32p, sz, sz, sz, f32]
    L.tenzo_hal_rmsnorm_host.restype, L.tenzo_hal_rmsnorm_host.argtypes = i32, [c_f32p, c_f32p, c_f32p, sz, f32]
    L.tenzo_hal_gemm_f32_host.restype, L.tenzo_hal_gemm_f32_host.argtypes = i32, [c_f32p, c_f32p, c_f32p, sz, sz, sz]
    L.tenzo_hal_call_count.restype, L.tenzo_hal_call_count.argtypes = C.c_ulonglong, []
    return L
