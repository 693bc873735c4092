"""ctypes bindings for the CPU oracle — TEST INFRASTRUCTURE, NOT PRODUCT CODE.

Three libraries, all built by ``oracle/Makefile``:

* ``liboracle.so``                 this repo's plain-C restatement (always available; ``load_oracle``)
* ``_ref/libtenzo_ref_kernels.so`` the unmodified reference engine plus per-kernel trampolines
                                   (``load_ref_kernels``; present wherever it was built)
* ``_ref/libtenzo_ref_fast.so``    the reference built with its own default flags, for timing

Only tests, the smoke check and the benchmark's CPU-baseline leg import this module.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent

c_f32p = C.POINTER(C.c_float)
c_i8p = C.POINTER(C.c_int8)
c_u8p = C.POINTER(C.c_uint8)
c_i32p = C.POINTER(C.c_int32)


def ptr(a: np.ndarray | None, ty):
    if a is None:
        return C.cast(None, ty)
    assert a.flags["C_CONTIGUOUS"], "oracle buffers must be contiguous"
    return a.ctypes.data_as(ty)


def build_oracle(force: bool = False) -> Path:
    so = HERE / "liboracle.so"
    src_new = max((HERE / "tenzo_oracle.c").stat().st_mtime, (HERE / "tenzo_oracle.h").stat().st_mtime)
    if force or not so.exists() or so.stat().st_mtime < src_new:
        subprocess.run(["make", "-C", str(HERE), "-B", "liboracle.so"], check=True, capture_output=True)
    return so


class OraConfig(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("hidden", "n_q", "n_kv", "head_dim", "layers", "ffn", "vocab", "max_seq")] + [
        ("rope_theta", C.c_float)
    ]


class OraLayer(C.Structure):
    _fields_ = (
        [(n, c_u8p) for n in ("q_w", "k_w", "v_w", "o_w", "gate_w", "up_w", "down_w")]
        + [(n, C.c_float) for n in ("q_s", "k_s", "v_s", "o_s", "gate_s", "up_s", "down_s")]
        + [(n, c_f32p) for n in ("in_norm", "attn_sub_norm", "post_norm", "ffn_sub_norm")]
    )


_oracle = None


def load_oracle():
    """Load (building if stale) the C restatement and declare its prototypes."""
    global _oracle
    if _oracle is not None:
        return _oracle
    L = C.CDLL(str(build_oracle()))
    i64, i32, f32, vp = C.c_int64, C.c_int, C.c_float, C.c_void_p
    sig = {
        "ora_tl1_pack": (None, [c_i8p, i64, i64, c_u8p]),
        "ora_tl1_pack_from_rows2bit": (None, [c_u8p, i64, i64, c_u8p]),
        "ora_tl1_unpack": (None, [c_u8p, i64, i64, c_i8p]),
        "ora_act_quant31": (f32, [c_f32p, i64, c_i8p]),
        "ora_build_lut": (f32, [c_f32p, i64, c_i8p]),
        "ora_tl1_gemv_lut": (None, [c_i8p, c_u8p, i64, i64, c_i32p]),
        "ora_bitlinear_tl1": (f32, [c_f32p, c_u8p, i64, i64, f32, c_f32p, c_i32p]),
        "ora_rms_norm": (None, [c_f32p, c_f32p, c_f32p, i32, f32]),
        "ora_relu2_glu": (None, [c_f32p, c_f32p, c_f32p, i32]),
        "ora_rope_table": (None, [i32, i32, f32, c_f32p, c_f32p]),
        "ora_rope_apply": (None, [c_f32p, i32, i32, c_f32p, c_f32p]),
        "ora_kv_quant_row": (f32, [c_f32p, i32, c_i8p]),
        "ora_attention_int8": (None, [i32, i32, i32, i32, i32, i32, f32, c_f32p, c_f32p, c_f32p, c_f32p,
                                      c_i8p, c_i8p, c_f32p, c_f32p]),
        "ora_attention_paged_int8": (None, [i32, i32, i32, i32, i32, i32, f32, c_f32p, c_f32p, c_f32p, c_f32p,
                                            c_i8p, c_i8p, c_f32p, c_f32p, c_i32p]),
        "ora_engine_use_paged_kv": (None, [vp]),
        "ora_engine_paged_kv": (None, [vp, C.POINTER(c_i8p), C.POINTER(c_i8p), C.POINTER(c_f32p), C.POINTER(c_f32p),
                                       C.POINTER(c_i32p), C.POINTER(i32)]),
        "ora_embedding_i8": (None, [c_i8p, c_f32p, i32, i32, c_f32p]),
        "ora_act_quant127": (f32, [c_f32p, i32, c_i8p]),
        "ora_lm_head_i8": (None, [c_i8p, f32, c_i8p, c_f32p, i32, i32, c_f32p, c_i32p]),
        "ora_quantize_rows_i8": (None, [c_f32p, i32, i32, c_i8p, c_f32p]),
        "ora_sample": (i32, [c_f32p, i32, f32, f32, i32, f32, c_i32p, i32, f32]),
        "ora_engine_create": (vp, [C.POINTER(OraConfig)]),
        "ora_engine_destroy": (None, [vp]),
        "ora_engine_set_layer": (None, [vp, i32, C.POINTER(OraLayer)]),
        "ora_engine_set_final_norm": (None, [vp, c_f32p]),
        "ora_engine_set_lm_head_i8": (None, [vp, c_i8p, c_f32p]),
        "ora_engine_reset": (None, [vp]),
        "ora_engine_seq_len": (i32, [vp]),
        "ora_engine_prefill": (None, [vp, i32]),
        "ora_engine_generate": (i32, [vp, i32, f32, f32, i32, f32, c_i32p, i32, f32]),
        "ora_engine_buffer": (c_f32p, [vp, i32]),
        "ora_engine_kv": (None, [vp, C.POINTER(c_i8p), C.POINTER(c_i8p), C.POINTER(c_f32p), C.POINTER(c_f32p)]),
        "ora_engine_embedding": (None, [vp, i32]),
        "ora_engine_forward_layer": (None, [vp, i32]),
        "ora_engine_advance": (None, [vp]),
        "ora_engine_logits": (None, [vp]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(L, name)
        fn.restype, fn.argtypes = res, args
    _oracle = L
    return L


# The reference's C ABI structs (include/tenzo.h:53-87) are mirrored once, in tenzo_b200/abi.py.
from tenzo_b200.abi import TenzoConfig, TenzoSampling, TenzoLayerWeights, declare_tenzo_abi  # noqa: E402


def ref_available(kind: str = "kernels") -> bool:
    return (HERE / "_ref" / _REF_FILES[kind]).exists()


_REF_FILES = {"kernels": "libtenzo_ref_kernels.so", "fast": "libtenzo_ref_fast.so", "plain": "libtenzo_ref.so",
              "kernels_fast": "libtenzo_ref_kernels_fast.so", "cuda": "libtenzo_ref_cuda.so"}
_refs: dict[str, C.CDLL] = {}


def load_ref(kind: str = "kernels"):
    """Load a compiled-reference library: 'kernels' (parity + trampolines), 'plain', 'fast' (the reference's default
    flags, for timing), 'kernels_fast' (trampolines, default flags) or 'cuda' (the reference engine compiled against this
    repository's CUDARuntime.h and linked to libtenzo_runtime.so: its device = "cuda" path runs on the GPU)."""
    if kind in _refs:
        return _refs[kind]
    L = declare_tenzo_abi(C.CDLL(str(HERE / "_ref" / _REF_FILES[kind]), mode=os.RTLD_LOCAL))
    if kind in ("kernels", "kernels_fast", "cuda"):
        vp, i32, i64, f32 = C.c_void_p, C.c_int, C.c_int64, C.c_float
        sig = {
            "refk_build_lut": (f32, [c_f32p, i64, c_u8p]),
            "refk_bitlinear_tl1": (f32, [c_f32p, c_i8p, i64, i64, f32, c_f32p, c_i32p]),
            "refk_rms_norm": (None, [c_f32p, c_f32p, c_f32p, i32, f32]),
            "refk_kv_create": (vp, [i32, i32, i32, i32, i32]),
            "refk_kv_destroy": (None, [vp]),
            "refk_kv_set_len": (None, [vp, i32]),
            "refk_kv_k": (c_i8p, [vp]), "refk_kv_v": (c_i8p, [vp]),
            "refk_kv_k_scales": (c_f32p, [vp]), "refk_kv_v_scales": (c_f32p, [vp]),
            "refk_kv_attention": (None, [vp, i32, c_f32p, c_f32p, c_f32p, c_f32p]),
            "refk_paged_create": (vp, [i32, i32, i32, i32, i32]),
            "refk_paged_destroy": (None, [vp]),
            "refk_paged_set_len": (None, [vp, i32]),
            "refk_paged_k": (c_i8p, [vp]), "refk_paged_v": (c_i8p, [vp]),
            "refk_paged_k_scales": (c_f32p, [vp]), "refk_paged_v_scales": (c_f32p, [vp]),
            "refk_paged_table": (i32, [vp, c_i32p, i32]),
            "refk_paged_push_block": (None, [vp, i32]),
            "refk_paged_attention": (None, [vp, i32, c_f32p, c_f32p, c_f32p, c_f32p]),
            "refk_engine_paged_kv": (vp, [vp]),
            "refk_engine_buffer": (c_f32p, [vp, i32]),
            "refk_engine_x_i8": (c_i8p, [vp]),
            "refk_engine_kv": (vp, [vp]),
            "refk_engine_embedding": (None, [vp, i32]),
            "refk_engine_forward_layer": (None, [vp, i32]),
            "refk_engine_advance": (None, [vp]),
            "refk_engine_logits": (None, [vp]),
            "refk_engine_sample": (i32, [vp, C.POINTER(TenzoSampling), c_i32p, i32]),
        }
        for n, (res, args) in sig.items():
            fn = getattr(L, n)
            fn.restype, fn.argtypes = res, args
    _refs[kind] = L
    return L


def view(p, n: int, dtype) -> np.ndarray:
    """numpy view over n elements at a ctypes pointer (no copy)."""
    ct = {np.float32: C.c_float, np.int8: C.c_int8, np.int32: C.c_int32, np.uint8: C.c_uint8}[dtype]
    return np.ctypeslib.as_array(C.cast(p, C.POINTER(ct)), shape=(n,))


BUF = {n: i for i, n in enumerate(["x", "norm_x", "q", "k", "v", "attn_out", "attn_sub", "out", "h1", "post_norm",
                                   "gate", "up", "act", "ffn_norm", "down", "logits"])}
