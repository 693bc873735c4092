"""The drop-in boundary, checked without a GPU: the library loads, exports every symbol the
headers declare, struct layouts match the reference's tenzo.h, and the entry points that need no
device behave as the reference's do (TenzoEngine.cpp:2088-2114, null-handle branches :2129-2200)."""
import ctypes as C
import os
import re
from pathlib import Path

import pytest
from tenzo_b200 import abi, load_library

ROOT = Path(__file__).resolve().parents[1]


@pytest.fixture(scope="module")
def lib():
    return load_library()


def declared(header: str):
    text = (ROOT / "include" / header).read_text()
    return re.findall(r"TENZO_API\s+[^;(]*?\b(tenzo_\w+)\s*\(", text)


@pytest.mark.parametrize("header,expected", [("tenzo.h", abi.ENGINE_SYMBOLS), ("tenzo_ext.h", abi.EXT_SYMBOLS),
                                             ("tenzo_kernels.h", abi.KERNEL_SYMBOLS)])
def test_every_declared_symbol_is_exported(lib, header, expected):
    names = declared(header)
    assert sorted(names) == sorted(expected), "header and abi.py disagree"
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in {header} but not exported"


def test_hal_symbols(lib):
    for n in abi.HAL_SYMBOLS:
        assert hasattr(lib, n)
    import subprocess
    out = subprocess.run(["nm", "-D", "--defined-only", "-C", str(ROOT / "tenzo_b200/lib/libtenzo_runtime.so")],
                         capture_output=True, text=True).stdout
    for m in ("tenzo::CUDARuntime::getInstance()", "tenzo::CUDARuntime::initialize()", "tenzo::CUDARuntime::executeBitLinearTL1",
              "tenzo::CUDARuntime::executeRMSNorm", "tenzo::CUDARuntime::executeGemmF32"):
        assert m in out, f"{m} missing from the dynamic symbol table"


def test_struct_layouts_match_reference_header():
    # reference include/tenzo.h:53-87 on LP64: 8 ints + 2 pointers; 3 floats + int; 7 x (ptr, float) + 4 ptr
    assert C.sizeof(abi.TenzoConfig) == 48 and abi.TenzoConfig.kv_mode.offset == 32 and abi.TenzoConfig.device.offset == 40
    assert C.sizeof(abi.TenzoSampling) == 16 and abi.TenzoSampling.top_k.offset == 8
    assert C.sizeof(abi.TenzoLayerWeights) == 7 * 16 + 4 * 8
    assert abi.TenzoLayerWeights.q_scale.offset == 8 and abi.TenzoLayerWeights.down_w.offset == 96
    assert abi.TenzoLayerWeights.in_norm.offset == 112 and abi.TenzoLayerWeights.ffn_sub_norm.offset == 136


def test_c_header_layout_agrees_with_ctypes(tmp_path):
    """Compile a probe against include/tenzo.h (and the reference's own header when present) with gcc."""
    import subprocess
    src = tmp_path / "probe.c"
    src.write_text('#include <stdio.h>\n#include <stddef.h>\n#include "tenzo.h"\nint main(){printf("%zu %zu %zu %zu %zu %zu\\n",'
                   'sizeof(tenzo_config_t),offsetof(tenzo_config_t,kv_mode),sizeof(tenzo_sampling_params_t),'
                   'sizeof(tenzo_layer_weights_t),offsetof(tenzo_layer_weights_t,down_scale),offsetof(tenzo_layer_weights_t,in_norm));return 0;}')
    outs = []
    for inc in (ROOT / "include", Path(os.environ.get("TENZO_REFERENCE", ROOT.parent / "reference")) / "include"):
        if not (inc / "tenzo.h").exists():
            continue
        exe = tmp_path / ("p_" + inc.parent.name)
        subprocess.run(["gcc", "-I", str(inc), str(src), "-o", str(exe)], check=True)
        outs.append(subprocess.run([str(exe)], capture_output=True, text=True).stdout.split())
    assert outs[0] == ["48", "32", "16", "144", "104", "112"]
    assert all(o == outs[0] for o in outs)


def test_version_and_defaults(lib):
    assert lib.tenzo_get_version() == b"1.0.0-beta.1"
    c = lib.tenzo_default_config()
    assert (c.hidden_size, c.num_q_heads, c.num_kv_heads, c.head_dim, c.num_layers, c.ffn_dim, c.vocab_size, c.max_seq_len) == \
        (2560, 20, 5, 128, 30, 6912, 128256, 8192)
    assert c.kv_mode == b"int8_fused" and c.device == b"cpu"
    p = lib.tenzo_default_sampling_params()
    assert (round(p.temperature, 6), round(p.top_p, 6), p.top_k, round(p.repetition_penalty, 6)) == (0.7, 0.9, 40, 1.15)
    o = lib.tenzo_ext_default_options()
    assert o.batch == 1 and o.rope_theta == 10000.0


def test_null_handle_behaviour(lib):
    assert lib.tenzo_get_seq_len(None) == 0
    lib.tenzo_reset(None)
    lib.tenzo_destroy_engine(None)
    w = abi.TenzoLayerWeights()
    assert lib.tenzo_set_layer_weights(None, 0, C.byref(w)) == abi.ERR_INVALID
    assert lib.tenzo_set_final_norm(None, None) == abi.ERR_INVALID
    assert lib.tenzo_set_lm_head_i8(None, None, None, 1, 1) == abi.ERR_INVALID
    assert lib.tenzo_set_lm_head_f32(None, None, 1, 1) == abi.ERR_INVALID
    assert lib.tenzo_load_model(None, b"a", b"b") == abi.ERR_INVALID
    assert lib.tenzo_prefill_token(None, 0) == abi.ERR_INVALID
    assert lib.tenzo_generate_step(None, 0, None, None, 0) == -1


def test_kernel_entry_points_reject_bad_arguments_without_a_device(lib):
    assert lib.tenzo_cuda_tl1_gemv(None, None) == abi.ERR_INVALID
    g = abi.Tl1GemvArgs()
    assert lib.tenzo_cuda_tl1_gemv(C.byref(g), None) == abi.ERR_INVALID
    assert lib.tenzo_cuda_attention_int8(None, None) == abi.ERR_INVALID
    assert lib.tenzo_cuda_lm_head_i8(None, None, 1, 1e-5, None, None, 0, 0, 0, 0, None, None, None, None, 0, None) == abi.ERR_INVALID
    assert lib.tenzo_cuda_tl1_gemv_ksplit(40, 2560, 0) >= 1
    # tensor-core GEMM, BitNet-2B shapes at 64 sequences: out / down / q|k|v split K over a cluster of four, gate|up (108 tiles) does not
    assert [lib.tenzo_cuda_tl1_gemm_ksplit(n, k, 64, e) for n, k, e in ((40, 2560, 1), (40, 6912, 1), (60, 2560, 0), (216, 2560, 2))] == [4, 4, 4, 1]
    assert lib.tenzo_cuda_tl1_gemm_ksplit(2, 16384, 17, 0) == 8 and lib.tenzo_cuda_tl1_gemm_ksplit(40, 2560, 8, 0) == 0
    assert lib.tenzo_cuda_attention_heads_per_cta(1, 20, 5, 256) == 1 and lib.tenzo_cuda_attention_heads_per_cta(64, 20, 5, 8192) == 4


def test_tensor_core_gemm_layout_invariants(lib):
    """What the batched GEMM's hand-offs rely on, for every batch it can be given: the ring has a multiple of four slots
    (slot s then always belongs to expand group s % 4 and issuing thread s % 4, so each barrier's phases are seen in order
    by one waiter - a parity wait cannot tell phase k from phase k - 2), at least four of them, the A slots fit in tensor
    memory beside the accumulators, everything fits in an SM's shared memory, and the two rings can hold what the
    epilogue assembles in them."""
    for batch in list(range(16, 273)) + [300, 1000, 4096]:
        slots, groups, smem, epi = C.c_int(), C.c_int(), C.c_size_t(), C.c_size_t()
        assert lib.tenzo_cuda_tl1_gemm_layout(batch, C.byref(slots), C.byref(groups), C.byref(smem), C.byref(epi)) == 0
        n_box = (min(batch, 256) + 15) // 16 * 16
        assert slots.value % 4 == 0 and 4 <= slots.value <= 16, (batch, slots.value)
        assert (n_box + 31) // 32 * 32 + 32 * slots.value <= 512, "accumulators + A slots exceed tensor memory"
        assert groups.value in (2, 3)
        assert smem.value <= 227 * 1024, (batch, smem.value)
        rings = slots.value * n_box * 128 + groups.value * 8 * 4096
        assert rings + 1024 < smem.value                 # plus alignment slack, barriers, per-sequence operands
        assert epi.value <= rings, (batch, epi.value, rings)
    assert lib.tenzo_cuda_tl1_gemm_layout(15, None, None, None, None) == -1


def test_engine_creation_fails_loudly_without_a_gpu(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    assert not lib.tenzo_create_engine(None)
    assert b"no CPU path" in lib.tenzo_ext_last_error() or b"CUDA" in lib.tenzo_ext_last_error()
