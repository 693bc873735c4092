"""Python mirror of the reference's RAII wrapper ``tenzo::Engine`` (include/tenzo.hpp:18-94).

Same method names, arguments and error behaviour (a non-success status raises RuntimeError, as the
C++ wrapper throws std::runtime_error), plus the batched / device-resident calls of tenzo_ext.h.
Every method is one C-ABI call into libtenzo_runtime.so.
"""
from __future__ import annotations

import ctypes as C
from typing import Sequence

import numpy as np

from . import abi, load_library


def _p(a: np.ndarray | None, ty):
    if a is None:
        return C.cast(None, ty)
    if not a.flags["C_CONTIGUOUS"]:
        raise ValueError("array must be C-contiguous")
    return a.ctypes.data_as(ty)


class Engine:
    def __init__(self, config: abi.TenzoConfig | None = None, *, batch: int = 1, rope_theta: float = 10000.0,
                 use_graph: int = -1, use_pdl: int = -1, persistent: int = -1, attention_mode: int = -1, **overrides):
        self.lib = load_library()
        cfg = config if config is not None else self.lib.tenzo_default_config()
        for k, v in overrides.items():
            setattr(cfg, k, v)
        self.config = cfg
        opt = abi.TenzoExtOptions(batch, rope_theta, use_graph, use_pdl, persistent, attention_mode)
        self._h = self.lib.tenzo_ext_create_engine(C.byref(cfg), C.byref(opt))
        if not self._h:
            raise RuntimeError("Failed to initialize Tenzo execution engine: " + self.last_error())
        self.batch = batch

    # -- lifetime ---------------------------------------------------------------------------
    def close(self):
        if getattr(self, "_h", None):
            self.lib.tenzo_destroy_engine(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def last_error(self) -> str:
        return self.lib.tenzo_ext_last_error().decode()

    def _check(self, status: int, what: str):
        if status != abi.SUCCESS:
            raise RuntimeError(f"{what} failed with status {status}: {self.last_error()}")

    # -- tenzo.hpp surface ------------------------------------------------------------------
    def load_model(self, weights_path: str, mlir_path: str):
        self._check(self.lib.tenzo_load_model(self._h, weights_path.encode(), mlir_path.encode()),
                    "Failed to load Tenzo model from " + weights_path)

    def reset(self):
        self.lib.tenzo_reset(self._h)

    def get_seq_len(self) -> int:
        return self.lib.tenzo_get_seq_len(self._h)

    def prefill_token(self, token_id: int):
        self._check(self.lib.tenzo_prefill_token(self._h, int(token_id)), "Failed to prefill token")

    def generate_step(self, cur_token: int, params: abi.TenzoSampling | None = None,
                      past_tokens: Sequence[int] = ()) -> int:
        past = np.asarray(past_tokens, dtype=np.int32)
        pp = C.byref(params) if params is not None else None
        nxt = self.lib.tenzo_generate_step(self._h, int(cur_token), pp, _p(past, abi.c_i32p) if past.size else None,
                                           int(past.size))
        if nxt < 0:
            raise RuntimeError("Failed during tenzo_generate_step: " + self.last_error())
        return nxt

    def get_raw_handle(self):
        return self._h

    # -- weight setters (tenzo.h) -------------------------------------------------------------
    def set_layer_weights(self, layer_idx: int, w: abi.TenzoLayerWeights) -> int:
        return self.lib.tenzo_set_layer_weights(self._h, layer_idx, C.byref(w))

    def set_final_norm(self, norm_w: np.ndarray) -> int:
        return self.lib.tenzo_set_final_norm(self._h, _p(norm_w, abi.c_f32p))

    def set_lm_head_i8(self, w: np.ndarray, scales: np.ndarray) -> int:
        return self.lib.tenzo_set_lm_head_i8(self._h, _p(w, abi.c_i8p), _p(scales, abi.c_f32p), w.shape[0], w.shape[1])

    def load_synthetic(self, model) -> "Engine":
        """Upload a tenzo_b200.synth.SyntheticModel through the public setters."""
        for l in range(model.cfg["num_layers"]):
            self._check(self.set_layer_weights(l, model.layer_struct(l)), f"set_layer_weights({l})")
        self._check(self.set_final_norm(model.final_norm), "set_final_norm")
        self._check(self.set_lm_head_i8(model.lm_w, model.lm_scales), "set_lm_head_i8")
        return self

    # -- tenzo_ext.h ----------------------------------------------------------------------------
    def prefill_tokens(self, tokens: Sequence[int]):
        t = np.ascontiguousarray(tokens, dtype=np.int32)
        assert t.size == self.batch
        self._check(self.lib.tenzo_ext_prefill_tokens(self._h, _p(t, abi.c_i32p)), "tenzo_ext_prefill_tokens")

    def prefill_chunk(self, tokens: Sequence[int]):
        """All of `tokens` (consecutive tokens of the one sequence) through the layers together."""
        t = np.ascontiguousarray(tokens, dtype=np.int32)
        self._check(self.lib.tenzo_ext_prefill_chunk(self._h, _p(t, abi.c_i32p), int(t.size)), "tenzo_ext_prefill_chunk")

    def generate_steps(self, cur_tokens: Sequence[int]) -> np.ndarray:
        t = np.ascontiguousarray(cur_tokens, dtype=np.int32)
        out = np.zeros(self.batch, np.int32)
        self._check(self.lib.tenzo_ext_generate_step(self._h, _p(t, abi.c_i32p), None, _p(out, abi.c_i32p)),
                    "tenzo_ext_generate_step")
        return out

    def decode_greedy(self, first_tokens: Sequence[int], n_steps: int) -> np.ndarray:
        t = np.ascontiguousarray(first_tokens, dtype=np.int32)
        out = np.zeros((n_steps, self.batch), np.int32)
        self._check(self.lib.tenzo_ext_decode_greedy(self._h, _p(t, abi.c_i32p), n_steps, _p(out, abi.c_i32p)),
                    "tenzo_ext_decode_greedy")
        return out

    def kv_import(self, seq: int, layer: int, k: np.ndarray, v: np.ndarray, sk: np.ndarray, sv: np.ndarray):
        self._check(self.lib.tenzo_ext_kv_import(self._h, seq, layer, _p(k, abi.c_i8p), _p(v, abi.c_i8p),
                                                 _p(sk, abi.c_f32p), _p(sv, abi.c_f32p), k.shape[1]), "tenzo_ext_kv_import")

    def kv_export(self, seq: int, layer: int, length: int):
        nkv, hd = self.config.num_kv_heads, self.config.head_dim
        k = np.zeros((nkv, length, hd), np.int8)
        v = np.zeros_like(k)
        sk = np.zeros((nkv, length), np.float32)
        sv = np.zeros_like(sk)
        self._check(self.lib.tenzo_ext_kv_export(self._h, seq, layer, _p(k, abi.c_i8p), _p(v, abi.c_i8p),
                                                 _p(sk, abi.c_f32p), _p(sv, abi.c_f32p), length), "tenzo_ext_kv_export")
        return k, v, sk, sv

    def kv_fill_random(self, length: int, seed: int = 0):
        self._check(self.lib.tenzo_ext_kv_fill_random(self._h, length, seed), "tenzo_ext_kv_fill_random")

    def set_seq_len(self, seq: int, length: int):
        self._check(self.lib.tenzo_ext_set_seq_len(self._h, seq, length), "tenzo_ext_set_seq_len")

    def seq_len(self, seq: int = 0) -> int:
        return self.lib.tenzo_ext_get_seq_len(self._h, seq)

    def read_buffer(self, which: int, seq: int = 0, count: int | None = None) -> np.ndarray:
        c = self.config
        sizes = {0: c.hidden_size, 2: c.num_q_heads * c.head_dim, 3: c.num_kv_heads * c.head_dim,
                 4: c.num_kv_heads * c.head_dim, 5: c.num_q_heads * c.head_dim, 8: c.hidden_size, 12: c.ffn_dim,
                 15: c.vocab_size}
        n = count if count is not None else sizes[which]
        out = np.zeros(n, np.float32)
        self._check(self.lib.tenzo_ext_read_buffer(self._h, which, seq, _p(out, abi.c_f32p), n), "tenzo_ext_read_buffer")
        return out

    def write_x(self, x: np.ndarray, seq: int = 0):
        self._check(self.lib.tenzo_ext_write_x(self._h, seq, _p(np.ascontiguousarray(x, np.float32), abi.c_f32p)),
                    "tenzo_ext_write_x")

    def run_layer(self, layer: int):
        self._check(self.lib.tenzo_ext_run_layer(self._h, layer), "tenzo_ext_run_layer")

    def synchronize(self):
        self._check(self.lib.tenzo_ext_synchronize(self._h), "tenzo_ext_synchronize")

    def last_device_ms(self) -> float:
        return float(self.lib.tenzo_ext_last_device_ms(self._h))

    def persistent_phase_ns(self, reset: bool = True):
        """Per-phase nanoseconds of the persistent single-sequence kernel since the last reset, or None when the engine
        runs the per-operator kernel chain."""
        out = (C.c_ulonglong * 8)()
        self.lib.tenzo_ext_persistent_phase_ns.restype = C.c_int
        self.lib.tenzo_ext_persistent_phase_ns.argtypes = [C.c_void_p, C.POINTER(C.c_ulonglong), C.c_int]
        rc = self.lib.tenzo_ext_persistent_phase_ns(self._h, out, int(reset))
        if rc < 0:
            raise RuntimeError("tenzo_ext_persistent_phase_ns failed")
        return [int(v) for v in out] if rc == 1 else None

    def kernel_launches(self) -> int:
        return int(self.lib.tenzo_ext_kernel_launches(self._h))
