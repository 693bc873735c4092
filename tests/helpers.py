"""Shared test plumbing: drive the compiled reference, the C oracle and the CUDA library from one
SyntheticModel. Test infrastructure only."""
from __future__ import annotations

import ctypes as C
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from oracle import oracle_py as ora  # noqa: E402
from tenzo_b200 import abi, synth  # noqa: E402


class RefEngine:
    """The unmodified reference engine (compiled by oracle/Makefile) loaded with a SyntheticModel."""

    def __init__(self, model: synth.SyntheticModel, max_seq_len: int | None = None, kind: str = "kernels"):
        self.L = ora.load_ref(kind)
        self.model = model
        self.cfg = model.config_struct(**({"max_seq_len": max_seq_len} if max_seq_len else {}))
        self.h = self.L.tenzo_create_engine(C.byref(self.cfg))
        assert self.h
        self._keep = []
        for l in range(model.cfg["num_layers"]):
            s = model.layer_struct(l)
            self._keep.append(s)
            assert self.L.tenzo_set_layer_weights(self.h, l, C.byref(s)) == 0
        assert self.L.tenzo_set_final_norm(self.h, model.final_norm.ctypes.data_as(abi.c_f32p)) == 0
        assert self.L.tenzo_set_lm_head_i8(self.h, model.lm_w.ctypes.data_as(abi.c_i8p),
                                           model.lm_scales.ctypes.data_as(abi.c_f32p), model.cfg["vocab_size"],
                                           model.cfg["hidden_size"]) == 0

    def close(self):
        if self.h:
            self.L.tenzo_destroy_engine(self.h)
            self.h = None

    def prefill(self, tok: int):
        assert self.L.tenzo_prefill_token(self.h, int(tok)) == 0

    def generate(self, tok: int, temperature=0.0, top_p=0.9, top_k=40, rep=1.0, past=()):
        p = abi.TenzoSampling(temperature, top_p, top_k, rep)
        past = np.asarray(past, np.int32)
        return self.L.tenzo_generate_step(self.h, int(tok), C.byref(p), past.ctypes.data_as(abi.c_i32p) if past.size else None,
                                          int(past.size))

    def buffer(self, name: str, n: int) -> np.ndarray:
        return ora.view(self.L.refk_engine_buffer(self.h, ora.BUF[name]), n, np.float32).copy()

    def set_buffer(self, name: str, data: np.ndarray):
        ora.view(self.L.refk_engine_buffer(self.h, ora.BUF[name]), data.size, np.float32)[:] = data

    def seq_len(self) -> int:
        return self.L.tenzo_get_seq_len(self.h)


class OracleEngine:
    """The C restatement's engine loaded with a SyntheticModel."""

    def __init__(self, model: synth.SyntheticModel, max_seq_len: int | None = None, rope_theta: float = 10000.0):
        self.O = ora.load_oracle()
        c = model.cfg
        self.cfg = ora.OraConfig(c["hidden_size"], c["num_q_heads"], c["num_kv_heads"], c["head_dim"], c["num_layers"],
                                 c["ffn_dim"], c["vocab_size"], max_seq_len or c["max_seq_len"], rope_theta)
        self.e = self.O.ora_engine_create(C.byref(self.cfg))
        self.model = model
        self._keep = []
        for l, lw in enumerate(model.layers):
            s = ora.OraLayer()
            for dst, src in (("q", "q"), ("k", "k"), ("v", "v"), ("o", "out"), ("gate", "gate"), ("up", "up"), ("down", "down")):
                setattr(s, dst + "_w", lw[src + "_w"].ctypes.data_as(ora.c_u8p))
                setattr(s, dst + "_s", float(lw[src + "_scale"]))
            for n in ("in_norm", "attn_sub_norm", "post_norm", "ffn_sub_norm"):
                setattr(s, n, lw[n].ctypes.data_as(ora.c_f32p))
            self._keep.append(s)
            self.O.ora_engine_set_layer(self.e, l, C.byref(s))
        self.O.ora_engine_set_final_norm(self.e, model.final_norm.ctypes.data_as(ora.c_f32p))
        self.O.ora_engine_set_lm_head_i8(self.e, model.lm_w.ctypes.data_as(ora.c_i8p), model.lm_scales.ctypes.data_as(ora.c_f32p))

    def close(self):
        if self.e:
            self.O.ora_engine_destroy(self.e)
            self.e = None

    def prefill(self, tok: int):
        self.O.ora_engine_prefill(self.e, int(tok))

    def generate(self, tok: int, temperature=0.0, top_p=0.9, top_k=40, rep=1.0, past=(), u=0.5):
        past = np.asarray(past, np.int32)
        return self.O.ora_engine_generate(self.e, int(tok), temperature, top_p, top_k, rep,
                                          past.ctypes.data_as(ora.c_i32p) if past.size else None, int(past.size), u)

    def buffer(self, name: str, n: int) -> np.ndarray:
        return ora.view(self.O.ora_engine_buffer(self.e, ora.BUF[name]), n, np.float32).copy()

    def set_buffer(self, name: str, data: np.ndarray):
        ora.view(self.O.ora_engine_buffer(self.e, ora.BUF[name]), data.size, np.float32)[:] = data

    def seq_len(self) -> int:
        return self.O.ora_engine_seq_len(self.e)


def best_cpu_engine(model, max_seq_len=None):
    """The compiled reference when it is present (it is the authority), else the C oracle."""
    if ora.ref_available("kernels"):
        return RefEngine(model, max_seq_len)
    return OracleEngine(model, max_seq_len)


def greedy_stream(engine, prompt, n_gen):
    """Prefill all but the last prompt token, then n_gen greedy steps (main_inference.cpp:469-492 shape)."""
    for t in prompt[:-1]:
        engine.prefill(int(t))
    cur, out = int(prompt[-1]), []
    for _ in range(n_gen):
        cur = engine.generate(cur, temperature=0.0, rep=1.0)
        out.append(cur)
    return np.asarray(out, np.int32)


def rel_err(a: np.ndarray, b: np.ndarray) -> float:
    """max|a-b| normalised by max|b| (tensor-level relative error used for every fp32 comparison)."""
    d = float(np.abs(a.astype(np.float64) - b.astype(np.float64)).max())
    return d / max(float(np.abs(b).max()), 1e-30)
