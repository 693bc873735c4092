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

    def __init__(self, model: synth.SyntheticModel, max_seq_len: int | None = None, kind: str = "kernels", kv_mode: str = "int8_fused",
                 device: bytes = b"cpu"):
        self.L = ora.load_ref(kind)
        self.model = model
        self.cfg = model.config_struct(kv_mode=kv_mode, **({"max_seq_len": max_seq_len} if max_seq_len else {}))
        self.cfg.device = device
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

    def __init__(self, model: synth.SyntheticModel, max_seq_len: int | None = None, rope_theta: float = 10000.0,
                 kv_mode: str = "int8_fused"):
        self.O = ora.load_oracle()
        c = model.cfg
        self.cfg = ora.OraConfig(c["hidden_size"], c["num_q_heads"], c["num_kv_heads"], c["head_dim"], c["num_layers"],
                                 c["ffn_dim"], c["vocab_size"], max_seq_len or c["max_seq_len"], rope_theta)
        self.e = self.O.ora_engine_create(C.byref(self.cfg))
        if kv_mode == "paged_int8":
            self.O.ora_engine_use_paged_kv(self.e)
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


def best_cpu_engine(model, max_seq_len=None, kv_mode="int8_fused"):
    """The compiled reference when it is present (it is the authority), else the C oracle."""
    if ora.ref_available("kernels"):
        return RefEngine(model, max_seq_len, kv_mode=kv_mode)
    return OracleEngine(model, max_seq_len, kv_mode=kv_mode)


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


# ---- checkpoint files in the reference's format (weights.bin + model.mlir) ---------------------------------
def tl1_to_export_rows(packed: np.ndarray, n: int, k: int) -> np.ndarray:
    """TL1-packed ternary matrix -> the exporter's [N/4][K] bytes (four rows per byte, 2-bit value+1; TenzoEngine.cpp:1849-1859)."""
    code = (synth.unpack_tl1(packed, n, k).astype(np.int16) + 1).astype(np.uint8).reshape(n // 4, 4, k)
    return (code[:, 0] | (code[:, 1] << 2) | (code[:, 2] << 4) | (code[:, 3] << 6)).astype(np.uint8)


def loader_quantised_embedding(emb: np.ndarray):
    """What the loader makes of an fp32 embedding table: per-row absmax/127 scales and rounded int8 (TenzoEngine.cpp:1932-1943)."""
    amax = np.maximum(np.abs(emb).max(axis=1), np.float32(1e-8)).astype(np.float32)
    scale = (amax / np.float32(127.0)).astype(np.float32)
    inv = (np.float32(1.0) / scale).astype(np.float32)
    y = (emb * inv[:, None]).astype(np.float32)
    q = np.clip(np.sign(y) * np.floor(np.abs(y) + np.float32(0.5)), -127, 127)
    return q.astype(np.int8), scale


def write_checkpoint(model: synth.SyntheticModel, weights_path, mlir_path, with_manifest: bool = True, gap: int = 0):
    """Write `model` as weights.bin + model.mlir. The embedding table is the dequantised tied LM head. With a manifest
    every tensor gets a memref.view offset (tensors `gap` bytes apart) and every matrix its scale constant; without,
    the tensors sit back to back and the loader's scales default to 1. Returns the fp32 embedding table written."""
    c = model.cfg
    emb = (model.lm_w.astype(np.float32) * model.lm_scales[:, None]).astype(np.float32)
    blobs = [emb.tobytes()]
    order = [("in_norm", None), ("q", "q"), ("k", "k"), ("v", "v"), ("attn_sub_norm", None), ("out", "out"), ("post_norm", None),
             ("gate", "gate"), ("up", "up"), ("ffn_sub_norm", None), ("down", "down")]
    scales = []
    for lw in model.layers:
        for name, mat in order:
            if mat is None:
                blobs.append(lw[name].astype(np.float32).tobytes())
            else:
                n, k = model.shapes[mat]
                blobs.append(tl1_to_export_rows(lw[mat + "_w"], n, k).tobytes())
                scales.append(np.float32(lw[mat + "_scale"]))
    blobs.append(model.final_norm.astype(np.float32).tobytes())
    offsets, data, pos = [], bytearray(), 0
    for i, b in enumerate(blobs):
        pad = gap if (with_manifest and i > 0) else 0
        data += b"\xAA" * pad
        pos += pad
        offsets.append(pos)
        data += b
        pos += len(b)
    with open(weights_path, "wb") as f:
        f.write(bytes(data))
    lines = ["module {", "  func.func @main(%buf: memref<?xi8>) {"]
    if with_manifest:
        for i, off in enumerate(offsets):
            lines.append(f"    %c{i} = arith.constant {off} : index")
            lines.append(f"    %v{i} = memref.view %buf[%c{i}][] : memref<?xi8> to memref<{len(blobs[i])}xi8>")
        for i, s in enumerate(scales):
            lines.append(f"    %s{i} = arith.constant {float(s):.9e} : f32")
            lines.append(f"    %y{i} = \"tenzo.bitlinear_elut\"(%x{i}, %v{i}, %s{i}) : (memref<?xf32>, memref<?xi8>, f32) -> memref<?xf32>")
    lines += ["    return", "  }", "}"]
    with open(mlir_path, "w") as f:
        f.write("\n".join(lines) + "\n")
    return emb
