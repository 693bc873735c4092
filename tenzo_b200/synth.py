"""Seeded synthetic weights with the shapes and value distributions of the benchmark configs.

Real BitNet checkpoints are not available offline; these stand in for them. Ternary weights are
i.i.d. uniform over {-1,0,+1}; since a TL1 nibble is (w0+1)|((w1+1)<<2), drawing each nibble
uniformly from its nine legal values is the same distribution and lets the packed bytes be
generated directly (no 2-billion-entry ternary matrix is ever materialised). The per-tensor
weight scale is mean|W| of a seeded latent N(0, 0.02^2) sample. The tied INT8 embedding / LM head
is a latent N(0, sigma_e^2) table quantised per row (amax/127, clamp +-127), which is what the
reference's loader does to an fp32 embedding (src/runtime/TenzoEngine.cpp:1934-1946).
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import abi

NIBBLES = np.array([0, 1, 2, 4, 5, 6, 8, 9, 10], dtype=np.uint8)
# byte value for each of the 81 (low nibble, high nibble) pairs
_BYTE81 = (NIBBLES[:, None] | (NIBBLES[None, :] << 4)).reshape(-1).astype(np.uint8)

BITNET_2B = dict(hidden_size=2560, num_q_heads=20, num_kv_heads=5, head_dim=128, num_layers=30, ffn_dim=6912,
                 vocab_size=128256, max_seq_len=8192)
SYNTH_8B = dict(hidden_size=4096, num_q_heads=32, num_kv_heads=8, head_dim=128, num_layers=32, ffn_dim=14336,
                vocab_size=128256, max_seq_len=4096)
TINY = dict(hidden_size=256, num_q_heads=2, num_kv_heads=1, head_dim=128, num_layers=2, ffn_dim=384,
            vocab_size=1024, max_seq_len=128)


def random_tl1_packed(rng: np.random.Generator, n_rows: int, k_cols: int) -> np.ndarray:
    """TL1-packed [n_rows/64][k_cols/2][32] bytes of i.i.d. uniform ternary weights."""
    assert n_rows % 64 == 0 and k_cols % 2 == 0
    idx = rng.integers(0, 81, size=n_rows * k_cols // 4, dtype=np.uint8)
    return _BYTE81[idx]


def pack_tl1(tern: np.ndarray) -> np.ndarray:
    """Ternary [N][K] int8 -> TL1 layout (numpy restatement of the packing, for small test cases)."""
    n, k = tern.shape
    assert n % 64 == 0 and k % 2 == 0
    t = (tern.astype(np.int16) + 1).astype(np.uint8).reshape(n // 64, 2, 32, k // 2, 2)   # [b][half][c][kp][parity]
    nib = t[..., 0] | (t[..., 1] << 2)                                                    # [b][half][c][kp]
    byte = nib[:, 0] | (nib[:, 1] << 4)                                                   # [b][c][kp]
    return np.ascontiguousarray(byte.transpose(0, 2, 1)).reshape(-1)                      # [b][kp][c]


def unpack_tl1(packed: np.ndarray, n: int, k: int) -> np.ndarray:
    byte = packed.reshape(n // 64, k // 2, 32).transpose(0, 2, 1)                          # [b][c][kp]
    out = np.empty((n // 64, 2, 32, k // 2, 2), np.int8)
    out[:, 0, :, :, 0] = (byte & 3).astype(np.int8) - 1
    out[:, 0, :, :, 1] = ((byte >> 2) & 3).astype(np.int8) - 1
    out[:, 1, :, :, 0] = ((byte >> 4) & 3).astype(np.int8) - 1
    out[:, 1, :, :, 1] = ((byte >> 6) & 3).astype(np.int8) - 1
    return out.reshape(n, k)


def weight_scale(rng: np.random.Generator) -> np.float32:
    """mean|W| of a latent N(0, 0.02^2) sample (export_bitnet.py:182 of the reference)."""
    return np.float32(np.abs(rng.normal(0.0, 0.02, 65536).astype(np.float32)).mean())


def quantize_rows_i8(w: np.ndarray):
    amax = np.maximum(np.abs(w).max(axis=1), np.float32(1e-8)).astype(np.float32)
    scale = (amax / np.float32(127.0)).astype(np.float32)
    inv = (np.float32(1.0) / scale).astype(np.float32)
    q = np.clip(np.sign(w * inv[:, None]) * np.floor(np.abs(w * inv[:, None]) + np.float32(0.5)), -127, 127)
    return q.astype(np.int8), scale


class SyntheticModel:
    """All tensors of one model, host side, in the form the tenzo.h setters take."""

    def __init__(self, cfg: dict, seed: int = 0, sigma_e: float = 0.02):
        self.cfg = dict(cfg)
        h, f = cfg["hidden_size"], cfg["ffn_dim"]
        qd, kvd = cfg["num_q_heads"] * cfg["head_dim"], cfg["num_kv_heads"] * cfg["head_dim"]
        self.shapes = dict(q=(qd, h), k=(kvd, h), v=(kvd, h), out=(h, h), gate=(f, h), up=(f, h), down=(h, f))
        self.layers = []
        for l in range(cfg["num_layers"]):
            rng = np.random.default_rng([seed, 1000 + l])
            lw = {}
            for name, (n, k) in self.shapes.items():
                lw[name + "_w"] = random_tl1_packed(rng, n, k)
                lw[name + "_scale"] = weight_scale(rng)
            for name, dim in (("in_norm", h), ("attn_sub_norm", h), ("post_norm", h), ("ffn_sub_norm", f)):
                lw[name] = (1.0 + 0.1 * rng.standard_normal(dim)).astype(np.float32)
            self.layers.append(lw)
        rng = np.random.default_rng([seed, 7])
        self.final_norm = (1.0 + 0.1 * rng.standard_normal(h)).astype(np.float32)
        v = cfg["vocab_size"]
        self.lm_w = np.empty((v, h), np.int8)
        self.lm_scales = np.empty(v, np.float32)
        step = 8192
        for r0 in range(0, v, step):
            r1 = min(v, r0 + step)
            lat = (sigma_e * rng.standard_normal((r1 - r0, h))).astype(np.float32)
            self.lm_w[r0:r1], self.lm_scales[r0:r1] = quantize_rows_i8(lat)

    def layer_struct(self, l: int) -> abi.TenzoLayerWeights:
        lw, s = self.layers[l], abi.TenzoLayerWeights()
        for name in self.shapes:
            setattr(s, name + "_w", lw[name + "_w"].ctypes.data_as(abi.c_i8p))
            setattr(s, name + "_scale", float(lw[name + "_scale"]))
        for name in ("in_norm", "attn_sub_norm", "post_norm", "ffn_sub_norm"):
            setattr(s, name, lw[name].ctypes.data_as(abi.c_f32p))
        return s

    def config_struct(self, lib=None, **overrides) -> abi.TenzoConfig:
        c = abi.TenzoConfig()
        kv_mode = overrides.pop("kv_mode", "int8_fused")
        for k, v in {**self.cfg, **overrides}.items():
            setattr(c, k, v)
        c.kv_mode = kv_mode.encode() if isinstance(kv_mode, str) else kv_mode
        c.device = b"cpu"
        return c

    def weight_bytes_per_token(self) -> int:
        """Algorithmic bytes one decoded token streams: TL1 matrices + norm weights + LM head."""
        c = self.cfg
        tl1 = sum(n * k // 4 for n, k in self.shapes.values()) * c["num_layers"]
        norms = (3 * c["hidden_size"] + c["ffn_dim"]) * 4 * c["num_layers"] + c["hidden_size"] * 4
        lm = c["vocab_size"] * c["hidden_size"] + 4 * c["vocab_size"]
        return tl1 + norms + lm


def prompt_tokens(seed: int, n: int, vocab: int) -> np.ndarray:
    return np.random.default_rng([seed, 99]).integers(0, vocab, n, dtype=np.int32)
