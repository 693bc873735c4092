"""Helpers for the gpu-marked parity tests (device staging via torch; arithmetic only in the library)."""
from __future__ import annotations

import numpy as np
import torch
from helpers import ora

P = ora.ptr


def dev(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().numpy()


def cpu_bitlinear(x: np.ndarray, w: np.ndarray, N: int, K: int, scale: float):
    """(out, acc, inv) from the compiled reference when present, else the C oracle."""
    out, acc = np.zeros(N, np.float32), np.zeros(N, np.int32)
    if ora.ref_available("kernels"):
        inv = ora.load_ref("kernels").refk_bitlinear_tl1(P(x, ora.c_f32p), P(w.view(np.int8), ora.c_i8p), N, K, float(scale),
                                                         P(out, ora.c_f32p), P(acc, ora.c_i32p))
    else:
        inv = ora.load_oracle().ora_bitlinear_tl1(P(x, ora.c_f32p), P(w, ora.c_u8p), N, K, float(scale), P(out, ora.c_f32p),
                                                  P(acc, ora.c_i32p))
    return out, acc, np.float32(inv)


def cpu_rms_norm(x: np.ndarray, w: np.ndarray | None, eps: float = 1e-5) -> np.ndarray:
    y = np.zeros_like(x)
    O = ora.load_oracle()
    O.ora_rms_norm(P(x, ora.c_f32p), P(w, ora.c_f32p) if w is not None else None, P(y, ora.c_f32p), x.size, eps)
    return y
