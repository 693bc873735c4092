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


class Guarded:
    """Device buffers with 256 bytes of 0xA5 in front and behind, standing in for a memory checker: a kernel that writes
    one element outside the buffer it was given trips check()."""

    PAD = 256

    def __init__(self):
        self.raws = []

    def empty(self, shape, dtype, fill=None) -> torch.Tensor:
        n = int(np.prod(shape)) * torch.empty((), dtype=dtype).element_size()
        raw = torch.full((self.PAD + n + self.PAD,), 0xA5, dtype=torch.uint8, device="cuda")
        self.raws.append((raw, n))
        view = raw[self.PAD:self.PAD + n].view(dtype).view(*shape)
        if fill is not None:
            view.copy_(fill)
        return view

    def check(self):
        torch.cuda.synchronize()
        for i, (raw, n) in enumerate(self.raws):
            assert bool((raw[:self.PAD] == 0xA5).all()), f"buffer {i}: bytes in FRONT of it were written"
            assert bool((raw[self.PAD + n:] == 0xA5).all()), f"buffer {i}: bytes BEHIND it were written"
