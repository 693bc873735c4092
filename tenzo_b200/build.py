"""Build libtenzo_runtime.so (the sm_100a CUDA kernels + engine + C ABI) in-tree with nvcc.

    python -m tenzo_b200.build            # build if stale
    python -m tenzo_b200.build --force

nvcc cross-compiles without a GPU. Flags that matter for results: -fmad=false (no silent FMA
contraction; the reference's CPU arithmetic rounds products and sums separately unless it uses an
explicit fused intrinsic) and no fast-math (IEEE division, sqrt, round-half-away).
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "lib" / "libtenzo_runtime.so"
SOURCES = ["tl1_gemv.cu", "tl1_umma.cu", "norm_quant.cu", "attention.cu", "attention_fast.cu", "lm_head.cu", "lm_head_umma.cu", "sampler.cu", "decode_persistent.cu", "engine.cu", "capi.cu",
           "cuda_runtime_hal.cu", "model_loader.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-fmad=false", "-Xcompiler", "-fPIC,-fvisibility=hidden,-O2", "-Xptxas", "-v",
]


def nvcc_path() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.sep not in cand or os.path.exists(cand)):
            return cand
    raise RuntimeError("nvcc not found")


def stale() -> bool:
    if not LIB.exists():
        return True
    t = LIB.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + \
        list((PKG.parent / "include").glob("*.h")) + [Path(__file__)]
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not stale():
        return LIB
    LIB.parent.mkdir(parents=True, exist_ok=True)
    objdir = PKG / "lib" / "obj"
    objdir.mkdir(exist_ok=True)
    nvcc = nvcc_path()
    procs = []
    for src in SOURCES:
        obj = objdir / (src[:-3] + ".o")
        cmd = [nvcc, *NVCC_FLAGS, *os.environ.get("TENZO_NVCC_EXTRA", "").split(), "-c", str(CSRC / src), "-o", str(obj)]
        procs.append((src, obj, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    objs, log = [], []
    for src, obj, p in procs:
        out, _ = p.communicate()
        log.append(f"== {src}\n{out}")
        if p.returncode != 0:
            sys.stderr.write("\n".join(log))
            raise RuntimeError(f"nvcc failed on {src}")
        objs.append(str(obj))
    (PKG / "lib" / "ptxas.log").write_text("\n".join(log))
    if verbose:
        print("\n".join(log))
    link = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(LIB), *objs, "-cudart", "static"]
    r = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout)
        raise RuntimeError("link failed")
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("-v", "--verbose", action="store_true")
    a = ap.parse_args()
    print(build(a.force, a.verbose))
