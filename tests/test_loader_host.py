"""tenzo_load_model, host side: the manifest reader against the reference's two patterns run with Python's `re`,
and the checkpoint writer used by the GPU loader test against the compiled reference's own loader (CPU)."""
import ctypes as C
import re

import numpy as np
import pytest

from helpers import RefEngine, greedy_stream, loader_quantised_embedding, ora, synth, write_checkpoint
from tenzo_b200 import abi, load_library

VIEW_RE = re.compile(r"(%\w+)\s*=\s*arith\.constant\s+(\d+)\s*:\s*index\s*\r?\n\s*(%\w+)\s*=\s*memref\.view\s+%\w+\[\1\]\[\]\s*:\s*memref<\?xi8>\s+to\s+memref<([^>]+)>")
SCALE_RE = re.compile(r"(%\w+)\s*=\s*arith\.constant\s+([0-9\.e\+\-]+)\s*:\s*f32\s*\r?\n\s*%\w+\s*=\s*\"tenzo\.bitlinear_elut\"\([^,]+,\s*[^,]+,\s*\1\)")   # TenzoEngine.cpp:1947, :1956


def parse_with_library(text: str):
    L = load_library()
    views, scales = (C.c_ulonglong * 4096)(), (C.c_float * 4096)()
    nv, ns = C.c_int(0), C.c_int(0)
    assert L.tenzo_ext_parse_manifest(text.encode(), views, 4096, C.byref(nv), scales, 4096, C.byref(ns)) == 0
    return list(views[: nv.value]), [np.float32(x) for x in scales[: ns.value]]


def test_manifest_reader_matches_the_reference_patterns():
    rng = np.random.default_rng(7)
    lines = ["module {", "  func.func @main(%buf: memref<?xi8>) {"]
    for i in range(40):
        kind = rng.integers(0, 6)
        if kind == 0:
            lines += [f"    %c{i} = arith.constant {int(rng.integers(0, 2**40))} : index",
                      f"    %v{i} = memref.view %buf[%c{i}][] : memref<?xi8> to memref<{int(rng.integers(1, 999))}x2560xf32>"]
        elif kind == 1:
            lines += [f"    %s{i} = arith.constant {float(rng.random()):.9e} : f32",
                      f"    %y{i} = \"tenzo.bitlinear_elut\"(%a{i}, %b{i}, %s{i}) : (memref<?xf32>) -> memref<?xf32>"]
        elif kind == 2:      # a view through another constant: no match
            lines += [f"    %c{i} = arith.constant 12 : index", f"    %v{i} = memref.view %buf[%other][] : memref<?xi8> to memref<4xf32>"]
        elif kind == 3:      # the scale is not the third operand: no match
            lines += [f"    %s{i} = arith.constant 0.5 : f32", f"    %y{i} = \"tenzo.bitlinear_elut\"(%s{i}, %b{i}, %z{i})"]
        elif kind == 4:      # windows line ends and extra blanks
            lines += [f"    %c{i}  =  arith.constant   77 :  index\r", f"\t%v{i} =  memref.view  %buf[%c{i}][]  :  memref<?xi8>  to  memref<8xi8>"]
        else:
            lines += [f"    %k{i} = arith.constant 3 : i32", "    // comment"]
    text = "\n".join(lines + ["  }", "}"]) + "\n"
    views, scales = parse_with_library(text)
    assert views == [int(m.group(2)) for m in VIEW_RE.finditer(text)]
    assert scales == [np.float32(float(m.group(2))) for m in SCALE_RE.finditer(text)]
    assert len(views) > 3 and len(scales) > 3
    assert parse_with_library("") == ([], [])


@pytest.mark.skipif(not ora.ref_available("kernels"), reason="compiled reference not present")
@pytest.mark.parametrize("with_manifest", [True, False])
def test_checkpoint_writer_against_the_reference_loader(tmp_path, with_manifest):
    """The reference loads the written files and decodes the same tokens as when the same tensors are handed to it
    through its setters: pins the writer (and so the GPU loader test's input) to the reference's format."""
    cfg = dict(synth.BITNET_2B, num_layers=1, vocab_size=512, max_seq_len=32)
    model = synth.SyntheticModel(cfg, seed=9)
    w, m = tmp_path / "weights.bin", tmp_path / "model.mlir"
    emb = write_checkpoint(model, w, m, with_manifest=with_manifest, gap=64)
    if not with_manifest:
        for lw in model.layers:
            for name in model.shapes:
                lw[name + "_scale"] = np.float32(1.0)
    model.lm_w, model.lm_scales = loader_quantised_embedding(emb)
    prompt = synth.prompt_tokens(3, 4, cfg["vocab_size"])
    by_setters = RefEngine(model, max_seq_len=32)
    want = greedy_stream(by_setters, prompt, 6)
    by_setters.close()
    L = ora.load_ref("kernels")
    c = model.config_struct(max_seq_len=32)
    h = L.tenzo_create_engine(C.byref(c))
    assert h and L.tenzo_load_model(h, str(w).encode(), str(m).encode()) == 0

    class Loaded:
        def prefill(self, t): assert L.tenzo_prefill_token(h, int(t)) == 0
        def generate(self, t, temperature=0.0, rep=1.0):
            p = abi.TenzoSampling(temperature, 0.9, 40, rep)
            return L.tenzo_generate_step(h, int(t), C.byref(p), None, 0)
    got = greedy_stream(Loaded(), prompt, 6)
    L.tenzo_destroy_engine(h)
    assert np.array_equal(got, want)
