"""The drop-in boundary, proven by compilation (no GPU needed): with the reference checkout present,

  * tests/consumer/hpp_consumer.cpp, written against the reference's own include/tenzo.hpp (tenzo::Engine, the loop of
    examples/basic_inference.cpp:143-171), compiles with the reference's include directory and links against
    libtenzo_runtime.so;
  * the reference's engine source (src/runtime/TenzoEngine.cpp) compiles with THIS repository's include/CUDARuntime.h in
    place of its stub header and links against libtenzo_runtime.so, leaving tenzo::CUDARuntime's members to be resolved
    from it - so its device = "cuda" branch (forward_layer_cuda, :1369-1418) runs this library's kernels.

tests/test_gpu_boundary.py runs both artefacts on a GPU."""
import os
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
REF = Path(os.environ.get("TENZO_REFERENCE", ROOT.parent / "reference"))


@pytest.fixture(scope="module")
def built():
    if not (REF / "src" / "runtime" / "TenzoEngine.cpp").exists():
        pytest.skip("needs the reference checkout (TENZO_REFERENCE)")
    from tenzo_b200.build import build
    build()
    r = subprocess.run(["make", "-C", str(ROOT / "oracle"), "boundary", f"REF={REF}"], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    return ROOT / "oracle" / "_ref"


def symbols(path, flag):
    out = subprocess.run(["nm", "-D", flag, str(path)], capture_output=True, text=True, check=True).stdout
    return {line.split()[-1] for line in out.splitlines() if line.strip()}


def test_reference_cpp_wrapper_consumer_links_against_the_library(built):
    exe = built / "hpp_consumer"
    assert exe.exists()
    need = symbols(exe, "--undefined-only")
    have = symbols(ROOT / "tenzo_b200" / "lib" / "libtenzo_runtime.so", "--defined-only")
    used = {s for s in need if s.startswith("tenzo_")}
    assert {"tenzo_create_engine", "tenzo_destroy_engine", "tenzo_load_model", "tenzo_prefill_token", "tenzo_generate_step",
            "tenzo_default_config", "tenzo_default_sampling_params", "tenzo_get_seq_len"} <= used
    assert used <= have


def test_reference_engine_links_its_cuda_branch_against_the_backend_class(built):
    lib = built / "libtenzo_ref_cuda.so"
    assert lib.exists()
    need = symbols(lib, "--undefined-only")
    have = symbols(ROOT / "tenzo_b200" / "lib" / "libtenzo_runtime.so", "--defined-only")
    members = {s for s in need if "CUDARuntime" in s}
    assert any("getInstance" in s for s in members) and any("executeBitLinearTL1" in s for s in members) and any("executeRMSNorm" in s for s in members)
    assert members <= have, members - have
