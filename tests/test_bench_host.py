"""Host-side checks of the benchmark driver: every workload the documentation names is dispatched, an unknown one is
refused, and the reference arm's bookkeeping helpers work without a GPU."""
import argparse
import inspect
import re
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def _dispatched():
    from tenzo_b200 import bench_extra
    src = inspect.getsource(bench_extra.run)
    return set(re.findall(r'"(\w+)": run_', src))


def test_documented_workloads_are_dispatched():
    from tenzo_b200 import bench_extra
    documented = set(re.findall(r"^  (\w+) {2,}\S", bench_extra.__doc__, flags=re.M))
    assert documented, "the module docstring lists the workloads"
    assert documented <= _dispatched(), documented - _dispatched()
    readme = (ROOT / "README.md").read_text()
    listed = re.search(r"--workload\s+([\w|\s]+)\]", readme).group(1).replace("\n", "").replace(" ", "").split("|")
    assert set(listed) - {"decode_b1"} <= _dispatched()


def test_unknown_workload_is_refused():
    from tenzo_b200 import bench_extra
    with pytest.raises(SystemExit):
        bench_extra.run(argparse.Namespace(workload="no_such_workload"))


def test_host_thread_helpers():
    import bench
    n = bench.physical_cores()
    assert n >= 1
    assert bench.use_host_threads() >= 1
