"""The reference's own test driver, unmodified, against the drop-in `moe_test` module.

test/torch_test.py of the reference (fetched into the git-ignored baseline/_ref/test/ by
tests/reference_drivers/fetch.py) is run as a child process with dqmoe_b200/dropin first on PYTHONPATH. On a
B200 (compute capability 10.0) the script exercises its bf16 section over its four shapes
(test/torch_test.py:19-25, 174-181): for each it times the kernels whose profiler name contains
"GemmUniversal" (test/bench.py:77-168), prints a TFLOPS line, the error against torch_moe_grouped
(IS_PRINT=1, test/torch_test.py:28-42) and the end-to-end time of 100 calls."""
import os
import re
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_TEST = os.path.join(ROOT, "baseline", "_ref", "test")
pytestmark = pytest.mark.gpu


def _have_scripts():
    return all(os.path.exists(os.path.join(REF_TEST, f)) for f in ("torch_test.py", "bench.py", "util.py"))


@pytest.mark.skipif(not _have_scripts(), reason="baseline/_ref/test is not populated (run tests/reference_drivers/fetch.py)")
@pytest.mark.parametrize("module_dir", ["dropin", "dropin_ext"])
def test_reference_torch_test_runs_unmodified_on_the_drop_in(module_dir):
    """module_dir: dropin = the ctypes moe_test.py, dropin_ext = the compiled pybind11 moe_test extension."""
    mod_path = os.path.join(ROOT, "dqmoe_b200", module_dir)
    if module_dir == "dropin_ext" and not any(f.startswith("moe_test") and f.endswith(".so") for f in os.listdir(mod_path)):
        pytest.skip("the pybind11 extension is not built (python -m dqmoe_b200.build --ext)")
    env = dict(os.environ, IS_PRINT="1",
               PYTHONPATH=os.pathsep.join([mod_path, REF_TEST, os.environ.get("PYTHONPATH", "")]))
    res = subprocess.run([sys.executable, "torch_test.py"], cwd=REF_TEST, env=env, capture_output=True, text=True,
                         timeout=1500)
    out = res.stdout
    log_dir = os.path.join(ROOT, "gpurun_out")
    if os.path.isdir(log_dir):
        with open(os.path.join(log_dir, f"reference_torch_test_{module_dir}.log"), "w") as f:
            f.write(out + "\n--- stderr ---\n" + res.stderr[-4000:])
    assert res.returncode == 0, res.stderr[-2000:]
    assert "Eror in perf measurement" not in out
    # one TFLOPS line per shape of enumerate_m_grouped_contiguous
    tflops = [float(m.group(1)) for m in re.finditer(r"\|\s*([0-9.]+) TFLOPS", out)]
    assert len(tflops) == 4, out[-2000:]
    assert tflops[2] > 100 and tflops[3] > 100  # the two large shapes run on the tensor cores
    # the script's own error metric against the bf16 torch result: mean relative error of a bf16 layer
    rel = [float(m.group(1)) for m in re.finditer(r"RelErr \(%\)\s*:\s*([0-9.]+)%", out)]
    mse = [float(m.group(1)) for m in re.finditer(r"MSE\s*:\s*([0-9.e+-]+)", out)]
    assert len(rel) == 4 and len(mse) == 4
    assert all(m < 1e-4 for m in mse), mse
    assert out.count("Moe end to end bench.") == 4
