"""A tuned-table entry really decides which kernel e5ma_gemm launches, and every plan a table can name gives a
result inside the tolerance (the table file is read once per process: each plan runs in a subprocess)."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CODE = """
import sys
sys.path.insert(0, {tests!r})
from harness import GemmCase, GemmData, check_tolerance, E5M2, E4M3, BF16
from e5m2effma_b200 import capi
d = GemmData(GemmCase(1, 0, 2560, 2816, 272, E5M2, E4M3, BF16, -1, BF16, 1.0, 0.0, vec=1, seed=11))
got, amax = d.run_gpu()
route = capi.last_route()
check_tolerance(d, got, amax)
assert capi.gemm_fault() == 0
print("ROUTE", route)
"""


@pytest.mark.parametrize("plan,route", [(-1, (5, 6)), (0, (3,)), (512, (4,)), (384, (4,)), (None, (3, 4))])
def test_table_entry_selects_the_kernel(tmp_path, plan, route):
    env = dict(os.environ)
    if plan is not None:
        path = tmp_path / "tuned.txt"
        path.write_text(f"gemm 1 2560 2816 272 {plan}\n")
        env["E5MA_TUNE_FILE"] = str(path)
    out = subprocess.run([sys.executable, "-c", CODE.format(tests=os.path.join(ROOT, "tests"))], capture_output=True, text=True,
                         cwd=ROOT, env=env, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    assert int(out.stdout.split("ROUTE")[1]) in route, out.stdout


GEMV_CODE = """
import sys
sys.path.insert(0, {tests!r})
from harness import GemmCase, GemmData, check_tolerance, E5M2, BF16
from e5m2effma_b200 import capi
routes = []
for n in (1, 2, 3, 4, 5):
    d = GemmData(GemmCase(1, 0, 300, n, 1040, E5M2, BF16, BF16, -1, BF16, 1.0, 0.0, vec=1, seed=20 + n))
    got, amax = d.run_gpu()
    routes.append(capi.last_route())
    check_tolerance(d, got, amax)
print("ROUTES", *routes)
"""


@pytest.mark.parametrize("maxn,routes", [(0, [1, 1, 1, 1, 1]), (2, [9, 9, 1, 1, 1]), (4, [9, 9, 9, 9, 1]), (8, [9, 9, 9, 9, 1])])
def test_table_entry_sets_the_batch_limit_of_the_fp32_pipe_gemv(tmp_path, maxn, routes):
    path = tmp_path / "tuned.txt"
    path.write_text(f"gemv fma_maxn {maxn}\n")
    out = subprocess.run([sys.executable, "-c", GEMV_CODE.format(tests=os.path.join(ROOT, "tests"))], capture_output=True, text=True,
                         cwd=ROOT, env=dict(os.environ, E5MA_TUNE_FILE=str(path)), timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    assert [int(x) for x in out.stdout.split("ROUTES")[1].split()] == routes, out.stdout
