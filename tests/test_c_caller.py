"""A C program that includes the public headers and calls the library the way the reference's own C
callers do (tests/test_gemm.cu, bench/bench_gemm.cu) is compiled with gcc, linked against
libe5m2effma.so and run.  No GPU needed: it exercises only paths that answer on the host."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CUDA = os.environ.get("CUDA_HOME", "/usr/local/cuda")


@pytest.mark.skipif(shutil.which("gcc") is None or not os.path.isdir(os.path.join(CUDA, "include")),
                    reason="needs gcc and the CUDA headers")
def test_c_caller_compiles_links_and_runs(tmp_path):
    lib_dir = os.path.join(ROOT, "e5m2effma_b200")
    assert os.path.exists(os.path.join(lib_dir, "libe5m2effma.so")), "build the library first (__graft_entry__.build())"
    exe = str(tmp_path / "caller")
    cmd = ["gcc", "-std=gnu99", "-Wall", "-Werror", os.path.join(ROOT, "tests", "c_caller", "caller.c"),
           "-I", os.path.join(ROOT, "include"), "-I", os.path.join(CUDA, "include"),
           "-L", lib_dir, "-le5m2effma", "-Wl,-rpath," + lib_dir,
           "-L", os.path.join(CUDA, "lib64"), "-lcudart", "-Wl,-rpath," + os.path.join(CUDA, "lib64"), "-o", exe]
    build = subprocess.run(cmd, capture_output=True, text=True)
    assert build.returncode == 0, build.stderr
    run = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert run.returncode == 0, run.stdout + run.stderr
    assert "ok" in run.stdout.splitlines()[-1]
    assert "INVALID_VALUE" in run.stdout or "invalid" in run.stdout.lower()
