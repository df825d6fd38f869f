"""The tuned selection table: the tuner's text form round-trips, the library parses it (E5MA_TUNE_FILE, read once
per process, hence the subprocess) and lets it override the compiled-in entries, and the compiled-in header holds
what the tuner would write.  The GPU half (a table entry really changes the launched kernel, and the result stays
inside the tolerance) is in tests/test_gpu_tuned_table.py."""
import os
import re
import subprocess
import sys

from e5m2effma_b200 import capi, tune

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_text_table_round_trips():
    rows = [(1, 8192, 4096, 14336, 512), (2, 4096, 4096, 4096, 0), (1, 2048, 2048, 2048, -1)]
    gemv = {"kernel": 1, "stages": 3, "kmap": 1, "fma_maxn": 2}
    assert tune.parse_table(tune.table_text(rows, gemv)) == (rows, gemv)
    assert tune.parse_table("# comment\n\ngemm 1 2 3\nnonsense\n") == ([], {})


def test_compiled_table_is_what_the_tuner_writes():
    text = open(os.path.join(ROOT, "e5m2effma_b200", "csrc", "tuned_sm100.h")).read()
    rows = [tuple(int(x) for x in m) for m in re.findall(r"\{(-?\d+), (-?\d+), (-?\d+), (-?\d+), (-?\d+)\}", text)]
    gemv = {k.lower(): int(v) for k, v in re.findall(r"#define E5B_TUNED_GEMV_(KERNEL|STAGES|KMAP|FMA_MAXN) (-?\d+)", text)}
    assert rows and set(gemv) == {"kernel", "stages", "kmap", "fma_maxn"}
    assert tune.header_text(rows, gemv, "NVIDIA B200 (148 SMs)").split("#pragma once")[1] == text.split("#pragma once")[1]
    for eb, m, n, k, plan in rows:               # the library answers with the compiled entries
        assert capi.tuned_plan(eb, m, n, k) == plan
    assert capi.tuned_plan(1, 12345, 512, 16) == -2


def test_library_reads_the_file_named_in_the_environment(tmp_path):
    path = tmp_path / "tuned.txt"
    path.write_text(tune.table_text([(1, 4096, 4096, 4096, 384), (2, 1024, 2048, 512, -1)], {"kernel": 0, "stages": 3, "kmap": 1, "fma_maxn": 0}))
    code = ("from e5m2effma_b200 import capi; "
            "print(capi.tuned_plan(1, 4096, 4096, 4096), capi.tuned_plan(2, 1024, 2048, 512), capi.tuned_plan(1, 8192, 4096, 14336), "
            "capi.tuned_plan(1, 7, 7, 16))")
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, cwd=ROOT,
                         env=dict(os.environ, E5MA_TUNE_FILE=str(path)))
    assert out.returncode == 0, out.stderr
    # file entries win over compiled ones; compiled ones remain for problems the file does not list
    assert out.stdout.split() == ["384", "-1", "512", "-2"]
