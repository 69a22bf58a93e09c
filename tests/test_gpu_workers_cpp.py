"""The C++ worker mirror (include/tkv_workers.hpp): PrefillWorker / DecodeWorker /
DisaggregatedPipeline over GPU pools.  tests/cpp/test_disaggregated.cu restates the
reference's own pipeline tests (engine/src/disaggregated.rs:292-400); here it is compiled
against the in-tree library and run."""
import os
import shutil
import subprocess

import pytest

from tempura_b200 import _build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_worker_header_is_plain_cxx17(tmp_path):
    """No CUDA needed to include the header: a host-only engine build can use it."""
    src = tmp_path / "include_only.cpp"
    src.write_text('#include "tkv_workers.hpp"\nint main() { tkv_host::SamplingParams p; return p.top_k == 50 ? 0 : 1; }\n')
    gxx = shutil.which("g++")
    assert gxx, "g++ not found"
    proc = subprocess.run([gxx, "-std=c++17", "-Wall", "-Werror", "-fsyntax-only", "-I", os.path.join(ROOT, "include"), str(src)],
                          capture_output=True, text=True)
    assert proc.returncode == 0, proc.stderr


@pytest.mark.gpu
def test_reference_pipeline_tests_over_gpu_workers(tmp_path):
    _build.build()
    exe = tmp_path / "test_disaggregated"
    cmd = [_build._nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-O2", "-I", os.path.join(ROOT, "include"),
           "-o", str(exe), os.path.join(ROOT, "tests", "cpp", "test_disaggregated.cu"),
           "-L", _build.LIB_DIR, "-ltkv", "-Xlinker", "-rpath", "-Xlinker", _build.LIB_DIR]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stdout + proc.stderr
    run = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300)
    assert run.returncode == 0, run.stdout[-2000:] + run.stderr[-4000:]
    assert "ALL PASSED" in run.stdout
