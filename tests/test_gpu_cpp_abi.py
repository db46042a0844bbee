"""The kernel library is a C interface (csrc/api.h): a C++ program that includes the header and links the shared
library, with no Python anywhere in it, is compiled here and run."""
import os
import shutil
import subprocess

import pytest

from citlali_b200 import ops

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def test_a_cpp_program_calls_the_kernels_through_the_c_interface(tmp_path):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("no nvcc to build the example with")
    ops.lib()                                                   # makes sure the library is built
    csrc = os.path.join(os.path.dirname(HERE), "citlali-llm-engine_b200", "csrc")
    lib_dir = os.path.join(csrc, "_build")
    exe = str(tmp_path / "abi_example")
    build = subprocess.run([nvcc, "-std=c++17", "-O1", "-I", csrc, os.path.join(HERE, "cpp", "abi_example.cpp"), "-o", exe,
                            "-L", lib_dir, "-lcitlali_b200", "-Xlinker", f"-rpath={lib_dir}"], capture_output=True, text=True, timeout=300)
    assert build.returncode == 0, build.stdout + build.stderr
    run = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert run.returncode == 0 and run.stdout.startswith("ok"), run.stdout + run.stderr
    assert "multiple of 8" in run.stdout                        # the refusal's text came through citlali_last_error
