"""The CMake build of the host control plane (no nvcc needed): configure, build, and run the stress under ctest."""
import shutil
import subprocess

import os
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.timeout(900)
def test_host_only_cmake_build_and_ctest(tmp_path):
    cmake, ctest = shutil.which("cmake"), shutil.which("ctest")
    if cmake is None or ctest is None or shutil.which("g++") is None:
        pytest.skip("cmake / ctest / g++ not available")
    build = str(tmp_path / "build")
    cfg = subprocess.run([cmake, "-S", ROOT, "-B", build, "-DPSB_BUILD_CUDA=OFF", f"-DCMAKE_CXX_COMPILER={shutil.which('g++')}"],
                         capture_output=True, text=True, timeout=300)
    assert cfg.returncode == 0, cfg.stdout[-2000:] + cfg.stderr[-2000:]
    make = subprocess.run([cmake, "--build", build, "-j", "4"], capture_output=True, text=True, timeout=600)
    assert make.returncode == 0, make.stdout[-3000:] + make.stderr[-3000:]
    assert any(n.startswith("libpsb.") for n in os.listdir(build))            # the static and the shared library
    test = subprocess.run([ctest, "--test-dir", build, "--output-on-failure"], capture_output=True, text=True, timeout=600)
    assert test.returncode == 0 and "100% tests passed" in test.stdout, test.stdout[-3000:]
