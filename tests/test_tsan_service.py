"""ThreadSanitizer run of the host control plane (master, servers, client, handlers with request coalescing,
reshard under load): tests/cpp/service_stress.cpp is built with -fsanitize=thread and must finish with every
gradient applied exactly once and without a single race report. The reference builds without sanitizers
(CMakeLists.txt:32-36); its concurrency rests on the same integration style of test."""
import os
import shutil
import subprocess

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(os.path.dirname(HERE), "parameter_server_b200", "csrc")


@pytest.mark.timeout(600)
def test_control_plane_under_thread_sanitizer(tmp_path):
    gxx = shutil.which("g++")
    if gxx is None:
        pytest.skip("no g++")
    exe = str(tmp_path / "service_stress")
    build = subprocess.run([gxx, "-std=c++17", "-O1", "-g", "-fsanitize=thread", "-I", CSRC,
                            os.path.join(HERE, "cpp", "service_stress.cpp"), os.path.join(CSRC, "operator", "operators.cpp"),
                            "-o", exe, "-lpthread", "-ldl"], capture_output=True, text=True, timeout=400)
    if build.returncode != 0 and "tsan" in build.stderr.lower():
        pytest.skip("this toolchain has no ThreadSanitizer runtime")
    assert build.returncode == 0, build.stderr[-3000:]
    env = dict(os.environ, TSAN_OPTIONS="halt_on_error=0 exitcode=66")
    run = subprocess.run([exe], capture_output=True, text=True, timeout=300, env=env)
    assert "STRESS OK" in run.stdout, run.stdout[-2000:] + run.stderr[-2000:]
    assert "WARNING: ThreadSanitizer" not in run.stderr, run.stderr[:6000]
    assert run.returncode == 0
