"""Sanitizer runs of the host control plane (master, servers, client, handlers with request coalescing,
reshard under load, node loss + restore, scans against pushes): tests/cpp/service_stress.cpp is built once
with -fsanitize=thread and once with -fsanitize=address,undefined; it must finish with every gradient applied
exactly once and without a single report. The reference builds without sanitizers (CMakeLists.txt:32-36);
its concurrency rests on the same integration style of test."""
import os
import shutil
import subprocess

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(os.path.dirname(HERE), "parameter_server_b200", "csrc")


@pytest.mark.timeout(900)
@pytest.mark.parametrize("sanitizer,marker", [("thread", "WARNING: ThreadSanitizer"),
                                              ("address,undefined", "ERROR: AddressSanitizer")])
def test_control_plane_under_sanitizer(tmp_path, sanitizer, marker):
    gxx = shutil.which("g++")
    if gxx is None:
        pytest.skip("no g++")
    exe = str(tmp_path / "service_stress")
    build = subprocess.run([gxx, "-std=c++17", "-O1", "-g", f"-fsanitize={sanitizer}", "-fno-omit-frame-pointer", "-I", CSRC,
                            os.path.join(HERE, "cpp", "service_stress.cpp"), os.path.join(CSRC, "operator", "operators.cpp"),
                            "-o", exe, "-lpthread", "-ldl"], capture_output=True, text=True, timeout=400)
    if build.returncode != 0 and ("tsan" in build.stderr.lower() or "asan" in build.stderr.lower()):
        pytest.skip("this toolchain lacks the sanitizer runtime")
    assert build.returncode == 0, build.stderr[-3000:]
    env = dict(os.environ, TSAN_OPTIONS="halt_on_error=0 exitcode=66", ASAN_OPTIONS="detect_leaks=1",
               UBSAN_OPTIONS="print_stacktrace=1")
    run = subprocess.run([exe], capture_output=True, text=True, timeout=400, env=env)
    assert "STRESS OK" in run.stdout, run.stdout[-2000:] + run.stderr[-2000:]
    assert marker not in run.stderr and "runtime error:" not in run.stderr, run.stderr[:6000]
    assert run.returncode == 0


@pytest.mark.timeout(600)
def test_window_walking_scans_of_a_storage_without_snapshots(tmp_path):
    """KVStorage's default scan_shard / update_shard (what the GPU back-end runs) on the CPU, under
    AddressSanitizer: every key once on a quiet table, a restart or an error when the index is rebuilt under the
    scan, changed rows written back exactly once (tests/cpp/kv_window_scan.cpp)."""
    gxx = shutil.which("g++")
    if gxx is None:
        pytest.skip("no g++")
    exe = str(tmp_path / "kv_window_scan")
    flags = ["-fsanitize=address,undefined", "-fno-omit-frame-pointer"]
    cmd = [gxx, "-std=c++17", "-O1", "-g", *flags, "-I", CSRC, os.path.join(HERE, "cpp", "kv_window_scan.cpp"), "-o", exe, "-lpthread"]
    build = subprocess.run(cmd, capture_output=True, text=True, timeout=400)
    if build.returncode != 0 and "asan" in build.stderr.lower():
        build = subprocess.run([c for c in cmd if c not in flags], capture_output=True, text=True, timeout=400)
    assert build.returncode == 0, build.stderr[-3000:]
    run = subprocess.run([exe], capture_output=True, text=True, timeout=200)
    assert run.returncode == 0 and "WINDOW SCAN OK" in run.stdout, run.stdout[-2000:] + run.stderr[-2000:]
    assert "ERROR: AddressSanitizer" not in run.stderr and "runtime error:" not in run.stderr, run.stderr[:4000]
