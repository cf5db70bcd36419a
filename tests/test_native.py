"""Native-code checks that need a compiler run: the threaded tcp driver against a ThreadSanitizer build of
the library (race detection for the host code).  Slow (compiles the library twice), so it only runs with
MCCL_TEST_TSAN=1."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(os.environ.get("MCCL_TEST_TSAN") != "1", reason="set MCCL_TEST_TSAN=1 to build and run the TSAN flavour")
def test_threaded_tcp_ranks_under_thread_sanitizer(tmp_path):
    build = tmp_path / "tsan"
    subprocess.run(["cmake", "-S", ROOT, "-B", str(build), "-DMCCL_SANITIZE_THREAD=ON", "-DCMAKE_BUILD_TYPE=RelWithDebInfo"],
                   check=True, capture_output=True)
    subprocess.run(["cmake", "--build", str(build), "-j", "8"], check=True, capture_output=True)
    exe = build / "tsan_tcp"
    subprocess.run(["g++", "-std=c++17", "-O1", "-g", "-fsanitize=thread", f"-I{ROOT}/include", f"{ROOT}/tests/native/tsan_tcp.cc",
                    "-o", str(exe), f"-L{build}", "-lmccl", f"-Wl,-rpath,{build}", "-pthread"], check=True)
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=600,
                       env=dict(os.environ, TSAN_OPTIONS="halt_on_error=0 report_signal_unsafe=0"))
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    assert "WARNING: ThreadSanitizer" not in r.stderr
