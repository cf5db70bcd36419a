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


def test_c_examples_build_and_the_tcp_one_runs(tmp_path):
    """The C examples compile against the public header and the in-tree library; the tcp one runs as two ranks."""
    import socket
    import sys
    sys.path.insert(0, ROOT)
    from mccl_b200 import _lib as L
    L.load()                                                   # builds the library if it is missing
    lib_dir = os.path.join(ROOT, "mccl_b200", "lib")
    common = [f"-I{ROOT}/include", f"-L{lib_dir}", "-lmccl", f"-Wl,-rpath,{lib_dir}"]
    tcp = tmp_path / "allreduce_tcp"
    subprocess.run(["gcc", "-Wall", "-Werror", f"{ROOT}/examples/allreduce_tcp.c", "-o", str(tcp), *common], check=True)
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    if os.path.exists(os.path.join(cuda_home, "include", "cuda_runtime.h")):
        subprocess.run(["gcc", "-Wall", "-Werror", f"-I{cuda_home}/include", f"{ROOT}/examples/allreduce_cuda.c", "-o",
                        str(tmp_path / "allreduce_cuda"), *common, f"-L{cuda_home}/lib64", "-lcudart"], check=True)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    procs = [subprocess.Popen([str(tcp)], env=dict(os.environ, MCCL_BOOTSTRAP_PORT=str(port), MCCL_WORLD_SIZE="2", MCCL_RANK=str(r)),
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = [p.communicate(timeout=120)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), outs
    assert all("-> 3 (expected 3)" in o for o in outs), outs
