"""Host-only native code (shared-memory ring, safetensors I/O) built as C++ with AddressSanitizer +
UndefinedBehaviorSanitizer and, separately, ThreadSanitizer, and run through a producer / consumer and a round-trip
driver. The GPU kernels cannot be run under compute-sanitizer on the shared pool; their checks are the numerics tests."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "openrlhf_b200", "csrc", "host_io.cu")
DRV = os.path.join(ROOT, "tests", "native", "san_driver.cpp")


@pytest.mark.parametrize("flags", [("-fsanitize=address,undefined", "-fno-sanitize-recover=all"), ("-fsanitize=thread",)])
def test_host_io_under_sanitizers(tmp_path, flags):
    gxx = shutil.which("g++")
    if gxx is None:
        pytest.skip("no g++")
    exe = str(tmp_path / "san_driver")
    cmd = [gxx, "-std=c++17", "-O1", "-g", *flags, "-x", "c++", SRC, "-x", "c++", DRV, "-o", exe, "-lpthread", "-lrt"]
    b = subprocess.run(cmd, capture_output=True, text=True)
    if b.returncode != 0 and ("cannot find" in b.stderr or "sanitizer" in b.stderr.lower() and "unsupported" in b.stderr.lower()):
        pytest.skip("sanitizer runtime not installed: " + b.stderr[-200:])
    assert b.returncode == 0, b.stderr[-3000:]
    env = dict(os.environ, ASAN_OPTIONS="detect_leaks=1:abort_on_error=0", TSAN_OPTIONS="halt_on_error=1")
    r = subprocess.run([exe], capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0 and "SANITIZER_DRIVER_OK" in r.stdout, r.stdout[-1000:] + r.stderr[-4000:]
