"""The host library (cache manager, scheduler, batch layout) under the address and undefined-behaviour
sanitizers: its CPU tests run once more in a child process that loads the library built with
`-fsanitize=address,undefined`.  A heap overrun, a use after free or undefined arithmetic in the C++ code
ends that process with a report instead of passing silently."""
import os
import subprocess
import sys

import pytest

from mini_rsglang_b200.csrc import build as native
from mini_rsglang_b200.errors import BackendError

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_host_tests_pass_under_asan_and_ubsan():
    if native.host_sanitized():
        pytest.skip("already inside the sanitized run")
    try:
        env = native.sanitizer_environment()
    except BackendError as e:
        pytest.skip(str(e))
    files = [os.path.join(ROOT, "tests", f) for f in ("test_cache_manager.py", "test_scheduler.py", "test_step_layout.py", "test_prefix_cache.py", "test_scheduler_lookahead.py")]
    proc = subprocess.run([sys.executable, "-m", "pytest", "-x", "-q", "-p", "no:cacheprovider", *files],
                          env=env, capture_output=True, text=True, timeout=900, cwd=ROOT)
    tail = (proc.stdout + proc.stderr)[-3000:]
    assert proc.returncode == 0, tail
    assert "passed" in proc.stdout and "AddressSanitizer" not in tail and "runtime error" not in tail
    built = [f for f in os.listdir(native.BUILD_DIR) if f.startswith("libmrs_host_sanitized_")]
    assert built, "the sanitized library was not built"
