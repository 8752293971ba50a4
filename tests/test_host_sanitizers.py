"""The host code (the cache's books, the prefix tree, the scheduler: csrc/host_core.cu) built with
AddressSanitizer and UndefinedBehaviorSanitizer, under the tests that drive it hardest.

compute-sanitizer covers device code; this is its counterpart for the C++ that runs on the host: the
randomized tests of the cache manager, the prefix tree and the scheduler run in a child process against a
build of the same source with ``-fsanitize=address,undefined``.  A heap overflow, a use after free or
undefined arithmetic in the books ends that process with the sanitizer's report.
"""
import os
import shutil
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SOURCE = os.path.join(ROOT, "sglang_rs_b200", "csrc", "host_core.cu")


def runtime(name: str) -> str:
    path = subprocess.run(["gcc", f"-print-file-name={name}"], capture_output=True, text=True).stdout.strip()
    return path if os.path.isabs(path) and os.path.exists(path) else ""


@pytest.mark.skipif(shutil.which("g++") is None or not runtime("libasan.so"), reason="g++ with libasan is needed")
def test_host_books_under_address_and_undefined_behaviour_sanitizers(tmp_path):
    library = str(tmp_path / "host_core_sanitized.so")
    subprocess.check_call(["g++", "-x", "c++", "-std=c++17", "-O1", "-g", "-fsanitize=address,undefined",
                           "-fno-sanitize-recover=undefined", "-shared", "-fPIC", "-o", library, SOURCE])
    # (the child sees no GPU: the CUDA driver does not start under AddressSanitizer, and the host books need none)
    env = dict(os.environ, SRB_LIBRARY_HOST_CORE=library, LD_PRELOAD=runtime("libasan.so"), CUDA_VISIBLE_DEVICES="",
               ASAN_OPTIONS="detect_leaks=0:abort_on_error=1:protect_shadow_gap=0",
               UBSAN_OPTIONS="print_stacktrace=1:halt_on_error=1")
    tests = [os.path.join(ROOT, "tests", name) for name in ("test_cache_manager.py", "test_prefix_tree.py", "test_scheduler.py")]
    process = subprocess.run([sys.executable, "-m", "pytest", "-q", "-x", "-m", "not gpu", "-p", "no:cacheprovider", *tests],
                             env=env, capture_output=True, text=True, timeout=900, cwd=ROOT)
    tail = (process.stdout + process.stderr)[-3000:]
    assert process.returncode == 0, tail
    assert "passed" in process.stdout and "ERROR: AddressSanitizer" not in tail and "runtime error" not in tail
    # the child really ran the sanitized build
    check = subprocess.run([sys.executable, "-c", "import ctypes, os; from sglang_rs_b200.csrc.build import load_library; "
                            "load_library('host_core'); print(open('/proc/self/maps').read().count('host_core_sanitized'))"],
                           env=env, capture_output=True, text=True, timeout=300, cwd=ROOT)
    assert check.returncode == 0 and int(check.stdout.strip().splitlines()[-1]) > 0, check.stderr[-2000:]
