"""Host-side native code (block codec and container, tokenizers, HTTP server) under AddressSanitizer + UBSan and under
ThreadSanitizer: the harness csrc/san/san_driver.cpp feeds every format ragged block sizes, truncated and random payloads,
truncated / corrupted files, and a server under concurrent well-formed and malformed requests.  A report from a sanitizer
aborts the harness with a non-zero exit code."""
import subprocess

import pytest

from transformers_fusion_b200 import build


def _harness(kind, tmp_path, section="all"):
    try:
        exe = build.build_sanitized(kind)
    except RuntimeError as e:                      # a toolchain without the sanitizer run-time
        pytest.skip(f"cannot build with -fsanitize ({kind}): {str(e)[-200:]}")
    r = subprocess.run([str(exe), str(tmp_path), section], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, (r.stdout[-2000:], r.stderr[-4000:])
    assert "0 failed check(s)" in r.stdout
    assert "runtime error" not in r.stderr and "Sanitizer" not in r.stderr, r.stderr[-4000:]


def test_address_and_undefined_behaviour_sanitizers(tmp_path):
    _harness("asan", tmp_path)


def test_thread_sanitizer(tmp_path):
    _harness("tsan", tmp_path)
