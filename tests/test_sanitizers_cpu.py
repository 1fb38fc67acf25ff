"""The native host runtime (scheduler, cache manager, control plane) under ThreadSanitizer and AddressSanitizer:
the stand-alone stress driver is built with -fsanitize=... and must exit 0 without a sanitizer report."""
import subprocess

import pytest

from ksanallm_b200.build import build_host_stress


@pytest.mark.parametrize("sanitizer", ["thread", "address"])
def test_host_runtime_is_clean_under_sanitizer(sanitizer):
    binary = build_host_stress(sanitizer)
    r = subprocess.run([str(binary)], capture_output=True, text=True, timeout=600)
    report = r.stdout[-2000:] + r.stderr[-4000:]
    assert r.returncode == 0, report
    assert "host stress ok" in r.stdout
    assert "ThreadSanitizer" not in r.stderr and "AddressSanitizer" not in r.stderr, report
    assert "swap preemptions" in r.stdout
