"""The host runtime (backends, collectives, loader, planner, NMS sweep) under ThreadSanitizer and AddressSanitizer + UBSan: the self-test
driver runs ranks as threads over the in-process fabric and over TCP on loopback; any sanitizer report fails the run."""
import os
import subprocess

import pytest

from ferrotorch_b200 import _build


@pytest.mark.parametrize("sanitizer", ["thread", "address"])
def test_runtime_selftest_is_clean_under_sanitizer(tmp_path, sanitizer):
    try:
        exe = _build.build_runtime_selftest(sanitizer, tmp_path / f"selftest_{sanitizer}")
    except FileNotFoundError:
        pytest.skip("no C++ compiler")
    except subprocess.CalledProcessError as e:
        if "cannot find" in (e.stderr or "") or "unrecognized" in (e.stderr or ""):
            pytest.skip(f"toolchain has no {sanitizer} sanitizer runtime")
        raise AssertionError(e.stderr)
    env = dict(os.environ, TSAN_OPTIONS="halt_on_error=1 exitcode=66", ASAN_OPTIONS="detect_leaks=1 exitcode=67", UBSAN_OPTIONS="halt_on_error=1 exitcode=68")
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0, f"rc {r.returncode}\n{r.stdout[-2000:]}\n{r.stderr[-4000:]}"
    assert "selftest ok" in r.stdout
    assert "runtime error" not in r.stderr and "WARNING: ThreadSanitizer" not in r.stderr
