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


def test_generated_c_headers_compile_and_link(tmp_path):
    """The generated public headers declare what the libraries export: a C++ program that includes them, links both libraries and calls into
    each one builds and runs (the kernels library is only asked for a constant here; no GPU is touched)."""
    import shutil
    from pathlib import Path
    cxx = shutil.which("g++")
    if cxx is None:
        pytest.skip("no C++ compiler")
    headers = _build.generate_headers()
    assert {h.name for h in headers} == {"kernels.h", "runtime.h"}
    for h in headers:
        assert h.read_text().count(";") > 20
    inc, libdir = _build.CSRC / "include", _build.OUT
    cuda_inc = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda")) / "include"
    if not (cuda_inc / "cuda_runtime.h").exists() or not (libdir / "libft_kernels.so").exists():
        pytest.skip("CUDA headers or the built libraries are not present")
    src = tmp_path / "use_headers.cpp"
    src.write_text('#include "ferrotorch/kernels.h"\n#include "ferrotorch/noalloc.h"\n#include "ferrotorch/runtime.h"\n#include <cstdio>\n'
                   'int main() { int64_t n[3] = {10, 20, 30}; int b[3];\n'
                   '  int nb = ft_ddp_plan_buckets(n, 3, 4, 100, b);\n'
                   '  std::printf("%d %d %d\\n", ft_runtime_abi_version(), nb, ft_comm_flag_bytes());\n'
                   '  return (ft_runtime_abi_version() == 1 && nb == 3 && b[2] == 0 && b[0] == 2) ? 0 : 1; }\n')
    exe = tmp_path / "use_headers"
    r = subprocess.run([cxx, "-std=c++17", "-I", str(inc), "-I", str(cuda_inc), str(src), "-L", str(libdir), "-lft_runtime", "-lft_kernels",
                        f"-Wl,-rpath,{libdir}", "-o", str(exe)], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-3000:]
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
