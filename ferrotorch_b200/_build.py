"""In-tree build of the native libraries.

Two shared objects are produced under ``ferrotorch_b200/_C``:

* ``libft_kernels.so``  - every ``csrc/kernels/*.cu`` compiled by nvcc for
  ``sm_100a`` only (``-gencode arch=compute_100a,code=sm_100a``), CUDA runtime
  linked statically, no link-time dependency on the driver library, so the
  library imports on a machine without a GPU.
* ``libft_runtime.so``  - the host runtime in ``csrc/runtime/*.cpp``: the
  distributed backends and collectives (``dist_runtime.cpp``), the native CPU
  tensor / autograd core with its SGD (``core.cpp``), the data-loader helpers
  (``loader.cpp``) and the host NMS sweep (``vision_ops.cpp``), plain C++20.

Objects are rebuilt only when the source (or a header) is newer than the object.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
OUT = ROOT / "_C"
OBJ = OUT / "obj"

NVCC = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
CXX = os.environ.get("CXX") or shutil.which("g++") or "g++"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--use_fast_math", "-Xcompiler", "-fPIC,-fvisibility=hidden", "--expt-relaxed-constexpr",
    "-I", str(CSRC / "kernels"), "-I", str(CSRC / "include"),
]
# bandwidth-bound generic kernels keep IEEE-accurate transcendentals (they are compared against f32 / f64 references at tight tolerances)
PRECISE_MATH = {"elementwise.cu", "reduce_index.cu", "nn_ops.cu"}
# no errno / trap bookkeeping for the math builtins (lets the Box-Muller and Philox loops vectorise); no FMA contraction, so the random streams are
# the same on every x86-64 machine whatever instruction set the vector path picks
CXX_FLAGS = ["-O3", "-fno-math-errno", "-fno-trapping-math", "-ffp-contract=off", "-std=c++20", "-fPIC", "-fvisibility=hidden", "-pthread", "-I", str(CSRC / "include"), "-I", str(CSRC / "runtime")]


def _newest_header_mtime(dirs) -> float:
    m = 0.0
    for d in dirs:
        for ext in ("*.h", "*.hpp", "*.cuh"):
            for p in Path(d).rglob(ext):
                m = max(m, p.stat().st_mtime)
    return m


def _compile(cmd, src, obj, verbose):
    if verbose:
        print(" ".join(map(str, cmd)), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"compile failed: {src}\n{r.stdout}\n{r.stderr}")
    if verbose and r.stderr.strip():
        print(r.stderr, flush=True)
    return obj


def _build_lib(name, sources, compiler, flags, link_cmd, hdr_dirs, verbose, extra_flags=()):
    OBJ.mkdir(parents=True, exist_ok=True)
    lib = OUT / name
    hdr_m = _newest_header_mtime(hdr_dirs)
    jobs, objs = [], []
    for src in sources:
        obj = OBJ / (src.stem + ("_cu.o" if src.suffix == ".cu" else "_cpp.o"))
        objs.append(obj)
        if (not obj.exists()) or obj.stat().st_mtime < max(src.stat().st_mtime, hdr_m):
            fl = [f for f in flags if not (f == "--use_fast_math" and src.name in PRECISE_MATH)]
            jobs.append(([compiler, *fl, *extra_flags, "-c", str(src), "-o", str(obj)], src, obj))
    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 4)) as ex:
            futs = [ex.submit(_compile, c, s, o, verbose) for c, s, o in jobs]
            for f in futs:
                f.result()
    if jobs or not lib.exists():
        cmd = [*link_cmd, "-o", str(lib), *map(str, objs)]
        if verbose:
            print(" ".join(cmd), flush=True)
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed: {name}\n{r.stdout}\n{r.stderr}")
    return lib


def kernel_sources():
    return sorted((CSRC / "kernels").glob("*.cu"))


def runtime_sources():
    return sorted((CSRC / "runtime").glob("*.cpp"))


def build_kernels(verbose=False, ptxas_info=False):
    extra = ["-Xptxas", "-v"] if ptxas_info else []
    link = [NVCC, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-cudart", "static", "-Xcompiler", "-fPIC", "-Xlinker", "--exclude-libs,ALL"]
    return _build_lib("libft_kernels.so", kernel_sources(), NVCC, NVCC_FLAGS, link, [CSRC / "kernels", CSRC / "include"],
                      verbose or ptxas_info, extra)


def build_runtime(verbose=False):
    srcs = runtime_sources()
    if not srcs:
        return None
    link = [CXX, "-shared", "-pthread"]
    lib = _build_lib("libft_runtime.so", srcs, CXX, CXX_FLAGS, link, [CSRC / "runtime", CSRC / "include"], verbose)
    return lib


SANITIZERS = {"thread": "thread", "address": "address,undefined"}


def build_runtime_selftest(sanitizer: str, out_path) -> Path:
    """Builds the host runtime together with its self-test driver (``csrc/runtime/selftest/runtime_selftest.cpp``: ranks as threads over the
    in-process fabric and loopback TCP, the loader and planner entry points) as one executable under ThreadSanitizer (``"thread"``) or
    AddressSanitizer + UBSan (``"address"``). Raises ``subprocess.CalledProcessError`` with the compiler output if the toolchain lacks the
    sanitizer runtime."""
    out_path = Path(out_path)
    # the configured compiler may ship without the sanitizer runtimes; the system compiler usually has them
    compilers = list(dict.fromkeys(c for c in (CXX, shutil.which("g++"), "/usr/bin/g++", shutil.which("clang++")) if c))
    last = None
    for cxx in compilers:
        cmd = [cxx, "-std=c++20", "-O1", "-g", f"-fsanitize={SANITIZERS[sanitizer]}", "-fno-omit-frame-pointer", "-pthread",
               *[str(s) for s in runtime_sources()], str(CSRC / "runtime" / "selftest" / "runtime_selftest.cpp"), "-o", str(out_path)]
        try:
            subprocess.run(cmd, check=True, capture_output=True, text=True)
            return out_path
        except (subprocess.CalledProcessError, FileNotFoundError) as e:
            last = e
    raise last


_DECL_RE = None


def _exports(path: Path, macros):
    """(comment, declaration) of every exported function of a source file: the contiguous ``//`` block directly above the definition and its
    signature up to the opening brace."""
    import re
    global _DECL_RE
    text = path.read_text()
    pat = re.compile(r"^(?:" + "|".join(re.escape(m) for m in macros) + r")\s+([^;{]*?\))\s*\{", re.M | re.S)
    out = []
    for m in pat.finditer(text):
        head = text[: m.start()].rstrip("\n").split("\n")
        comment = []
        while head and head[-1].lstrip().startswith("//"):
            comment.insert(0, head.pop().strip())
        out.append((comment, " ".join(m.group(1).split())))
    return out


def generate_headers() -> list:
    """Writes ``csrc/include/ferrotorch/kernels.h`` and ``runtime.h``: the C ABI of ``libft_kernels.so`` (every ``FT_EXPORT`` launcher of
    ``csrc/kernels/*.cu``) and of ``libft_runtime.so`` (every ``FT_API`` function of ``csrc/runtime/*.cpp``), with the comment that stands above
    each definition. The Python loader parses the same definitions, so the headers and the bindings cannot drift apart."""
    inc = CSRC / "include" / "ferrotorch"
    inc.mkdir(parents=True, exist_ok=True)
    written = []
    for name, sources, macros, includes, intro in (
            ("kernels.h", kernel_sources() + [CSRC / "kernels" / "host_common.cu"], ("FT_EXPORT", 'extern "C" __attribute__((visibility("default")))'),
             ["<cuda_runtime.h>", "<stdint.h>", "<sys/types.h>"],
             "C ABI of libft_kernels.so: launchers of the sm_100a kernels. Every function returns 0 when the work was launched, a negative FtError\n"
             "// code (-1 argument, -2 driver entry point, -3 tensor map, -4 too large, -5 guard bytes overwritten) when it refused before launching,\n"
             "// or a positive CUDA runtime error code. Pointers are device pointers unless a comment says otherwise; `stream` arguments take the\n"
             "// CUDA stream to launch on."),
            ("runtime.h", runtime_sources(), ("FT_API", "FT_EXPORT"), ["<stdint.h>"],
             "C ABI of libft_runtime.so: host-side distributed runtime (backends, collectives, bucket planner), data-loader helpers and the\n"
             "// host NMS sweep. Functions that return int return 0 on success or the error code documented in dist_runtime.cpp (1 invalid world,\n"
             "// 2 invalid rank, 3 self send, 4 size mismatch, 5 io, 7 channel closed, 8 unsupported, 9 timeout, 10 no connection, 12 argument).")):
        seen, body = set(), []
        for src in sorted(set(sources)):
            ex = [e for e in _exports(src, macros) if e[1] not in seen]
            if not ex:
                continue
            body.append(f"// ---- {src.name} " + "-" * max(4, 100 - len(src.name)))
            for comment, decl in ex:
                seen.add(decl)
                body.extend(comment)
                body.append(decl + ";")
                body.append("")
        text = ("// Generated by `python -m ferrotorch_b200._build` from the definitions in the sources; do not edit.\n// " + intro + "\n#pragma once\n"
                + "".join(f"#include {i}\n" for i in includes) + "\n#ifdef __cplusplus\nextern \"C\" {\n#endif\n\n" + "\n".join(body)
                + "\n#ifdef __cplusplus\n}  // extern \"C\"\n#endif\n")
        path = inc / name
        if not path.exists() or path.read_text() != text:
            path.write_text(text)
        written.append(path)
    return written


def build_all(verbose=False):
    OUT.mkdir(parents=True, exist_ok=True)
    k = build_kernels(verbose)
    r = build_runtime(verbose)
    generate_headers()
    return k, r


if __name__ == "__main__":
    v = "-v" in sys.argv
    if "--selftest" in sys.argv:
        kind = sys.argv[sys.argv.index("--selftest") + 1]
        exe = build_runtime_selftest(kind, OUT / f"runtime_selftest_{kind}")
        sys.exit(subprocess.run([str(exe)]).returncode)
    elif "--ptxas" in sys.argv:
        for o in OBJ.glob("*_cu.o"):
            o.unlink()
        build_kernels(ptxas_info=True)
    else:
        print(build_all(verbose=v))
