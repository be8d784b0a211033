"""Code generation for fused elementwise regions.

A ``fused`` node (a DAG of elementwise ops over one output shape, inputs possibly broadcast or strided) becomes one kernel:

* **CUDA C++ for sm_100a**, compiled in-process with NVRTC to a cubin and launched through the native loader
  (``ft_jit_load / ft_jit_get_kernel / ft_jit_launch``). When every non-scalar operand is contiguous with the output's shape
  the kernel moves 16 bytes per thread per operand (8 bf16 / 4 f32); otherwise it resolves broadcast strides per element.
  Arithmetic runs in f32 (f64 for double operands); bf16/f16 are converted at the loads and stores.
* **C++ for the host**, compiled with the system compiler into a shared object and called through ctypes (the counterpart of the
  reference's in-process CPU JIT).

Kernels are cached by the fingerprint of the fused body plus the layout class, in memory and (images) on disk.

Reference parity: ferrotorch-jit/src/{codegen_ir.rs:25-833 (loop IR), codegen_gpu.rs:75,561 (CUDA C / PTX text), codegen_cpu.rs:36,
codegen_jit.rs:91-313 (in-process CPU JIT), fusion.rs:281,534 (fused chains, NVRTC)}.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import re
import subprocess
import tempfile
import threading
from pathlib import Path
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..errors import FerrotorchError, InvalidArgument
from .ir import IrGraph, IrNode, dtype_of

_CTYPE = {"f32": "float", "f64": "double", "bf16": "__nv_bfloat16", "f16": "__half", "i64": "long long", "i32": "int", "bool": "unsigned char",
          "u8": "unsigned char", "i8": "signed char", "i16": "short"}
_HOST_CTYPE = dict(_CTYPE, bf16="unsigned short", f16=None)
_FLOATS = {"f32", "f64", "bf16", "f16"}
MAX_DIMS = 6


def _acc_type(dt: str) -> str:
    if dt == "f64":
        return "double"
    if dt in _FLOATS:
        return "float"
    if dt == "bool":
        return "bool"
    return "long long"


def _lit(x: float, acc: str) -> str:
    if acc == "bool":
        return "true" if x else "false"
    if acc == "long long":
        return f"{int(x)}LL"
    if x != x:
        return "NAN"
    if x in (float("inf"), float("-inf")):
        return ("-" if x < 0 else "") + "INFINITY"
    return f"{float(x)!r}" + ("f" if acc == "float" else "")


def _fn(name: str, acc: str) -> str:
    return name + ("f" if acc == "float" else "")


def _emit_expr(n: IrNode, a: List[str], acc: str, in_acc: List[str]) -> str:
    op = n.op
    f = lambda nm: _fn(nm, acc)                                   # noqa: E731
    one, zero, half = _lit(1.0, acc), _lit(0.0, acc), _lit(0.5, acc)
    U = {"neg": "-{0}", "abs": f("fabs") + "({0})", "exp": f("exp") + "({0})", "exp2": f("exp2") + "({0})", "log": f("log") + "({0})",
         "log2": f("log2") + "({0})", "sqrt": f("sqrt") + "({0})", "rsqrt": f"({one} / " + f("sqrt") + "({0}))", "reciprocal": f"({one} / {{0}})",
         "sin": f("sin") + "({0})", "cos": f("cos") + "({0})", "tanh": f("tanh") + "({0})", "sigmoid": f"({one} / ({one} + " + f("exp") + "(-{0})))",
         "relu": f"({{0}} > {zero} ? {{0}} : {zero})", "silu": f"({{0}} / ({one} + " + f("exp") + "(-{0})))", "erf": f("erf") + "({0})",
         "floor": f("floor") + "({0})", "ceil": f("ceil") + "({0})", "round": f("nearbyint") + "({0})",
         "sign": f"(({{0}} > {zero}) - ({{0}} < {zero}))", "square": "({0} * {0})",
         "softplus": f"({{0}} > {_lit(20.0, acc)} ? {{0}} : " + f("log1p") + "(" + f("exp") + "({0})))",
         "gelu": f"({half} * {{0}} * ({one} + " + f("erf") + f"({{0}} * {_lit(0.7071067811865476, acc)})))",
         "gelu_tanh": f"({half} * {{0}} * ({one} + " + f("tanh") + f"({_lit(0.7978845608028654, acc)} * ({{0}} + {_lit(0.044715, acc)} * {{0}} * {{0}} * {{0}}))))",
         "mish": "({0} * " + f("tanh") + "(" + f("log1p") + "(" + f("exp") + "({0}))))", "logical_not": "(!{0})", "isnan": "({0} != {0})"}
    B = {"add": "({0} + {1})", "sub": "({0} - {1})", "mul": "({0} * {1})", "div": "({0} / {1})", "pow": f("pow") + "({0}, {1})",
         "maximum": "(({0} > {1} || {0} != {0}) ? {0} : {1})", "minimum": "(({0} < {1} || {0} != {0}) ? {0} : {1})", "eq": "({0} == {1})", "ne": "({0} != {1})",
         "lt": "({0} < {1})", "le": "({0} <= {1})", "gt": "({0} > {1})", "ge": "({0} >= {1})", "logical_and": "({0} && {1})", "logical_or": "({0} || {1})",
         "fmod": f("fmod") + "({0}, {1})", "atan2": f("atan2") + "({0}, {1})"}
    if op in U:
        if acc == "long long" and op not in ("neg", "abs", "sign", "square", "relu"):
            raise InvalidArgument(f"codegen: {op} on an integer value")
        if acc == "long long" and op == "abs":
            return f"({a[0]} < 0 ? -{a[0]} : {a[0]})"
        return U[op].format(*a)
    if op in B:
        return B[op].format(*a)
    if op == "cast":
        return f"(({acc}){a[0]})"
    if op == "where":
        return f"({a[0]} ? {a[1]} : {a[2]})"
    if op == "clamp":
        return f"({a[0]} != {a[0]} ? {a[0]} : ({a[0]} < {a[1]} ? {a[1]} : ({a[0]} > {a[2]} ? {a[2]} : {a[0]})))"
    if op == "addcmul":
        return f"({a[0]} + {_lit(float(n.attrs.get('value', 1)), acc)} * {a[1]} * {a[2]})"
    if op == "addcdiv":
        return f"({a[0]} + {_lit(float(n.attrs.get('value', 1)), acc)} * {a[1]} / {a[2]})"
    if op == "lerp":
        return f"({a[0]} + {a[2]} * ({a[1]} - {a[0]}))"
    raise InvalidArgument(f"codegen: unsupported op {op}")


def _body_lines(body: IrGraph, in_names: Dict[int, str]) -> Tuple[List[str], Dict[int, str]]:
    """Straight-line code computing every node of the fused body; returns the lines and the variable of every value."""
    var: Dict[int, str] = dict(in_names)
    lines: List[str] = []
    for vid, c in body.constants.items():
        if c.numel() != 1:
            raise InvalidArgument("codegen: non-scalar constant inside a fused body")
        var[vid] = _lit(float(c), _acc_type(body.values[vid].dtype))
    for n in body.topo_order():
        out = body.values[n.outputs[0]]
        acc = _acc_type(out.dtype)
        ins = []
        for i in n.inputs:
            ia = _acc_type(body.values[i].dtype)
            ins.append(var[i] if ia == acc or n.op in ("where", "eq", "ne", "lt", "le", "gt", "ge", "cast", "isnan", "logical_not", "logical_and", "logical_or")
                       else f"(({acc}){var[i]})")
        # comparisons evaluate in the promoted type of their operands
        expr = _emit_expr(n, ins, acc if acc != "bool" else _acc_type(body.values[n.inputs[0]].dtype) if n.op not in ("logical_not", "logical_and", "logical_or", "isnan") else "bool", [])
        if out.dtype in ("bf16", "f16"):                          # round through the storage type, as eager execution does
            cv = "__bfloat162float(__float2bfloat16({}))" if out.dtype == "bf16" else "__half2float(__float2half({}))"
            expr = cv.format(expr) if "__HOST__" not in in_names.get(-1, "") else f"ft_round_bf16({expr})"
        name = f"v{n.outputs[0]}"
        lines.append(f"{acc} {name} = {expr};")
        var[n.outputs[0]] = name
    return lines, var


def _load(dt: str, ptr: str, idx: str, host: bool = False) -> str:
    if dt == "bf16":
        return f"ft_bf16_to_float({ptr}[{idx}])" if host else f"__bfloat162float({ptr}[{idx}])"
    if dt == "f16":
        return f"__half2float({ptr}[{idx}])"
    if dt == "bool":
        return f"({ptr}[{idx}] != 0)"
    return f"({_acc_type(dt)}){ptr}[{idx}]"


def _store(dt: str, ptr: str, idx: str, val: str, host: bool = False) -> str:
    if dt == "bf16":
        return f"{ptr}[{idx}] = ft_float_to_bf16({val});" if host else f"{ptr}[{idx}] = __float2bfloat16({val});"
    if dt == "f16":
        return f"{ptr}[{idx}] = __float2half({val});"
    return f"{ptr}[{idx}] = ({(_HOST_CTYPE if host else _CTYPE)[dt]}){val};"


def generate_cuda(body: IrGraph, name: str, vectorized: bool) -> str:
    """CUDA C++ source of the kernel ``name``. Signature: (in0, ..., out0, ..., n[, strides table]).

    ``vectorized``: all non-scalar inputs and all outputs are dense with the output shape; each thread handles VEC consecutive
    elements with 16-byte accesses on the widest type. Otherwise the kernel takes ``ndim``, ``shape[MAX_DIMS]`` and one stride row
    per input (element strides, 0 on broadcast dims) and each thread handles one element.
    """
    ins = [body.values[i] for i in body.inputs]
    outs = [body.values[o] for o in body.outputs]
    params = [f"const {_CTYPE[v.dtype]}* __restrict__ in{k}" for k, v in enumerate(ins)] + [f"{_CTYPE[v.dtype]}* __restrict__ out{k}" for k, v in enumerate(outs)]
    params.append("long long n")
    src = ["#include <cuda_bf16.h>", "#include <cuda_fp16.h>", f"struct FtStrides {{ int ndim; long long shape[{MAX_DIMS}]; long long stride[{max(len(ins), 1)}][{MAX_DIMS}]; }};"]
    scalar = [all(s == 1 for s in v.shape) for v in ins]
    if vectorized:
        vec = vector_width(body)                                  # the launch sizes its grid with the same figure
        src.append(f'extern "C" __global__ void __launch_bounds__(256) {name}({", ".join(params)}) {{')
        src.append(f"  const long long base = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * {vec};")
        src.append("  if (base >= n) return;")
        src.append(f"  if (base + {vec} <= n) {{")
        # vector path: stage each operand through an aligned register array
        for k, v in enumerate(ins):
            if scalar[k]:
                continue
            ct = _CTYPE[v.dtype]
            src.append(f"    alignas(16) {ct} r{k}[{vec}];")
            nbytes = vec * {"f64": 8, "i64": 8, "f32": 4, "i32": 4, "bf16": 2, "f16": 2, "i16": 2}.get(v.dtype, 1)
            chunks = max(nbytes // 16, 1)
            cty = "uint4" if nbytes >= 16 else "uint2" if nbytes == 8 else "unsigned int" if nbytes == 4 else "unsigned short"
            src.append(f"    for (int c = 0; c < {chunks}; c++) reinterpret_cast<{cty}*>(r{k})[c] = reinterpret_cast<const {cty}*>(in{k} + base)[c];")
        for k, v in enumerate(outs):
            src.append(f"    alignas(16) {_CTYPE[v.dtype]} w{k}[{vec}];")
        src.append("#pragma unroll")
        src.append(f"    for (int e = 0; e < {vec}; e++) {{")
        names = {}
        for k, v in enumerate(ins):
            acc = _acc_type(v.dtype)
            src.append(f"      const {acc} x{k} = {_load(v.dtype, 'in' + str(k), '0') if scalar[k] else _load(v.dtype, 'r' + str(k), 'e')};")
            names[body.inputs[k]] = f"x{k}"
        lines, var = _body_lines(body, names)
        src += ["      " + l for l in lines]
        for k, v in enumerate(outs):
            src.append("      " + _store(v.dtype, f"w{k}", "e", var[body.outputs[k]]))
        src.append("    }")
        for k, v in enumerate(outs):
            nbytes = vec * {"f64": 8, "i64": 8, "f32": 4, "i32": 4, "bf16": 2, "f16": 2, "i16": 2}.get(v.dtype, 1)
            chunks = max(nbytes // 16, 1)
            cty = "uint4" if nbytes >= 16 else "uint2" if nbytes == 8 else "unsigned int" if nbytes == 4 else "unsigned short"
            src.append(f"    for (int c = 0; c < {chunks}; c++) reinterpret_cast<{cty}*>(out{k} + base)[c] = reinterpret_cast<const {cty}*>(w{k})[c];")
        src.append("  } else {")
        src.append("    for (long long i = base; i < n; i++) {")
        names = {}
        for k, v in enumerate(ins):
            src.append(f"      const {_acc_type(v.dtype)} x{k} = {_load(v.dtype, 'in' + str(k), '0' if scalar[k] else 'i')};")
            names[body.inputs[k]] = f"x{k}"
        lines, var = _body_lines(body, names)
        src += ["      " + l for l in lines]
        for k, v in enumerate(outs):
            src.append("      " + _store(v.dtype, f"out{k}", "i", var[body.outputs[k]]))
        src += ["    }", "  }", "}"]
    else:
        params.append("const FtStrides st")
        src.append(f'extern "C" __global__ void __launch_bounds__(256) {name}({", ".join(params)}) {{')
        src.append("  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;")
        src.append("  if (i >= n) return;")
        src.append(f"  long long rem = i, off[{max(len(ins), 1)}] = {{}};")
        src.append("  for (int d = st.ndim - 1; d >= 0; d--) {")
        src.append("    const long long c = rem % st.shape[d];")
        src.append("    rem /= st.shape[d];")
        for k in range(len(ins)):
            src.append(f"    off[{k}] += c * st.stride[{k}][d];")
        src.append("  }")
        names = {}
        for k, v in enumerate(ins):
            src.append(f"  const {_acc_type(v.dtype)} x{k} = {_load(v.dtype, 'in' + str(k), f'off[{k}]')};")
            names[body.inputs[k]] = f"x{k}"
        lines, var = _body_lines(body, names)
        src += ["  " + l for l in lines]
        for k, v in enumerate(outs):
            src.append("  " + _store(v.dtype, f"out{k}", "i", var[body.outputs[k]]))
        src.append("}")
    return "\n".join(src) + "\n"


def vector_width(body: IrGraph) -> int:
    ins = [body.values[i] for i in body.inputs if not all(s == 1 for s in body.values[i].shape)]
    outs = [body.values[o] for o in body.outputs]
    width = min(2 if v.dtype in ("bf16", "f16", "i16") else 1 if v.dtype in ("bool", "u8", "i8") else 8 if v.dtype in ("f64", "i64") else 4 for v in ins + outs)
    return min(16 // width, 8) * _VEC_SCALE


# Elements per thread of the dense kernels, as a multiple of what fills one 16-byte access of the narrowest operand (FT_JIT_VEC_SCALE=1|2).
# Two accesses in flight per operand measured 0.152 ms against 0.175 ms on a 12-operation f32 chain over 64 M elements.
_VEC_SCALE = 1 if os.environ.get("FT_JIT_VEC_SCALE", "2") == "1" else 2


# ----------------------------------------------------------------------------------------------------------------------
# NVRTC
# ----------------------------------------------------------------------------------------------------------------------
_cache_dir = Path(os.environ.get("FT_JIT_CACHE", Path(tempfile.gettempdir()) / "ferrotorch_b200_jit"))
_mem_cache: Dict[str, bytes] = {}
_lock = threading.Lock()


def _cuda_include_dirs() -> List[str]:
    out = []
    for p in (os.environ.get("CUDA_HOME"), "/usr/local/cuda"):
        if p and (Path(p) / "include" / "cuda_bf16.h").exists():
            out.append(str(Path(p) / "include"))
    try:
        import nvidia.cuda_runtime as rt                          # wheel layout
        out.append(str(Path(rt.__file__).parent / "include"))
    except Exception:
        pass
    return out


def compile_cuda(source: str, arch: str = "sm_100a") -> bytes:
    """NVRTC: CUDA C++ text -> cubin for ``arch``. Works without a GPU. Cached by the hash of (source, arch)."""
    key = hashlib.sha256((arch + "\0" + source).encode()).hexdigest()
    with _lock:
        if key in _mem_cache:
            return _mem_cache[key]
    f = _cache_dir / f"{key}.cubin"
    if f.exists():
        img = f.read_bytes()
        _mem_cache[key] = img
        return img
    from cuda.bindings import nvrtc
    err, prog = nvrtc.nvrtcCreateProgram(source.encode(), b"fused.cu", 0, [], [])
    if err != nvrtc.nvrtcResult.NVRTC_SUCCESS:
        raise FerrotorchError(f"nvrtcCreateProgram failed: {err}")
    opts = [f"--gpu-architecture={arch}".encode(), b"-std=c++17", b"-lineinfo"] + [f"-I{d}".encode() for d in _cuda_include_dirs()]
    (err,) = nvrtc.nvrtcCompileProgram(prog, len(opts), opts)
    if err != nvrtc.nvrtcResult.NVRTC_SUCCESS:
        _, n = nvrtc.nvrtcGetProgramLogSize(prog)
        log = b" " * n
        nvrtc.nvrtcGetProgramLog(prog, log)
        raise FerrotorchError("NVRTC compilation failed:\n" + log.decode(errors="replace") + "\n--- source ---\n" + source)
    _, n = nvrtc.nvrtcGetCUBINSize(prog)
    img = b" " * n
    nvrtc.nvrtcGetCUBIN(prog, img)
    nvrtc.nvrtcDestroyProgram(prog)
    try:
        _cache_dir.mkdir(parents=True, exist_ok=True)
        f.write_bytes(img)
    except OSError:
        pass
    with _lock:
        _mem_cache[key] = img
    return img


class CudaFusedKernel:
    """A fused body compiled for the device. ``__call__(inputs) -> outputs`` picks the vectorised or the strided kernel per call."""

    def __init__(self, body: IrGraph):
        self.body = body
        self.fp = body.fingerprint()[:16]
        self.shape = tuple(body.values[body.outputs[0]].shape)
        self._kern: Dict[bool, object] = {}
        self._libs: List[object] = []
        self.sources = {v: generate_cuda(body, f"ft_fused_{self.fp}_{'v' if v else 's'}", v) for v in (True, False)}
        self.images = {v: compile_cuda(s) for v, s in self.sources.items()}
        self.vec = vector_width(body)

    def _kernel(self, vectorized: bool):
        k = self._kern.get(vectorized)
        if k is None:
            from .. import _lib
            lib, fn = ctypes.c_void_p(), ctypes.c_void_p()
            img = self.images[vectorized]
            self._img_keep = getattr(self, "_img_keep", []) + [ctypes.create_string_buffer(img, len(img))]
            _lib.call("ft_jit_load", ctypes.addressof(self._img_keep[-1]), ctypes.addressof(lib))
            name = f"ft_fused_{self.fp}_{'v' if vectorized else 's'}".encode()
            nb = ctypes.create_string_buffer(name)
            _lib.call("ft_jit_get_kernel", lib.value, ctypes.addressof(nb), ctypes.addressof(fn))
            self._libs.append(lib)
            k = self._kern[vectorized] = fn.value
        return k

    def __call__(self, inputs: Sequence[torch.Tensor]) -> List[torch.Tensor]:
        from .. import _lib
        body = self.body
        dev = next(t.device for t in inputs if t.is_cuda)
        outs = [torch.empty(self.shape, device=dev, dtype=dtype_of(body.values[o].dtype)) for o in body.outputs]
        n = outs[0].numel()
        if n == 0:
            return outs
        ins = [t if t.device == dev else t.to(dev) for t in inputs]
        dense = all(t.numel() == 1 or (tuple(t.shape) == self.shape and t.is_contiguous() and t.data_ptr() % 16 == 0) for t in ins)
        args: List[ctypes._SimpleCData] = [ctypes.c_void_p(t.data_ptr()) for t in ins] + [ctypes.c_void_p(t.data_ptr()) for t in outs] + [ctypes.c_longlong(n)]
        if dense:
            grid = (n + self.vec * 256 - 1) // (self.vec * 256)
        else:
            nd = max(len(self.shape), 1)
            if nd > MAX_DIMS:
                raise InvalidArgument(f"fused kernel supports at most {MAX_DIMS} dims")

            class St(ctypes.Structure):
                _fields_ = [("ndim", ctypes.c_int), ("shape", ctypes.c_longlong * MAX_DIMS), ("stride", (ctypes.c_longlong * MAX_DIMS) * max(len(ins), 1))]
            st = St()
            st.ndim = nd
            shp = self.shape or (1,)
            for d in range(nd):
                st.shape[d] = shp[d]
            for k, t in enumerate(ins):
                e = t.expand(shp) if t.numel() > 1 or t.dim() else t.reshape(()).expand(shp)
                for d in range(nd):
                    st.stride[k][d] = e.stride(d)
            args.append(st)
            grid = (n + 255) // 256
        arr = (ctypes.c_void_p * len(args))(*[ctypes.addressof(a) for a in args])
        _lib.call("ft_jit_launch", self._kernel(dense), grid, 256, 0, ctypes.addressof(arr), _lib.S())
        return outs


# ----------------------------------------------------------------------------------------------------------------------
# host C++
# ----------------------------------------------------------------------------------------------------------------------
_HOST_FLAGS_TAG = "// g++ -O3 -march=native -fno-math-errno -fno-trapping-math -fopenmp-simd\n"      # part of the cache key of compiled host kernels

_HOST_PRELUDE = r"""
#include <cmath>
#include <cstdint>
#include <cstring>
#include <algorithm>
#include <thread>
#include <vector>
static inline float ft_bf16_to_float(unsigned short h) { uint32_t u = (uint32_t)h << 16; float f; std::memcpy(&f, &u, 4); return f; }
static inline unsigned short ft_float_to_bf16(float f) { uint32_t u; std::memcpy(&u, &f, 4); if ((u & 0x7fffffffu) > 0x7f800000u) return (unsigned short)((u >> 16) | 0x40);
  u += 0x7fffu + ((u >> 16) & 1u); return (unsigned short)(u >> 16); }
static inline float ft_round_bf16(float f) { return ft_bf16_to_float(ft_float_to_bf16(f)); }
// Branch-free expf / tanhf (Cephes polynomials, about 1-2 ulp) used by the dense loop: plain arithmetic and selects, so the compiler vectorises
// the whole fused body. Infinities, NaN and exp(-inf) == 0 behave as in libm; results between 1e-45 and 1.2e-38 come out as the smallest normal.
static inline float ft_expf(float x) {
  const float xc = x > 88.72283935546875f ? 88.72283935546875f : (x < -87.33654022216797f ? -87.33654022216797f : x);
  const float n = nearbyintf(xc * 1.44269504088896341f);
  float r = fmaf(n, -0.693359375f, xc);
  r = fmaf(n, 2.12194440e-4f, r);
  float p = 1.9875691500e-4f;
  p = fmaf(p, r, 1.3981999507e-3f);
  p = fmaf(p, r, 8.3334519073e-3f);
  p = fmaf(p, r, 4.1665795894e-2f);
  p = fmaf(p, r, 1.6666665459e-1f);
  p = fmaf(p, r, 5.0000001201e-1f);
  const float e = fmaf(p, r * r, r) + 1.0f;
  const int32_t ni = (int32_t)n;
  // 2^n in two factors so that n = 128 (the top of the range) does not overflow the exponent field before the multiply
  const int32_t h = ni >> 1;
  uint32_t b0 = (uint32_t)(h + 127) << 23, b1 = (uint32_t)(ni - h + 127) << 23;
  float s0, s1;
  std::memcpy(&s0, &b0, 4);
  std::memcpy(&s1, &b1, 4);
  const float v = e * s0 * s1;
  return x > 88.72283935546875f ? INFINITY : (x < -103.972084045410f ? 0.0f : v);
}
// logf: exponent / mantissa split on the bit pattern, mantissa folded to [sqrt(1/2), sqrt(2)), degree-9 polynomial (Cephes). Zero -> -inf,
// negative -> NaN, inf and NaN pass through, denormals are rescaled first.
static inline float ft_logf(float x) {
  const bool den = x < 1.17549435e-38f;
  const float xs = den ? x * 8388608.0f : x;
  uint32_t b;
  std::memcpy(&b, &xs, 4);
  int32_t e = (int32_t)((b >> 23) & 0xffu) - 126 - (den ? 23 : 0);
  uint32_t mb = (b & 0x807fffffu) | 0x3f000000u;
  float m;
  std::memcpy(&m, &mb, 4);
  const bool lo = m < 0.707106781186547524f;
  e -= lo ? 1 : 0;
  m = lo ? m + m - 1.0f : m - 1.0f;
  const float z = m * m;
  float p = 7.0376836292e-2f;
  p = fmaf(p, m, -1.1514610310e-1f);
  p = fmaf(p, m, 1.1676998740e-1f);
  p = fmaf(p, m, -1.2420140846e-1f);
  p = fmaf(p, m, 1.4249322787e-1f);
  p = fmaf(p, m, -1.6668057665e-1f);
  p = fmaf(p, m, 2.0000714765e-1f);
  p = fmaf(p, m, -2.4999993993e-1f);
  p = fmaf(p, m, 3.3333331174e-1f);
  const float fe = (float)e;
  float y = p * m * z;
  y = fmaf(fe, -2.12194440e-4f, y);
  y = fmaf(-0.5f, z, y);
  const float r = fmaf(fe, 0.693359375f, m + y);
  return x > 3.4028234e38f ? x : (x == 0.0f ? -INFINITY : (x < 0.0f ? NAN : (x != x ? x : r)));
}
// erff: odd Taylor polynomial below 1 (relative accuracy near zero), 1 - poly(t) * exp(-x^2) with t = 1 / (1 + p |x|) above (absolute error
// about 1.5e-7, i.e. 1-2 ulp of a value between 0.84 and 1).
static inline float ft_expf(float x);
static inline float ft_erff(float x) {
  const float ax = fabsf(x), z = x * x;
  float s = -1.0892221020000000e-9f;                // -1 / 918086400: Taylor terms (-1)^k / (k! (2k+1)) of erf(x) sqrt(pi) / (2x), k = 11 .. 0
  s = fmaf(s, z, 1.3122532963802806e-8f);           // 1 / 76204800
  s = fmaf(s, z, -1.4503852223150468e-7f);          // -1 / 6894720
  s = fmaf(s, z, 1.4589169000933707e-6f);           // 1 / 685440
  s = fmaf(s, z, -1.3227513227513228e-5f);          // -1 / 75600
  s = fmaf(s, z, 1.0683760683760684e-4f);           // 1 / 9360
  s = fmaf(s, z, -7.5757575757575758e-4f);          // -1 / 1320
  s = fmaf(s, z, 4.6296296296296294e-3f);           // 1 / 216
  s = fmaf(s, z, -2.3809523809523808e-2f);          // -1 / 42
  s = fmaf(s, z, 0.1f);
  s = fmaf(s, z, -0.33333333333333331f);
  s = fmaf(s, z, 1.0f);
  const float small = 1.1283791670955126f * x * s;
  const float t = 1.0f / fmaf(0.3275911f, ax, 1.0f);
  float q = 1.061405429f;
  q = fmaf(q, t, -1.453152027f);
  q = fmaf(q, t, 1.421413741f);
  q = fmaf(q, t, -0.284496736f);
  q = fmaf(q, t, 0.254829592f);
  const float big = 1.0f - q * t * ft_expf(-z);
  return ax < 1.0f ? small : (x != x ? x : copysignf(big, x));
}
static inline float ft_tanhf(float x) {
  const float ax = fabsf(x);
  const float z = x * x;
  float p = -5.70498872745e-3f;
  p = fmaf(p, z, 2.06390887954e-2f);
  p = fmaf(p, z, -5.37397155531e-2f);
  p = fmaf(p, z, 1.33314422036e-1f);
  p = fmaf(p, z, -3.33332819422e-1f);
  const float small = fmaf(p * z, x, x);
  const float big = 1.0f - 2.0f / (ft_expf(2.0f * ax) + 1.0f);
  const float r = ax < 0.625f ? small : copysignf(big, x);
  return r;
}
struct FtStrides { int ndim; long long shape[%d]; long long stride[%d][%d]; };
"""


def generate_host(body: IrGraph, name: str) -> str:
    ins = [body.values[i] for i in body.inputs]
    outs = [body.values[o] for o in body.outputs]
    for v in ins + outs:
        if _HOST_CTYPE[v.dtype] is None:
            raise InvalidArgument("host codegen: f16 is not supported")
    params = [f"const {_HOST_CTYPE[v.dtype]}* __restrict__ in{k}" for k, v in enumerate(ins)] + [f"{_HOST_CTYPE[v.dtype]}* __restrict__ out{k}" for k, v in enumerate(outs)]
    params += ["long long n", "const FtStrides* st"]
    src = [_HOST_PRELUDE % (MAX_DIMS, max(len(ins), 1), MAX_DIMS), f'extern "C" void {name}({", ".join(params)}) {{']
    src.append("  auto body = [&](long long begin, long long end) {")
    # st == nullptr: every input is contiguous with the output's shape - a plain indexed loop the compiler can vectorise (libmvec for the
    # transcendental calls); otherwise the general strided / broadcasting walk below
    src.append("  if (st == nullptr) {")
    src.append("    for (long long i = begin; i < end; i++) {")
    dnames = {-1: "__HOST__"}
    for k, v in enumerate(ins):
        src.append(f"      const {_acc_type(v.dtype)} x{k} = {_load(v.dtype, 'in' + str(k), 'i', host=True)};")
        dnames[body.inputs[k]] = f"x{k}"
    dlines, dvar = _body_lines(body, dnames)
    dlines = [re.sub(r"(?<![A-Za-z0-9_])(expf|tanhf|logf|erff)\(", r"ft_\1(", l) for l in dlines]        # the vectorisable versions of the prelude
    src += ["      " + l for l in dlines]
    for k, v in enumerate(outs):
        src.append("      " + _store(v.dtype, f"out{k}", "i", dvar[body.outputs[k]], host=True))
    src += ["    }", "    return;", "  }"]
    # general case: walk the last dimension row by row. The offsets of the leading dimensions are computed once per row; inputs whose last
    # dimension is broadcast (statically known from the traced shapes) are loaded once per row, the others are expected to have unit stride
    # there (checked at run time), which leaves a vectorisable inner loop; anything else takes the strided inner loop.
    nin = max(len(ins), 1)
    out_last = outs[0].shape[-1] if len(outs[0].shape) else 1
    full = [len(v.shape) > 0 and v.shape[-1] == out_last and out_last > 1 for v in ins]
    src.append("  const int nd = st->ndim;")
    src.append("  const long long cols = st->shape[nd - 1];")
    cond = " && ".join([f"st->stride[{k}][nd - 1] == {1 if full[k] else 0}" for k in range(len(ins))]) or "true"
    src.append(f"  const bool rowfast = {cond};")
    src.append("  long long i = begin;")
    src.append("  while (i < end) {")
    src.append("    const long long row = i / cols, c0 = i % cols, c1 = std::min(cols, c0 + (end - i));")
    src.append(f"    long long rem = row, base[{nin}] = {{}};")
    src.append("    for (int d = nd - 2; d >= 0; d--) { const long long c = rem % st->shape[d]; rem /= st->shape[d];")
    for k in range(len(ins)):
        src.append(f"      base[{k}] += c * st->stride[{k}][d];")
    src.append("    }")
    src.append("    const long long o = row * cols;")
    src.append("    if (rowfast) {")
    rnames = {-1: "__HOST__"}
    for k, v in enumerate(ins):
        if full[k]:
            src.append(f"      const {_HOST_CTYPE[v.dtype]}* __restrict__ p{k} = in{k} + base[{k}];")
        else:
            src.append(f"      const {_acc_type(v.dtype)} x{k} = {_load(v.dtype, 'in' + str(k), f'base[{k}]', host=True)};")
        rnames[body.inputs[k]] = f"x{k}"
    src.append("      for (long long col = c0; col < c1; col++) {")
    for k, v in enumerate(ins):
        if full[k]:
            src.append(f"        const {_acc_type(v.dtype)} x{k} = {_load(v.dtype, 'p' + str(k), 'col', host=True)};")
    rlines, rvar = _body_lines(body, rnames)
    rlines = [re.sub(r"(?<![A-Za-z0-9_])(expf|tanhf|logf|erff)\(", r"ft_\1(", l) for l in rlines]
    src += ["        " + l for l in rlines]
    for k, v in enumerate(outs):
        src.append("        " + _store(v.dtype, f"out{k}", "o + col", rvar[body.outputs[k]], host=True))
    src += ["      }", "    } else {"]
    src.append("      for (long long col = c0; col < c1; col++) {")
    names = {-1: "__HOST__"}
    for k, v in enumerate(ins):
        src.append(f"        const {_acc_type(v.dtype)} x{k} = {_load(v.dtype, 'in' + str(k), f'base[{k}] + col * st->stride[{k}][nd - 1]', host=True)};")
        names[body.inputs[k]] = f"x{k}"
    lines, var = _body_lines(body, names)
    src += ["        " + l for l in lines]
    for k, v in enumerate(outs):
        src.append("        " + _store(v.dtype, f"out{k}", "o + col", var[body.outputs[k]], host=True))
    src += ["      }", "    }", "    i += c1 - c0;"]
    src += ["  }", "  };"]
    src.append("  const long long grain = 1 << 16;")
    src.append("  long long nt = std::min<long long>((n + grain - 1) / grain, (long long)std::max(1u, std::thread::hardware_concurrency()));")
    src.append("  if (nt <= 1) { body(0, n); return; }")
    src.append("  std::vector<std::thread> th; const long long per = (n + nt - 1) / nt;")
    src.append("  for (long long t = 0; t < nt; t++) th.emplace_back(body, t * per, std::min(n, (t + 1) * per));")
    src.append("  for (auto& x : th) x.join();")
    src.append("}")
    return "\n".join(src) + "\n"


class HostFusedKernel:
    def __init__(self, body: IrGraph):
        self.body = body
        self.fp = body.fingerprint()[:16]
        self.shape = tuple(body.values[body.outputs[0]].shape)
        self.name = f"ft_fused_{self.fp}_h"
        self.source = generate_host(body, self.name)
        key = hashlib.sha256((_HOST_FLAGS_TAG + self.source).encode()).hexdigest()
        _cache_dir.mkdir(parents=True, exist_ok=True)
        so = _cache_dir / f"{key}.so"
        if not so.exists():
            cpp = _cache_dir / f"{key}.cpp"
            cpp.write_text(self.source)
            tmp = _cache_dir / f"{key}.{os.getpid()}.tmp.so"
            r = subprocess.run([os.environ.get("CXX", "g++"), "-O3", "-march=native", "-fno-math-errno", "-fno-trapping-math", "-fopenmp-simd", "-pthread", "-shared", "-fPIC",
                                "-std=c++17", str(cpp), "-o", str(tmp)],
                               capture_output=True, text=True)
            if r.returncode != 0:
                raise FerrotorchError("host codegen compilation failed:\n" + r.stderr + "\n--- source ---\n" + self.source)
            os.replace(tmp, so)
        self.lib = ctypes.CDLL(str(so))
        self.fn = getattr(self.lib, self.name)
        self.fn.restype = None

    def __call__(self, inputs: Sequence[torch.Tensor]) -> List[torch.Tensor]:
        body = self.body
        outs = [torch.empty(self.shape, dtype=dtype_of(body.values[o].dtype)) for o in body.outputs]
        n = outs[0].numel()
        if n == 0:
            return outs
        if all(tuple(t.shape) == self.shape and t.is_contiguous() for t in inputs):
            self.fn(*([ctypes.c_void_p(t.data_ptr()) for t in inputs] + [ctypes.c_void_p(t.data_ptr()) for t in outs] + [ctypes.c_longlong(n), None]))
            return outs
        nd = max(len(self.shape), 1)
        nin = max(len(inputs), 1)

        class St(ctypes.Structure):
            _fields_ = [("ndim", ctypes.c_int), ("shape", ctypes.c_longlong * MAX_DIMS), ("stride", (ctypes.c_longlong * MAX_DIMS) * nin)]
        st = St()
        st.ndim = nd
        shp = self.shape or (1,)
        for d in range(nd):
            st.shape[d] = shp[d]
        for k, t in enumerate(inputs):
            e = t.expand(shp)
            for d in range(nd):
                st.stride[k][d] = e.stride(d)
        args = [ctypes.c_void_p(t.data_ptr()) for t in inputs] + [ctypes.c_void_p(t.data_ptr()) for t in outs] + [ctypes.c_longlong(n), ctypes.byref(st)]
        self.fn(*args)
        return outs


# ----------------------------------------------------------------------------------------------------------------------
# fused elementwise region + reduction over the last dimension
# ----------------------------------------------------------------------------------------------------------------------
_RED = {"sum": ("0", "{a} + {b}"), "mean": ("0", "{a} + {b}"), "amax": ("-INFINITY", "(({b} > {a} || {b} != {b}) ? {b} : {a})"),
        "amin": ("INFINITY", "(({b} < {a} || {b} != {b}) ? {b} : {a})")}


def _offset_lines(n_in: int, ptr_prefix: str, indent: str) -> List[str]:
    lines = [f"{indent}long long rem = i, off[{max(n_in, 1)}] = {{}};", f"{indent}for (int d = {ptr_prefix}ndim - 1; d >= 0; d--) {{",
             f"{indent}  const long long c = rem % {ptr_prefix}shape[d];", f"{indent}  rem /= {ptr_prefix}shape[d];"]
    lines += [f"{indent}  off[{k}] += c * {ptr_prefix}stride[{k}][d];" for k in range(n_in)]
    lines.append(f"{indent}}}")
    return lines


def generate_cuda_reduce(body: IrGraph, name: str, red_op: str, red_index: int) -> str:
    """One CTA per row of the region's ``[rows, cols]`` view: every thread evaluates the fused body for its columns, the reduced output goes through
    a warp-shuffle + shared-memory block reduction, the other outputs are stored elementwise. Signature: (in..., red_out, other outs..., rows, cols, strides)."""
    ins = [body.values[i] for i in body.inputs]
    outs = [body.values[o] for o in body.outputs]
    red_v = outs[red_index]
    acc = _acc_type(red_v.dtype)
    ident, comb = _RED[red_op]
    others = [(k, v) for k, v in enumerate(outs) if k != red_index]
    params = [f"const {_CTYPE[v.dtype]}* __restrict__ in{k}" for k, v in enumerate(ins)] + [f"{_CTYPE[red_v.dtype]}* __restrict__ red_out"]
    params += [f"{_CTYPE[v.dtype]}* __restrict__ out{k}" for k, v in others] + ["long long rows", "int cols", "const FtStrides st"]
    src = ["#include <cuda_bf16.h>", "#include <cuda_fp16.h>", f"struct FtStrides {{ int ndim; long long shape[{MAX_DIMS}]; long long stride[{max(len(ins), 1)}][{MAX_DIMS}]; }};",
           f'extern "C" __global__ void __launch_bounds__(256) {name}({", ".join(params)}) {{', f"  __shared__ {acc} red[8];", "  const long long row = blockIdx.x;",
           f"  {acc} acc = {ident};", "  for (int col = threadIdx.x; col < cols; col += 256) {", "    const long long i = row * cols + col;"]
    src += _offset_lines(len(ins), "st.", "    ")
    names = {}
    for k, v in enumerate(ins):
        src.append(f"    const {_acc_type(v.dtype)} x{k} = {_load(v.dtype, 'in' + str(k), f'off[{k}]')};")
        names[body.inputs[k]] = f"x{k}"
    lines, var = _body_lines(body, names)
    src += ["    " + l for l in lines]
    rv = var[body.outputs[red_index]]
    src.append("    acc = " + comb.format(a="acc", b=f"(({acc}){rv})") + ";")
    for k, v in others:
        src.append("    " + _store(v.dtype, f"out{k}", "i", var[body.outputs[k]]))
    src.append("  }")
    src += ["  for (int o = 16; o > 0; o >>= 1) { const " + acc + " other = __shfl_xor_sync(0xffffffffu, acc, o); acc = " + comb.format(a="acc", b="other") + "; }",
            "  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;", "  __syncthreads();", "  if (threadIdx.x < 32) {",
            f"    acc = threadIdx.x < 8 ? red[threadIdx.x] : ({acc}){ident};",
            "    for (int o = 4; o > 0; o >>= 1) { const " + acc + " other = __shfl_xor_sync(0xffffffffu, acc, o); acc = " + comb.format(a="acc", b="other") + "; }",
            "    if (threadIdx.x == 0) " + _store(red_v.dtype, "red_out", "row", "acc / cols" if red_op == "mean" else "acc"), "  }", "}"]
    return "\n".join(src) + "\n"


def generate_host_reduce(body: IrGraph, name: str, red_op: str, red_index: int) -> str:
    """Host form of the fused region + last-dimension reduction: rows are split over threads; per row the offsets of the leading dimensions are
    computed once, inputs whose last dimension is broadcast are loaded once, and the others are walked with unit stride when they have it (the
    vectorisable loop) or with their run-time stride otherwise."""
    ins = [body.values[i] for i in body.inputs]
    outs = [body.values[o] for o in body.outputs]
    red_v = outs[red_index]
    acc = _acc_type(red_v.dtype)
    ident, comb = _RED[red_op]
    others = [(k, v) for k, v in enumerate(outs) if k != red_index]
    nin = max(len(ins), 1)
    out_last = outs[0].shape[-1] if len(outs[0].shape) else 1
    full = [len(v.shape) > 0 and v.shape[-1] == out_last and out_last > 1 for v in ins]
    params = [f"const {_HOST_CTYPE[v.dtype]}* __restrict__ in{k}" for k, v in enumerate(ins)] + [f"{_HOST_CTYPE[red_v.dtype]}* __restrict__ red_out"]
    params += [f"{_HOST_CTYPE[v.dtype]}* __restrict__ out{k}" for k, v in others] + ["long long rows", "int cols", "const FtStrides* stp"]
    src = [_HOST_PRELUDE % (MAX_DIMS, nin, MAX_DIMS), f'extern "C" void {name}({", ".join(params)}) {{', "  const FtStrides& st = *stp;", "  const int nd = st.ndim;"]
    cond = " && ".join([f"st.stride[{k}][nd - 1] == {1 if full[k] else 0}" for k in range(len(ins))]) or "true"
    src.append(f"  const bool rowfast = {cond};")
    src.append("  auto work = [&](long long r0, long long r1) {")
    src.append("  for (long long row = r0; row < r1; row++) {")
    src.append(f"    long long rem = row, base[{nin}] = {{}};")
    src.append("    for (int d = nd - 2; d >= 0; d--) { const long long c = rem % st.shape[d]; rem /= st.shape[d];")
    for k in range(len(ins)):
        src.append(f"      base[{k}] += c * st.stride[{k}][d];")
    src.append("    }")
    src.append(f"    {acc} acc = {ident};")
    src.append("    const long long o = row * cols;")

    def inner(fast: bool, indent: str) -> List[str]:
        out = []
        names = {-1: "__HOST__"}
        if fast:
            for k, v in enumerate(ins):
                if full[k]:
                    out.append(f"{indent}const {_HOST_CTYPE[v.dtype]}* __restrict__ p{k} = in{k} + base[{k}];")
                else:
                    out.append(f"{indent}const {_acc_type(v.dtype)} x{k} = {_load(v.dtype, 'in' + str(k), f'base[{k}]', host=True)};")
        if fast and red_op in ("sum", "mean"):
            out.append(f"{indent}#pragma omp simd reduction(+:acc)")          # lets the compiler keep one partial sum per vector lane
        out.append(f"{indent}for (int col = 0; col < cols; col++) {{")
        for k, v in enumerate(ins):
            if fast and full[k]:
                out.append(f"{indent}  const {_acc_type(v.dtype)} x{k} = {_load(v.dtype, 'p' + str(k), 'col', host=True)};")
            elif not fast:
                out.append(f"{indent}  const {_acc_type(v.dtype)} x{k} = {_load(v.dtype, 'in' + str(k), f'base[{k}] + col * st.stride[{k}][nd - 1]', host=True)};")
            names[body.inputs[k]] = f"x{k}"
        lines, var = _body_lines(body, names)
        if fast:
            lines = [re.sub(r"(?<![A-Za-z0-9_])(expf|tanhf|logf|erff)\(", r"ft_\1(", l) for l in lines]
        out += [indent + "  " + l for l in lines]
        out.append(f"{indent}  acc = " + comb.format(a="acc", b=f"(({acc}){var[body.outputs[red_index]]})") + ";")
        for k, v in others:
            out.append(f"{indent}  " + _store(v.dtype, f"out{k}", "o + col", var[body.outputs[k]], host=True))
        out.append(f"{indent}}}")
        return out
    src.append("    if (rowfast) {")
    src += inner(True, "      ")
    src.append("    } else {")
    src += inner(False, "      ")
    src.append("    }")
    src.append("    " + _store(red_v.dtype, "red_out", "row", "acc / cols" if red_op == "mean" else "acc", host=True))
    src += ["  }", "  };"]
    src.append("  const long long grain = std::max<long long>(1, (1 << 16) / std::max(cols, 1));")
    src.append("  long long nt = std::min<long long>((rows + grain - 1) / grain, (long long)std::max(1u, std::thread::hardware_concurrency()));")
    src.append("  if (nt <= 1) { work(0, rows); return; }")
    src.append("  std::vector<std::thread> th; const long long per = (rows + nt - 1) / nt;")
    src.append("  for (long long t = 0; t < nt; t++) th.emplace_back(work, t * per, std::min(rows, (t + 1) * per));")
    src.append("  for (auto& x : th) x.join();")
    src.append("}")
    return "\n".join(src) + "\n"


class _FusedReduceBase:
    def __init__(self, body: IrGraph, red_op: str, red_index: int, keepdim: bool):
        self.body, self.red_op, self.red_index, self.keepdim = body, red_op, red_index, keepdim
        self.fp = hashlib.sha256((body.fingerprint() + red_op + str(red_index)).encode()).hexdigest()[:16]
        self.shape = tuple(body.values[body.outputs[0]].shape)
        if len(self.shape) < 1 or len(self.shape) > MAX_DIMS:
            raise InvalidArgument("fused reduction needs 1 to 6 dimensions")
        self.cols = self.shape[-1]
        self.rows = 1
        for s in self.shape[:-1]:
            self.rows *= s

    def _alloc(self, device):
        body = self.body
        rshape = self.shape[:-1] + ((1,) if self.keepdim else ())
        red = torch.empty(rshape, device=device, dtype=dtype_of(body.values[body.outputs[self.red_index]].dtype))
        others = [torch.empty(self.shape, device=device, dtype=dtype_of(body.values[o].dtype)) for k, o in enumerate(body.outputs) if k != self.red_index]
        return red, others

    def _strides(self, inputs):
        nin = max(len(inputs), 1)

        class St(ctypes.Structure):
            _fields_ = [("ndim", ctypes.c_int), ("shape", ctypes.c_longlong * MAX_DIMS), ("stride", (ctypes.c_longlong * MAX_DIMS) * nin)]
        st = St()
        st.ndim = len(self.shape)
        for d, s in enumerate(self.shape):
            st.shape[d] = s
        for k, t in enumerate(inputs):
            e = t.expand(self.shape)
            for d in range(len(self.shape)):
                st.stride[k][d] = e.stride(d)
        return st


class CudaFusedReduceKernel(_FusedReduceBase):
    def __init__(self, body, red_op, red_index, keepdim):
        super().__init__(body, red_op, red_index, keepdim)
        self.name = f"ft_fusedred_{self.fp}"
        self.source = generate_cuda_reduce(body, self.name, red_op, red_index)
        self.image = compile_cuda(self.source)
        self._kern = None

    def __call__(self, inputs: Sequence[torch.Tensor]) -> List[torch.Tensor]:
        from .. import _lib
        dev = next(t.device for t in inputs if t.is_cuda)
        ins = [t if t.device == dev else t.to(dev) for t in inputs]
        red, others = self._alloc(dev)
        if self.rows == 0 or self.cols == 0:
            return [red] + others
        if self._kern is None:
            lib, fn = ctypes.c_void_p(), ctypes.c_void_p()
            self._img = ctypes.create_string_buffer(self.image, len(self.image))
            _lib.call("ft_jit_load", ctypes.addressof(self._img), ctypes.addressof(lib))
            nb = ctypes.create_string_buffer(self.name.encode())
            _lib.call("ft_jit_get_kernel", lib.value, ctypes.addressof(nb), ctypes.addressof(fn))
            self._lib_handle, self._kern = lib, fn.value
        args = [ctypes.c_void_p(t.data_ptr()) for t in ins] + [ctypes.c_void_p(red.data_ptr())] + [ctypes.c_void_p(t.data_ptr()) for t in others]
        args += [ctypes.c_longlong(self.rows), ctypes.c_int(self.cols), self._strides(ins)]
        arr = (ctypes.c_void_p * len(args))(*[ctypes.addressof(a) for a in args])
        _lib.call("ft_jit_launch", self._kern, self.rows, 256, 0, ctypes.addressof(arr), _lib.S())
        return [red] + others


class HostFusedReduceKernel(_FusedReduceBase):
    def __init__(self, body, red_op, red_index, keepdim):
        super().__init__(body, red_op, red_index, keepdim)
        self.name = f"ft_fusedred_{self.fp}_h"
        self.source = generate_host_reduce(body, self.name, red_op, red_index)
        key = hashlib.sha256((_HOST_FLAGS_TAG + self.source).encode()).hexdigest()
        _cache_dir.mkdir(parents=True, exist_ok=True)
        so = _cache_dir / f"{key}.so"
        if not so.exists():
            cpp = _cache_dir / f"{key}.cpp"
            cpp.write_text(self.source)
            tmp = _cache_dir / f"{key}.{os.getpid()}.tmp.so"
            r = subprocess.run([os.environ.get("CXX", "g++"), "-O3", "-march=native", "-fno-math-errno", "-fno-trapping-math", "-fopenmp-simd", "-pthread", "-shared", "-fPIC",
                                "-std=c++17", str(cpp), "-o", str(tmp)],
                               capture_output=True, text=True)
            if r.returncode != 0:
                raise FerrotorchError("host codegen compilation failed:\n" + r.stderr + "\n--- source ---\n" + self.source)
            os.replace(tmp, so)
        self.lib = ctypes.CDLL(str(so))
        self.fn = getattr(self.lib, self.name)
        self.fn.restype = None

    def __call__(self, inputs: Sequence[torch.Tensor]) -> List[torch.Tensor]:
        red, others = self._alloc("cpu")
        if self.rows == 0 or self.cols == 0:
            return [red] + others
        st = self._strides(inputs)
        args = [ctypes.c_void_p(t.data_ptr()) for t in inputs] + [ctypes.c_void_p(red.data_ptr())] + [ctypes.c_void_p(t.data_ptr()) for t in others]
        self.fn(*args, ctypes.c_longlong(self.rows), ctypes.c_int(self.cols), ctypes.byref(st))
        return [red] + others
