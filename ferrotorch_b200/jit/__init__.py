"""Tracing JIT: record -> graph IR -> optimisation passes -> fused-kernel code generation (NVRTC sm_100a / host C++) or interpretation."""
from . import ir, trace as _trace_mod, interpreter, passes, codegen, module, script as _script_mod
from .ir import IrGraph, IrNode, IrValue
from .trace import trace
from .interpreter import Interpreter, run_graph
from .passes import (optimize, constant_folding, dead_code_elimination, common_subexpression_elimination, algebraic_simplification,
                     find_fusion_groups, fuse_elementwise, fuse_reductions, plan_memory, FusionGroup, MemoryPlan)
from .codegen import (generate_cuda, generate_host, generate_cuda_reduce, generate_host_reduce, compile_cuda, CudaFusedKernel, HostFusedKernel,
                      CudaFusedReduceKernel, HostFusedReduceKernel)
from .module import (compile, CompiledFunction, CompileStats, split_at_breaks, aot_trace_joint, aot_function, JointGraph, SymbolicDim, ShapeEnv,
                     export, ExportedProgram, Autotuner, TuneResult)
from .script import script, GraphBuilder, ScriptedFunction, Value

__all__ = [n for n in dir() if not n.startswith("_")]
