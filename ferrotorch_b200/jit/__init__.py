"""Tracing JIT: record -> graph IR -> optimisation passes -> fused-kernel code generation (NVRTC sm_100a / host C++) or interpretation."""
from . import ir, trace as _trace_mod, interpreter, passes, codegen, module, script as _script_mod
from .ir import IrGraph, IrNode, IrValue
from .trace import trace
from .interpreter import Interpreter, run_graph
from .passes import (optimize, constant_folding, dead_code_elimination, common_subexpression_elimination, algebraic_simplification,
                     find_fusion_groups, fuse_elementwise, fuse_reductions, plan_memory, FusionGroup, MemoryPlan)
from .codegen import (generate_cuda, generate_host, generate_cuda_reduce, generate_host_reduce, compile_cuda, CudaFusedKernel, HostFusedKernel,
                      CudaFusedReduceKernel, HostFusedReduceKernel)
from .module import (compile, CompiledFunction, CompileStats, split_at_breaks, GraphSegment, aot_trace_joint, aot_function, JointGraph, SymbolicDim, ShapeEnv,
                     export, ExportedProgram, Autotuner, TuneResult)
from .script import script, GraphBuilder, ScriptedFunction, Value
from .api_ext import (JitError, interpret, interpret_multi, interpret_multi_with_captures, OptimizationConfig, optimize_with_config, CompileConfig, TracedModule,
                      compile_with_config, Segment, SegmentedModule, TraceResult, trace_with_breaks, SymbolicDimSpec, ShapeSignature, Guard,
                      patch_reshape_for_symbolic_dims, SymbolicTracedModule, compile_symbolic, DimSpec, InputSpec, ExportedProgramMetadata, program_metadata,
                      DynamicExportedProgram, export_with_dynamic_shapes, AotGraphPair, decompose_forward_backward, AotCompiledModule, compile_aot,
                      CompiledGraph, Codegen, InterpreterBackend, NativeBackend, InductorTarget, InductorCompileStatus, InductorBackend, BinOpKind, UnaryOpKind,
                      Expr, LoopIR, CpuCodegen, GpuCodegen, JitCompiledKernel, compile_loop_ir_kernel, lower_to_loops, FusionGroupKind, ReductionKind, FusedOp,
                      FusedChain, is_fusion_enabled, with_fusion, apply_fused, estimate_numel_for_inputs, estimate_matmul_dims, generate_reduction_c,
                      generate_reduction_cuda, generate_reduction_ptx, AutotuneKey, AutotuneCandidate, AutotuneResult, Autotuner)

__all__ = [n for n in dir() if not n.startswith("_")]
