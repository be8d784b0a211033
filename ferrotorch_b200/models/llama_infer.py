"""Tensor-parallel Llama inference engine: prefill with the training-path kernels, decode with a paged KV cache
(block size 16), split-K weight-streaming GEMMs, fused plane-consuming epilogues and one-shot all-reduces over NVLink peer
memory, the whole decode step replayed from one CUDA graph.

Sharding (tensor-parallel degree ``tp`` = world size of the group):
  * ``wqkv``  column-parallel: each rank owns ``Hq/tp`` query heads and ``Hkv/tp`` KV heads (rows of the fused QKV matrix)
  * ``wo``    row-parallel:    each rank owns the matching ``Hq/tp * D`` input columns; outputs are partial sums -> all-reduce
  * ``wgu``   column-parallel: ``F/tp`` gate rows and ``F/tp`` up rows;   ``wd`` row-parallel over ``F/tp`` input columns -> all-reduce
  * ``lm_head`` vocabulary-parallel (``V/tp`` rows); the embedding table is replicated (2 GB at d=8192; avoids an extra all-reduce)

Reference parity: ferrotorch-llama/src/gpu.rs:83-700 (single-GPU, batch-1, no KV cache inferencer), generation.rs:110 (greedy),
kv_cache.rs:37-207; tensor parallelism itself is absent from the reference (docs/audit/11-ferrotorch-distributed.md:66-68).
"""
from __future__ import annotations

import ctypes
import math
import zlib
from dataclasses import dataclass
from typing import Dict, List, Optional

import torch

from .. import _lib, ops
from ..errors import InvalidArgument
from .llama import LlamaConfig

PAD_ROWS = 16          # decode token rows are padded to 16 (the GEMM's A-operand rows)
KV_BLOCK = 16


class TPContext:
    """Rank/world of the tensor-parallel group plus the symmetric buffers the decode all-reduce uses."""

    def __init__(self, device, group=None):
        import torch.distributed as dist
        self.device = torch.device(device)
        self.dist = dist if (dist.is_available() and dist.is_initialized()) else None
        self.group = group
        self.world = self.dist.get_world_size(group) if self.dist else 1
        self.rank = self.dist.get_rank(group) if self.dist else 0
        self.comm = None          # host-numbered launches (prefill all-reduces)
        self.comm_graph = None    # device-numbered launches (replayed from CUDA graphs); its own flag block, the two numberings must not mix
        if self.world > 1:
            from ..parallel.symm import SymmComm
            self.comm = SymmComm(self.device, group)
            self.comm_graph = SymmComm(self.device, group)

    def symmetric(self, numel: int, dtype: torch.dtype, zero: bool = True):
        """(local tensor, ctypes array of every rank's pointer) - a plain local buffer when the group has one rank."""
        if self.world == 1:
            t = torch.zeros(numel, device=self.device, dtype=dtype)
            return t, (ctypes.c_void_p * 1)(t.data_ptr()), None
        from ..parallel.symm import SymmetricBuffer
        b = SymmetricBuffer(numel, dtype, self.device, self.group, zero=zero)
        return b.tensor, b.ptr_array(), b


def _splits_for(N: int, K: int, sms: int = 148) -> int:
    """Number of K slices for a decode GEMM. Cost model per work item (one 256-row weight tile x one K slice): weight bytes streamed,
    32 KiB of partial-plane write + read, and ~90 KB-equivalent of pipeline fill/drain; the estimate is waves x item cost, minimised
    over the slice counts that leave no empty slice."""
    tiles_n = (N + 255) // 256
    kb = (K + 63) // 64
    best, best_t = 1, float("inf")
    for sp in range(1, min(kb, 64) + 1):
        kb_per = -(-kb // sp)
        if -(-kb // kb_per) != sp:
            continue
        items = tiles_n * sp
        t = math.ceil(items / sms) * (256 * kb_per * 64 * 2 + 32768 + 90000)
        if t < best_t:
            best, best_t = sp, t
    return best


class _SplitKGemm:
    """``P[s][16][N] = x[16,K] . W[N,K]^T`` restricted to K-slice s; owns its partial-plane buffer."""

    def __init__(self, weight: torch.Tensor, device, cache: Optional[dict] = None):
        self.w = weight
        self.N, self.K = weight.shape
        self.splits = _splits_for(self.N, self.K)
        self.ldp = (self.N + 3) // 4 * 4
        key = (self.N, self.K)
        if cache is not None and key in cache:          # layers of the same shape share one plane buffer (they run one after another)
            self.planes = cache[key]
        else:
            self.planes = torch.zeros(self.splits, PAD_ROWS, self.ldp, device=device, dtype=torch.float32)
            if cache is not None:
                cache[key] = self.planes
        self.plane_stride = PAD_ROWS * self.ldp

    def __call__(self, x16: torch.Tensor) -> None:
        _lib.call("ft_gemm_bf16_splitk", x16, self.w, self.planes, PAD_ROWS, self.N, self.K, x16.stride(0), self.w.stride(0), self.ldp, 0, 0,
                  self.splits, _lib.S())


class LlamaTPEngine:
    """``engine.generate(prompt_ids, max_new_tokens)`` -> greedy continuation; ``prefill`` / ``decode_step`` for finer control."""

    def __init__(self, cfg: LlamaConfig, ctx: Optional[TPContext] = None, max_batch: int = 8, max_seq: int = 2304, device="cuda", seed: int = 0,
                 weights: Optional[Dict[str, torch.Tensor]] = None, use_graph: bool = True):
        cfg.validate()
        if cfg.hidden_act not in ("silu", "swish"):
            raise InvalidArgument(f"the tensor-parallel decode kernels implement SwiGLU only; use models.LlamaGpuInferencer for {cfg.hidden_act!r}")
        self.cfg, self.ctx = cfg, ctx or TPContext(device)
        self.dev = self.ctx.device
        tp, r = self.ctx.world, self.ctx.rank
        if cfg.num_attention_heads % tp or cfg.num_key_value_heads % tp or cfg.intermediate_size % tp or cfg.vocab_size % tp:
            raise InvalidArgument(f"heads / kv heads / ffn / vocab must be divisible by the tensor-parallel degree {tp}")
        if cfg.head_dim != 128:
            raise InvalidArgument("the decode kernels are specialised for head_dim 128")
        if max_batch > PAD_ROWS:
            raise InvalidArgument(f"decode batch is limited to {PAD_ROWS} sequences per engine")
        self.B, self.max_seq = max_batch, max_seq
        self.Hq, self.Hkv, self.D = cfg.num_attention_heads // tp, cfg.num_key_value_heads // tp, cfg.head_dim
        self.F, self.d, self.V = cfg.intermediate_size // tp, cfg.hidden_size, cfg.vocab_size // tp
        self.use_graph = use_graph
        self._init_weights(seed, weights)
        self._init_buffers()
        self.graph = None

    # ------------------------------------------------------------------ weights ------------------------------------------------------------------
    def _init_weights(self, seed: int, weights) -> None:
        cfg, tp, r, dev = self.cfg, self.ctx.world, self.ctx.rank, self.dev
        D, d = self.D, self.d
        Hq_t, Hkv_t, F_t = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.intermediate_size
        g = torch.Generator(device=dev)

        def full(name: str, shape, layer: int):
            if weights is not None:
                return weights[name].to(dev, torch.bfloat16)
            g.manual_seed(seed * 1000003 + layer * 1009 + zlib.crc32(name.encode()) % 997)   # identical on every rank
            return (torch.randn(shape, device=dev, generator=g, dtype=torch.float32) * 0.02).to(torch.bfloat16)

        self.layers = []
        pc: dict = {}
        for i in range(cfg.num_hidden_layers):
            p = f"model.layers.{i}."
            q = full(p + "self_attn.q_proj.weight", (Hq_t * D, d), i)[r * self.Hq * D:(r + 1) * self.Hq * D]
            k = full(p + "self_attn.k_proj.weight", (Hkv_t * D, d), i)[r * self.Hkv * D:(r + 1) * self.Hkv * D]
            v = full(p + "self_attn.v_proj.weight", (Hkv_t * D, d), i)[r * self.Hkv * D:(r + 1) * self.Hkv * D]
            wqkv = torch.cat([q, k, v], 0).contiguous()
            del q, k, v
            wo = full(p + "self_attn.o_proj.weight", (d, Hq_t * D), i)[:, r * self.Hq * D:(r + 1) * self.Hq * D].contiguous()
            gate = full(p + "mlp.gate_proj.weight", (F_t, d), i)[r * self.F:(r + 1) * self.F]
            up = full(p + "mlp.up_proj.weight", (F_t, d), i)[r * self.F:(r + 1) * self.F]
            wgu = torch.cat([gate, up], 0).contiguous()
            del gate, up
            wd = full(p + "mlp.down_proj.weight", (d, F_t), i)[:, r * self.F:(r + 1) * self.F].contiguous()
            n1 = weights[p + "input_layernorm.weight"].to(dev, torch.bfloat16) if weights is not None else torch.ones(d, device=dev, dtype=torch.bfloat16)
            n2 = weights[p + "post_attention_layernorm.weight"].to(dev, torch.bfloat16) if weights is not None else torch.ones(d, device=dev, dtype=torch.bfloat16)
            self.layers.append(dict(wqkv=wqkv, wo=wo, wgu=wgu, wd=wd, n1=n1, n2=n2, g_qkv=_SplitKGemm(wqkv, dev, pc), g_o=_SplitKGemm(wo, dev, pc),
                                    g_gu=_SplitKGemm(wgu, dev, pc), g_d=_SplitKGemm(wd, dev, pc)))
        self.embed = full("model.embed_tokens.weight", (cfg.vocab_size, d), 10001)
        self.final_norm = weights["model.norm.weight"].to(dev, torch.bfloat16) if weights is not None else torch.ones(d, device=dev, dtype=torch.bfloat16)
        head = self.embed if cfg.tie_word_embeddings else full("lm_head.weight", (cfg.vocab_size, d), 10002)
        self.lm_head = head[r * self.V:(r + 1) * self.V].contiguous()
        self.g_head = _SplitKGemm(self.lm_head, dev)
        self.cos, self.sin = ops.rope_tables(self.max_seq, D, cfg.rope_theta, dev, cfg.rope_scaling)

    # ------------------------------------------------------------------ buffers ------------------------------------------------------------------
    def _init_buffers(self) -> None:
        dev, B, d = self.dev, self.B, self.d
        L = self.cfg.num_hidden_layers
        self.max_blocks = (self.max_seq + KV_BLOCK - 1) // KV_BLOCK
        nblk = B * self.max_blocks
        self.k_cache = [torch.zeros(nblk, KV_BLOCK, self.Hkv, self.D, device=dev, dtype=torch.bfloat16) for _ in range(L)]
        self.v_cache = [torch.zeros(nblk, KV_BLOCK, self.Hkv, self.D, device=dev, dtype=torch.bfloat16) for _ in range(L)]
        self.block_table = (torch.arange(B, device=dev, dtype=torch.int32).view(B, 1) * self.max_blocks
                            + torch.arange(self.max_blocks, device=dev, dtype=torch.int32).view(1, -1)).contiguous()
        self.positions = torch.zeros(B, device=dev, dtype=torch.int32)       # index of the token being decoded
        self.seq_lens = torch.zeros(B, device=dev, dtype=torch.int32)        # tokens in the cache after this step's write
        self.tokens = torch.zeros(B, device=dev, dtype=torch.int64)
        self.x = torch.zeros(PAD_ROWS, d, device=dev, dtype=torch.bfloat16)          # residual stream
        self.h = torch.zeros(PAD_ROWS, d, device=dev, dtype=torch.bfloat16)          # normalised activations
        self.q = torch.zeros(PAD_ROWS, self.Hq * self.D, device=dev, dtype=torch.bfloat16)
        self.attn = torch.zeros(PAD_ROWS, self.Hq * self.D, device=dev, dtype=torch.bfloat16)
        self.act = torch.zeros(PAD_ROWS, self.F, device=dev, dtype=torch.bfloat16)
        self.logits = torch.zeros(B, self.V, device=dev, dtype=torch.float32)
        # Splits over the sequence: up to 256 CTAs across (batch, kv head, split), which stays inside one resident wave of two CTAs per SM,
        # at most 16 splits (one round of partial loads in the combining CTA) and at least 64 cached tokens (one staged chunk) per split
        # at the longest sequence. Measured at batch 8, 2304 tokens: 1 KV head 17 us at 12-16 splits against 21.5 us at 37; 8 KV heads
        # 31 us at 4 splits against 47 us at 16.
        self.nsplit = max(1, min(16, 256 // max(1, B * self.Hkv), self.max_seq // 64))
        self.attn_ws = torch.zeros(B * self.Hkv * self.nsplit * (self.Hq // self.Hkv) * 132, device=dev, dtype=torch.float32)
        self.attn_ctr = torch.zeros(B * self.Hkv, device=dev, dtype=torch.int32)
        # all-reduce staging: two slots of [PAD_ROWS, d] floats per rank + flag block + grid-barrier ints
        self.ar_sym, self.ar_sym_ptrs, self._ar_sym_buf = self.ctx.symmetric(2 * PAD_ROWS * d, torch.float32)
        self.ar_flags, self.ar_flag_ptrs, self._ar_flag_buf = self.ctx.symmetric(8, torch.int32)
        # the cluster form of the kernel numbers its launches and keeps its flags apart from the grid-barrier form: either may run at any step
        self.ar_flags_cl, self.ar_flag_ptrs_cl, self._ar_flag_buf_cl = self.ctx.symmetric(8 * PAD_ROWS * 4, torch.int32)
        self.ar_sync_cl = torch.zeros(4, device=dev, dtype=torch.int32)
        import os
        form = os.environ.get("FT_DECODE_AR", "grid")
        self.ar_cluster = d % 16 == 0 and form in ("cluster", "push")
        # push form: every rank stores its partial rows into all staging buffers ([world][PAD_ROWS][d] per slot) and reads only local memory
        self.ar_push = self.ar_cluster and form == "push" and self.ctx.world > 1
        if self.ar_push:
            self.ar_sym_push, self.ar_sym_push_ptrs, self._ar_sym_push_buf = self.ctx.symmetric(2 * self.ctx.world * PAD_ROWS * d, torch.float32)
        self.ar_sync = torch.zeros(4, device=dev, dtype=torch.int32)
        self.ar_chunks = max(1, min(16, 128 // max(B, 1)))
        while d % self.ar_chunks:
            self.ar_chunks -= 1
        self.ar_sumsq = torch.zeros(2 * PAD_ROWS * self.ar_chunks, device=dev, dtype=torch.float32)
        # sampling exchange: every rank contributes (max logit, global index) per sequence
        self.pick_sym, self.pick_ptrs, self._pick_buf = self.ctx.symmetric(self.ctx.world * PAD_ROWS * 2, torch.float32)
        self.pick_out = torch.zeros(self.ctx.world * PAD_ROWS * 2, device=dev, dtype=torch.float32)
        self.pick_seq = torch.zeros(1, device=dev, dtype=torch.int32)
        if self.ctx.world > 1:
            torch.cuda.synchronize(dev)
            self.ctx.dist.barrier(self.ctx.group)

    # ------------------------------------------------------------------ pieces -------------------------------------------------------------------
    def _ar_norm(self, gemm: _SplitKGemm, w: torch.Tensor) -> None:
        if self.ar_cluster:
            _lib.call("ft_decode_ar_residual_norm_cluster", gemm.planes, gemm.splits, gemm.ldp, gemm.plane_stride,
                      self.ar_sym_push_ptrs if self.ar_push else self.ar_sym_ptrs, self.ar_flag_ptrs_cl, self.ctx.rank, self.ctx.world, self.ar_sync_cl,
                      self.x, w, self.h, self.B, PAD_ROWS, self.d, float(self.cfg.rms_norm_eps), int(self.ar_push), _lib.S())
            return
        _lib.call("ft_decode_ar_residual_norm", gemm.planes, gemm.splits, gemm.ldp, gemm.plane_stride, self.ar_sym_ptrs, self.ar_flag_ptrs,
                  self.ctx.rank, self.ctx.world, self.ar_sync, self.x, w, self.h, self.ar_sumsq, self.B, PAD_ROWS, self.d, self.ar_chunks,
                  float(self.cfg.rms_norm_eps), _lib.S())

    def _pick_tokens(self) -> None:
        """Greedy sampling across the vocabulary shards: local max/argmax, one-shot exchange, global argmax."""
        val, idx = self.logits.max(dim=1)
        w, r = self.ctx.world, self.ctx.rank
        if w == 1:
            self.tokens.copy_(idx)
            return
        slot = self.pick_sym.view(w, PAD_ROWS, 2)
        slot.zero_()
        slot[r, : self.B, 0] = val
        slot[r, : self.B, 1] = (idx + r * self.V).float()
        self.ctx.comm_graph.all_reduce_small(self._pick_buf, self.pick_out, w * PAD_ROWS * 2, seq_dev=self.pick_seq)
        allv = self.pick_out.view(w, PAD_ROWS, 2)
        best = allv[:, : self.B, 0].argmax(dim=0)
        self.tokens.copy_(allv[best, torch.arange(self.B, device=self.dev), 1].long())

    def _decode_body(self) -> None:
        """One decode step. The step's kernels are launched as programmatic dependents (each waits on the device for its predecessor before
        touching memory, but is scheduled while the predecessor drains), which hides the launch gaps between the ~9 small kernels of a layer.
        ``FT_DECODE_PDL=0`` switches to ordinary launches."""
        import os
        prev = _lib.kernels().ft_set_pdl(int(os.environ.get("FT_DECODE_PDL", "1") != "0"))
        try:
            self._decode_body_inner()
        finally:
            _lib.kernels().ft_set_pdl(prev)

    @torch.no_grad()
    def profile_decode(self, steps: int = 10) -> Dict[str, float]:
        """Per-kernel-class device time of an eager (no graph, ordinary launches) decode step, in microseconds per step, from CUDA events around
        every launch: where a step's time goes when it is latency-bound. Advances the sequence by ``steps`` tokens."""
        import os
        old_env = os.environ.get("FT_DECODE_PDL")
        os.environ["FT_DECODE_PDL"] = "0"
        totals: Dict[str, float] = {}
        try:
            for it in range(steps + 2):
                self._prof = []
                self._decode_body()
                torch.cuda.synchronize(self.dev)
                if it >= 2:
                    for name, e0, e1 in self._prof:
                        totals[name] = totals.get(name, 0.0) + e0.elapsed_time(e1) * 1e3 / steps
        finally:
            self._prof = None
            if old_env is None:
                os.environ.pop("FT_DECODE_PDL", None)
            else:
                os.environ["FT_DECODE_PDL"] = old_env
        totals["sum"] = sum(totals.values())
        return totals

    def _timed(self, name: str, fn, *args) -> None:
        prof = getattr(self, "_prof", None)
        if prof is None:
            fn(*args)
            return
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn(*args)
        e1.record()
        prof.append((name, e0, e1))

    def _decode_body_inner(self) -> None:
        cfg, B = self.cfg, self.B
        self.x[:B] = self.embed[self.tokens]
        _lib.call("ft_rmsnorm_fwd", self.x, None, self.layers[0]["n1"], self.h, None, None, B, self.d, float(cfg.rms_norm_eps), _lib.S())
        scale = 1.0 / math.sqrt(self.D)
        T = self._timed
        for li, L in enumerate(self.layers):
            T("gemm_qkv", L["g_qkv"], self.h)
            g = L["g_qkv"]
            T("rope_kvwrite", _lib.call, "ft_decode_qkv_rope_kvwrite", g.planes, g.splits, g.ldp, g.plane_stride, B, self.Hq, self.Hkv, self.D, self.positions,
              self.cos, self.sin, self.q, self.k_cache[li], self.v_cache[li], self.block_table, self.max_blocks, _lib.S())
            T("paged_attention", _lib.call, "ft_paged_attn_decode", self.q, self.k_cache[li], self.v_cache[li], self.block_table, self.max_blocks, self.seq_lens, B,
              self.Hq, self.Hkv, self.D, float(scale), self.nsplit, self.attn_ws, self.attn_ctr, self.attn, _lib.S())
            T("gemm_o", L["g_o"], self.attn)
            T("allreduce_residual_norm", self._ar_norm, L["g_o"], L["n2"])
            T("gemm_gate_up", L["g_gu"], self.h)
            g = L["g_gu"]
            T("swiglu", _lib.call, "ft_decode_swiglu", g.planes, g.splits, g.ldp, g.plane_stride, B, self.F, self.act, _lib.S())
            T("gemm_down", L["g_d"], self.act)
            nxt = self.layers[li + 1]["n1"] if li + 1 < len(self.layers) else self.final_norm
            T("allreduce_residual_norm", self._ar_norm, L["g_d"], nxt)
        self.g_head(self.h)
        g = self.g_head
        _lib.call("ft_splitk_reduce", g.planes, g.splits, B, self.V, g.ldp, g.plane_stride, None, self.logits, self.V, 1, _lib.S())
        self._pick_tokens()
        self.positions += 1
        self.seq_lens += 1

    # ------------------------------------------------------------------ public API ----------------------------------------------------------------
    @torch.no_grad()
    def prefill(self, ids: torch.Tensor) -> torch.Tensor:
        """Run the prompt (``ids`` ``[B, S]``, equal lengths), fill the KV cache, return the first generated token of every sequence."""
        cfg, ctx = self.cfg, self.ctx
        B, S = ids.shape
        if B != self.B or S + 1 > self.max_seq:
            raise InvalidArgument("prompt batch must equal the engine batch and fit the cache")
        T = B * S
        x = self.embed[ids.reshape(-1).to(self.dev)]
        ar_buf = None
        if ctx.world > 1:
            from ..parallel.symm import SymmetricBuffer
            ar_buf = SymmetricBuffer(T * self.d, torch.bfloat16, self.dev, ctx.group)
            torch.cuda.synchronize(self.dev)
            ctx.dist.barrier(ctx.group)

        def row_parallel(a, w):
            if ar_buf is None:
                return ops.gemm(a, w)
            out = ar_buf.tensor.view(T, self.d)
            ops.gemm(a, w, out=out)
            ctx.comm.all_reduce_(ar_buf, T * self.d, use_nvls=True)
            return out
        for li, L in enumerate(self.layers):
            h, _, _ = ops.rmsnorm_fwd(x, L["n1"], cfg.rms_norm_eps)
            qkv = ops.gemm(h, L["wqkv"])
            ops.rope_inplace(qkv, self.cos, self.sin, S, 0, self.Hq + self.Hkv, self.D)
            _lib.call("ft_paged_kv_write", qkv, qkv.stride(0), B, S, self.Hq, self.Hkv, self.D, self.k_cache[li], self.v_cache[li],
                      self.block_table, self.max_blocks, 0, _lib.S())
            attn, _ = ops.flash_fwd(qkv, B, S, self.Hq, self.Hkv, self.D, True)
            o = row_parallel(attn, L["wo"])
            h2, _, x = ops.rmsnorm_fwd(o, L["n2"], cfg.rms_norm_eps, residual=x)
            gu = ops.gemm(h2, L["wgu"])
            a = ops.swiglu_fwd(gu)
            dn = row_parallel(a, L["wd"])
            x = ops.add_(x, dn)
            del h, qkv, attn, o, h2, gu, a, dn
        last = x.view(B, S, self.d)[:, -1].contiguous()
        hl, _, _ = ops.rmsnorm_fwd(last, self.final_norm, cfg.rms_norm_eps)
        self.logits.copy_(ops.gemm(hl, self.lm_head, out_dtype=torch.float32))
        self.positions.fill_(S)
        self.seq_lens.fill_(S + 1)
        self._pick_tokens()
        if ctx.world > 1:
            torch.cuda.synchronize(self.dev)
            ctx.dist.barrier(ctx.group)
        return self.tokens.clone()

    @torch.no_grad()
    def decode_step(self) -> torch.Tensor:
        """Feed the last sampled tokens, append their K/V, return the next tokens ``[B]`` (greedy)."""
        if not self.use_graph:
            self._decode_body()
            return self.tokens
        if self.graph is None:
            # warm up outside capture (lazy initialisations: kernel attributes, status word), then capture one step
            state = (self.positions.clone(), self.seq_lens.clone(), self.tokens.clone())
            side = torch.cuda.Stream(self.dev)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                self._decode_body()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize(self.dev)
            if self.ctx.world > 1:
                self.ctx.dist.barrier(self.ctx.group)
            # the warm-up step was a real step: rewind its effects on the positions (its cache write is simply redone)
            self.positions.copy_(state[0]); self.seq_lens.copy_(state[1]); self.tokens.copy_(state[2])
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph):
                self._decode_body()
            self.positions.copy_(state[0]); self.seq_lens.copy_(state[1]); self.tokens.copy_(state[2])
        self.graph.replay()
        return self.tokens

    @torch.no_grad()
    def generate(self, ids: torch.Tensor, max_new_tokens: int) -> torch.Tensor:
        out = [self.prefill(ids)]
        for _ in range(max_new_tokens - 1):
            out.append(self.decode_step().clone())
        return torch.stack(out, 1)

    def check(self) -> None:
        st = _lib.read_status()
        if st:
            from ..errors import Timeout
            raise Timeout(message=f"device-side wait timed out (status {st:#x})")


@torch.no_grad()
def reference_last_logits(cfg: LlamaConfig, weights: Dict[str, torch.Tensor], seq: torch.Tensor) -> torch.Tensor:
    """f32 logits of the last position of ``seq`` ``[B, S]`` from a dense forward pass (the oracle for the engine tests)."""
    return _reference(cfg, weights, seq, 1, return_logits=True)


@torch.no_grad()
def reference_generate(cfg: LlamaConfig, weights: Dict[str, torch.Tensor], ids: torch.Tensor, max_new_tokens: int) -> torch.Tensor:
    """Plain PyTorch f32 greedy generation with a dense KV-less forward."""
    return _reference(cfg, weights, ids, max_new_tokens, return_logits=False)


def _reference(cfg, weights, ids, max_new_tokens, return_logits):
    D, Hq, Hkv = cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads
    dev = ids.device
    W = {k: v.to(dev).float() for k, v in weights.items()}
    cos, sin = ops.rope_tables(ids.shape[1] + max_new_tokens + 1, D, cfg.rope_theta, dev, cfg.rope_scaling)

    def rms(v, w):
        return v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + cfg.rms_norm_eps) * w

    def rot(t):
        S = t.shape[1]
        c, s = cos[:S].view(1, S, 1, -1), sin[:S].view(1, S, 1, -1)
        a, b = t[..., : D // 2], t[..., D // 2:]
        return torch.cat([a * c - b * s, b * c + a * s], -1)
    seq = ids.clone()
    outs = []
    for _ in range(max_new_tokens):
        B, S = seq.shape
        x = W["model.embed_tokens.weight"][seq]
        for i in range(cfg.num_hidden_layers):
            p = f"model.layers.{i}."
            h = rms(x, W[p + "input_layernorm.weight"])
            q = rot((h @ W[p + "self_attn.q_proj.weight"].t()).view(B, S, Hq, D)).transpose(1, 2)
            k = rot((h @ W[p + "self_attn.k_proj.weight"].t()).view(B, S, Hkv, D)).transpose(1, 2).repeat_interleave(Hq // Hkv, 1)
            v = (h @ W[p + "self_attn.v_proj.weight"].t()).view(B, S, Hkv, D).transpose(1, 2).repeat_interleave(Hq // Hkv, 1)
            a = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(B, S, Hq * D)
            x = x + a @ W[p + "self_attn.o_proj.weight"].t()
            h2 = rms(x, W[p + "post_attention_layernorm.weight"])
            x = x + (torch.nn.functional.silu(h2 @ W[p + "mlp.gate_proj.weight"].t()) * (h2 @ W[p + "mlp.up_proj.weight"].t())) @ W[p + "mlp.down_proj.weight"].t()
        hl = rms(x[:, -1], W["model.norm.weight"])
        head = W["model.embed_tokens.weight"] if cfg.tie_word_embeddings else W["lm_head.weight"]
        logits = hl @ head.t()
        if return_logits:
            return logits
        nxt = logits.argmax(-1)
        outs.append(nxt)
        seq = torch.cat([seq, nxt[:, None]], 1)
    return torch.stack(outs, 1)


def random_hf_weights(cfg: LlamaConfig, device="cpu", seed: int = 0, std: float = 0.02) -> Dict[str, torch.Tensor]:
    """Random N(0, std) weights under the HF key names (norm weights near one) for tests and synthetic benchmarks."""
    g = torch.Generator().manual_seed(seed)
    D, d, F = cfg.head_dim, cfg.hidden_size, cfg.intermediate_size
    W = {"model.embed_tokens.weight": torch.randn(cfg.vocab_size, d, generator=g) * std, "model.norm.weight": 1 + 0.05 * torch.randn(d, generator=g)}
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        W[p + "self_attn.q_proj.weight"] = torch.randn(cfg.num_attention_heads * D, d, generator=g) * std
        W[p + "self_attn.k_proj.weight"] = torch.randn(cfg.num_key_value_heads * D, d, generator=g) * std
        W[p + "self_attn.v_proj.weight"] = torch.randn(cfg.num_key_value_heads * D, d, generator=g) * std
        W[p + "self_attn.o_proj.weight"] = torch.randn(d, cfg.num_attention_heads * D, generator=g) * std
        W[p + "mlp.gate_proj.weight"] = torch.randn(F, d, generator=g) * std
        W[p + "mlp.up_proj.weight"] = torch.randn(F, d, generator=g) * std
        W[p + "mlp.down_proj.weight"] = torch.randn(d, F, generator=g) * std
        W[p + "input_layernorm.weight"] = 1 + 0.05 * torch.randn(d, generator=g)
        W[p + "post_attention_layernorm.weight"] = 1 + 0.05 * torch.randn(d, generator=g)
    if not cfg.tie_word_embeddings:
        W["lm_head.weight"] = torch.randn(cfg.vocab_size, d, generator=g) * std
    return {k: v.to(torch.bfloat16).to(device) for k, v in W.items()}
