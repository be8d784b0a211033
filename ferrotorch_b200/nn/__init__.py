"""Neural-network layers, losses, initialisers and utilities (API names follow ferrotorch-nn)."""
from .module import (Module, Parameter, Buffer, StateDict, Reduction, Sequential, ModuleList, ModuleDict, ParameterList, ParameterDict,
                     HookHandle, HookedModule, derive_module, param, submodule, skip, DeriveError)
from .layers import *  # noqa: F401,F403
from .layers import (Linear, LazyLinear, LoRALinear, SqueezeExcitation, RMSNorm, LayerNorm, Embedding, RoPEConvention, RoPEScaling,
                     RotaryPositionEmbedding, SwiGLU, KVCache, MultiheadAttention, CrossEntropyLoss, repeat_kv, reshape_to_heads,
                     transpose_heads_to_2d, standard_attention, flash_attention, attention_backend, PaddingMode, RNNNonlinearity, EmbeddingBagMode)
from .extras import (KVPage, PagePool, PagedKVCache, PagedAttentionManager, BlockMask, flex_attention, causal_score_mod, alibi_score_mod,
                     relative_position_score_mod, NonLinearity, init, clip_grad_norm_, clip_grad_value_, PackedSequence,
                     pack_padded_sequence, pad_packed_sequence, interpolate, grid_sample, affine_grid, functional_pad_1d,
                     functional_pad_2d, functional_pad_3d, ObserverType, QatConfig, FakeQuantize, QuantizedModel, QatModel, prepare_qat, InterpolateMode,
                     GridSampleMode, GridSamplePaddingMode, GeluApproximate, GELU, gelu, gelu_with, relative_position_bias_score_mod, max_pool1d, max_pool2d,
                     max_pool3d, avg_pool1d, avg_pool2d, avg_pool3d, adaptive_avg_pool1d, adaptive_avg_pool2d, adaptive_avg_pool3d, adaptive_max_pool1d,
                     adaptive_max_pool2d, adaptive_max_pool3d, lp_pool1d, lp_pool2d, max_unpool2d, pixel_shuffle, pixel_unshuffle, unfold, fold,
                     ForwardHook, ForwardPreHook, BackwardHook)
from .module import derive_module as DeriveModule  # noqa: E402,N812  (the reference's derive macro, here a class decorator)
from . import functional
from .compute_copy import attach_compute_copies, detach_compute_copies, compute_copy
from . import utils
