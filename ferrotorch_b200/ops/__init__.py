"""Hot-path operators: each one is a thin launcher around a hand-written sm_100a kernel
(with an f32 PyTorch evaluation of the same math for CPU tensors, used as the test oracle)."""
from .gemm import gemm, linear, linear_master, matmul_exact, mv, dot, bmm
from .norm import rms_norm, layer_norm, rmsnorm_fwd, rmsnorm_bwd
from .llama import (rope_tables, rope_inplace, apply_rope, swiglu, swiglu_fwd, swiglu_bwd, embedding, embedding_fwd,
                    embedding_bwd, add_)
from .loss import cross_entropy, cross_entropy_fwd_bwd
from .optim import adamw_flat_, sgd_flat_, grad_norm_, scale_
from .attention import attention_packed, flash_fwd, flash_bwd
from . import attention

__all__ = [n for n in dir() if not n.startswith("_")]
from . import tensor_ops  # noqa: E402
from . import nn_ops  # noqa: E402
from . import conv  # noqa: E402
from .conv import conv3x3, conv3x3_nhwc_raw  # noqa: E402
