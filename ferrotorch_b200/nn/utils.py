"""Gradient utilities (ferrotorch-nn/src/utils.rs:134-352) and sequence packing helpers (rnn_utils.rs)."""
from .extras import clip_grad_norm_, clip_grad_value_
from .rnn import PackedSequence, pack_padded_sequence, pad_packed_sequence, pad_sequence, pack_sequence

__all__ = ["clip_grad_norm_", "clip_grad_value_", "PackedSequence", "pack_padded_sequence", "pad_packed_sequence", "pad_sequence", "pack_sequence"]
