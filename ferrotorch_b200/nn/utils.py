"""Gradient utilities (ferrotorch-nn/src/utils.rs:134-352) and sequence packing helpers."""
from .extras import clip_grad_norm_, clip_grad_value_, PackedSequence, pack_padded_sequence, pad_packed_sequence

__all__ = ["clip_grad_norm_", "clip_grad_value_", "PackedSequence", "pack_padded_sequence", "pad_packed_sequence"]
