"""Serialization: SafeTensors, native state dict, training checkpoints, PyTorch .pt, GGUF, ONNX."""
from .safetensors_io import (save_safetensors, load_safetensors, load_safetensors_filtered, load_safetensors_mmap, safetensors_metadata,
                             save_safetensors_sharded, load_safetensors_sharded)
from .formats import (save_state_dict, load_state_dict, dumps_state_dict, loads_state_dict, TrainingCheckpoint, save_checkpoint,
                      load_checkpoint, AsyncCheckpointer, CheckpointFuture, load_pytorch_state_dict, save_pytorch_state_dict, parse_gguf,
                      dequantize_gguf, GgufFile, GgufTensorInfo, GGML_TYPES, export_onnx, OnnxExportConfig)
