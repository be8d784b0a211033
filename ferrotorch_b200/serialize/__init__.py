"""Serialization: SafeTensors, native state dict, training checkpoints, PyTorch .pt, GGUF, ONNX."""
from .safetensors_io import (save_safetensors, load_safetensors, load_safetensors_filtered, load_safetensors_mmap, safetensors_metadata,
                             save_safetensors_sharded, load_safetensors_sharded)
from .formats import (save_state_dict, load_state_dict, dumps_state_dict, loads_state_dict, TrainingCheckpoint, save_checkpoint,
                      load_checkpoint, AsyncCheckpointer, CheckpointFuture, load_pytorch_state_dict, save_pytorch_state_dict, parse_gguf,
                      dequantize_gguf, GgufFile, GgufTensorInfo, GGML_TYPES, export_onnx, OnnxExportConfig)
from .extras import (load_safetensors_auto, ShardProgress, load_safetensors_sharded_with_progress, load_safetensors_sharded_mmap,
                     load_safetensors_sharded_filtered, GgmlType, GgufValue, GgufMetadata, GgufTensor, GgufData, parse_gguf_bytes, load_gguf,
                     load_gguf_mmap, dequantize_gguf_tensor, load_gguf_state_dict, load_gguf_state_dict_mmap, PickleValue, parse_pickle,
                     save_pytorch, validate_checkpoint, load_pytorch_state_dict_mmap)
from .onnx_ir import ir_graph_to_onnx, export_ir_graph_to_onnx, export_from_program
