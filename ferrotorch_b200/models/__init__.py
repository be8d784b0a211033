"""Model zoo: Llama (training, tensor-parallel inference, generation), BERT, Whisper, Stable Diffusion, GCN, RL policies."""
from . import llama, llama_gen, bert, whisper, diffusion, graph, rl
from .llama import LlamaConfig, LlamaModel, LlamaForCausalLM, LlamaDecoderLayer
from .llama_gen import (CachedLlama, KvCache, LayerKvCache, GenerationConfig, generate, beam_search, SpecDecodeConfig, SpecDecodeStats,
                        speculative_generate, dequantize_gptq_q4, dequantize_awq_q4, dequantize_hqq, gguf_to_hf_name, remap_gguf_state_dict)
from .bert import BertConfig, BertModel, SentenceTransformer, load_bert_model
from .whisper import WhisperConfig, WhisperEncoder, log_mel_spectrogram, load_whisper_encoder
from .diffusion import (UNet2DConditionModel, UNetConfig, AutoencoderKL, VaeConfig, VaeEncoder, VaeDecoder, ClipTextEncoder, ClipTextConfig,
                        DDIMScheduler, StableDiffusionPipeline)
from .graph import Graph, GcnConv, GcnNet, load_gcn_net
from .rl import MlpPolicy, MlpPolicyConfig, load_ppo_policy, ppo_loss

__all__ = [n for n in dir() if not n.startswith("_")]
