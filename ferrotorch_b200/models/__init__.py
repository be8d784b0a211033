"""Model zoo: Llama (training, tensor-parallel inference, generation), BERT, Whisper, Stable Diffusion, GCN, RL policies."""
from . import llama, llama_gen, bert, whisper, diffusion, graph, rl
from .llama import LlamaConfig, LlamaModel, LlamaForCausalLM, LlamaDecoderLayer
from .llama_gen import (CachedLlama, KvCache, LayerKvCache, GenerationConfig, generate, beam_search, SpecDecodeConfig, SpecDecodeStats,
                        speculative_generate, dequantize_gptq_q4, dequantize_awq_q4, dequantize_hqq, gguf_to_hf_name, remap_gguf_state_dict)
from .bert import (BertConfig, HfBertConfig, BertModel, BertEmbeddings, BertSelfAttention, BertSelfOutput, BertAttention, BertIntermediate, BertOutput,
                   BertLayer, BertEncoder, BertPooler, DropReport, SentenceTransformer, load_bert_model, load_sentence_transformer)
from .whisper import (WhisperConfig, HfWhisperConfig, WhisperEncoder, WhisperConvStem, WhisperEncoderLayer, WhisperEncoderSelfAttention,
                      log_mel_spectrogram, load_whisper_encoder, SAMPLE_RATE, N_MELS, N_FRAMES, N_FFT, HOP_LENGTH, CHUNK_LENGTH, N_SAMPLES, N_FREQS)
from .diffusion import (UNet2DConditionModel, UNetConfig, AutoencoderKL, VaeConfig, VaeEncoder, VaeDecoder, ClipTextEncoder, ClipTextConfig,
                        DDIMScheduler, StableDiffusionPipeline)
from .graph import Graph, GcnConv, GcnNet, load_gcn_net
from .rl import MlpPolicy, MlpPolicyConfig, MlpExtractor, ActionNet, ValueHead, PolicyOutput, load_ppo_policy, ppo_loss

__all__ = [n for n in dir() if not n.startswith("_")]
