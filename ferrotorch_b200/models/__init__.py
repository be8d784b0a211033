"""Model zoo: Llama (training, tensor-parallel inference, generation), BERT, Whisper, Stable Diffusion, GCN, RL policies."""
from . import llama, llama_gen, bert, whisper, diffusion, graph, rl
from .llama import LlamaConfig, LlamaModel, LlamaForCausalLM, LlamaDecoderLayer
from .llama_gen import (CachedLlama, KvCache, LlamaKvCache, LayerKvCache, GenerationConfig, generate, generate_with_streamer, beam_search, SpecDecodeConfig,
                        SpecDecodeStats, SpecDecodeOutput, ModelHandle, LlamaHandle, speculative_generate, speculative_decode, XorShift64, apply_temperature,
                        apply_repetition_penalty, top_k_filter, top_p_filter, argmax, sample_softmax, sample_next, GptqQ4, AwqQ4, HqqWeights,
                        dequantize_gptq_q4, dequantize_awq_q4, dequantize_hqq, load_quantized_linear_weights, gguf_to_hf_name, gguf_key_to_hf,
                        remap_gguf_state_dict, gguf_to_hf_state_dict)
from .llama_blocks import LlamaActivation, LlamaMLP, LlamaAttention, LlamaGpuLayer, LlamaGpuInferencer, ProfiledForwardResult
from .. import grammar  # noqa: E402  (ferrotorch-llama re-exports the constrained-decoding package)
from .bert import (BertConfig, HfBertConfig, BertModel, BertEmbeddings, BertSelfAttention, BertSelfOutput, BertAttention, BertIntermediate, BertOutput,
                   BertLayer, BertEncoder, BertPooler, DropReport, SentenceTransformer, load_bert_model, load_sentence_transformer)
from .whisper import (WhisperConfig, HfWhisperConfig, WhisperEncoder, WhisperConvStem, WhisperEncoderLayer, WhisperEncoderSelfAttention,
                      log_mel_spectrogram, load_whisper_encoder, SAMPLE_RATE, N_MELS, N_FRAMES, N_FFT, HOP_LENGTH, CHUNK_LENGTH, N_SAMPLES, N_FREQS)
from .diffusion import (UNet2DConditionModel, UNetConfig, UNet2DConditionConfig, AutoencoderKL, VaeConfig, VaeDecoderConfig, VaeEncoderConfig, VaeEncoder,
                        VaeDecoder, Encoder, Decoder, DiagonalGaussianDistribution, ClipTextEncoder, ClipTextConfig, ClipTextEmbeddings,
                        ClipSelfAttention, ClipMlp, ClipEncoderLayer, ClipEncoder, DDIMScheduler, DDIMConfig, BetaSchedule, TimestepSpacing,
                        PredictionType, StableDiffusionPipeline, PipelineStepDump, Timesteps, TimestepEmbedding, Attention, FeedForward,
                        BasicTransformerBlock, Transformer2DModel, ResnetBlock2D, ResnetBlock2DTime, AttnBlock2D, Upsample2D, Downsample2D,
                        UpDecoderBlock2D, DownEncoderBlock2D, UNetMidBlock2D, UNetMidBlock2DCrossAttn, CrossAttnDownBlock2D, DownBlock2D,
                        CrossAttnUpBlock2D, UpBlock2D, AnyDownBlock, AnyUpBlock, load_unet, load_clip_text_encoder, load_vae_decoder,
                        load_vae_encoder, load_sd_component, GpuUNet2DConditional, GpuVaeDecoder, GpuVaeEncoder, GpuClipTextEncoder,
                        GpuStableDiffusionPipeline)
from .graph import Graph, GcnConv, GcnNet, load_gcn_net
from .rl import MlpPolicy, MlpPolicyConfig, MlpExtractor, ActionNet, ValueHead, PolicyOutput, load_ppo_policy, ppo_loss

__all__ = [n for n in dir() if not n.startswith("_")]
