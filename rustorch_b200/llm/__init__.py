"""LLM runtime: GGUF Llama inference with KV cache, quantised linears, sampling, metrics, CLI."""
from .convert import hf_to_gguf, interleave_rope_rows
from .llama import KVCache, LlamaConfig, LlamaRuntime
from .metrics import InferenceMetrics, InferenceTimer, MetricsCollector, MetricsReporter, PerformanceTargets
from .quant import QuantLinear
from .sampling import (Sampler, SamplingConfig, apply_repetition_penalty, apply_top_k_to_probs, apply_top_p_to_probs,
                       multinomial_sample, sample_token, softmax)
