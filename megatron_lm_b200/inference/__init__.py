"""Text generation engines, KV-cache contexts and sampling."""
from .engine import (ChunkAllocator, DynamicInferenceContext, DynamicInferenceEngine, EncoderDecoderInferenceEngine,
                     InferenceRequest, SamplingParams, Scheduler, StaticInferenceContext, StaticInferenceEngine,
                     VLMInferenceEngine, sample_from_logits)

__all__ = ["ChunkAllocator", "DynamicInferenceContext", "DynamicInferenceEngine", "EncoderDecoderInferenceEngine",
           "InferenceRequest", "SamplingParams", "Scheduler", "StaticInferenceContext", "StaticInferenceEngine",
           "VLMInferenceEngine", "sample_from_logits"]
