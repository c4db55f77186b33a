"""Text generation engines, KV-cache contexts and sampling."""
from .engine import (ChunkAllocator, DynamicInferenceContext, DynamicInferenceEngine, InferenceRequest, SamplingParams,
                     Scheduler, StaticInferenceContext, StaticInferenceEngine, sample_from_logits)

__all__ = ["ChunkAllocator", "DynamicInferenceContext", "DynamicInferenceEngine", "InferenceRequest", "SamplingParams",
           "Scheduler", "StaticInferenceContext", "StaticInferenceEngine", "sample_from_logits"]
