#!/usr/bin/env python
"""Generate with the static and the dynamic (paged KV cache, continuous batching) engines from a random-init
or converted model.  ``python examples/inference/generate.py --prompt-len 16 --new-tokens 32 --requests 8``"""
import argparse
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from megatron_lm_b200.config import TransformerConfig  # noqa: E402
from megatron_lm_b200.inference import DynamicInferenceEngine, SamplingParams, StaticInferenceEngine  # noqa: E402
from megatron_lm_b200.models.gpt import GPTModel  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=4); ap.add_argument("--hidden", type=int, default=1024)
    ap.add_argument("--heads", type=int, default=8); ap.add_argument("--vocab", type=int, default=32000)
    ap.add_argument("--prompt-len", type=int, default=16); ap.add_argument("--new-tokens", type=int, default=32)
    ap.add_argument("--requests", type=int, default=8); ap.add_argument("--core-checkpoint", default=None)
    a = ap.parse_args()
    cuda = torch.cuda.is_available()
    dt = torch.bfloat16 if cuda else torch.float32
    cfg = TransformerConfig(num_layers=a.layers, hidden_size=a.hidden, num_attention_heads=a.heads,
                            ffn_hidden_size=4 * a.hidden, normalization="RMSNorm", gated_linear_unit=True,
                            add_bias_linear=False, params_dtype=dt, bf16=cuda, use_cpu_initialization=not cuda,
                            hidden_dropout=0.0, attention_dropout=0.0)
    model = GPTModel(cfg, a.vocab, 4096, position_embedding_type="rope", parallel_output=False)
    if a.core_checkpoint:
        from megatron_lm_b200.checkpoint.convert import load_core
        model.load_state_dict(load_core(a.core_checkpoint), strict=False)
    if cuda:
        model = model.cuda()
    prompts = [torch.randint(1, a.vocab, (a.prompt_len + i,)).tolist() for i in range(a.requests)]
    sp = SamplingParams(top_k=1, num_tokens_to_generate=a.new_tokens)
    for name, eng in (("static", StaticInferenceEngine(model, max_batch_size=a.requests, max_sequence_length=2048)),
                      ("dynamic", DynamicInferenceEngine(model, max_requests=a.requests, max_sequence_length=2048))):
        t0 = time.time()
        out = eng.generate(prompts, sp)
        if cuda:
            torch.cuda.synchronize()
        n = sum(len(o.generated_tokens) for o in out)
        print(f"{name}: {n} tokens in {time.time() - t0:.2f} s; first request -> {out[0].generated_tokens[:8]}")


if __name__ == "__main__":
    main()
