"""Throughput / latency test of the generation engines:
``python -m megatron_lm_b200.inference.perf_test --engine dynamic --num-requests 32 --prompt-length 128 --num-tokens-to-generate 64``
(reference: tools/run_inference_performance_test.py).  Builds a random-init GPT of the given shape (or loads a core
checkpoint), generates for synthetic prompts and prints requests/s, generated tokens/s and time to first token."""
from __future__ import annotations

import argparse
import json
import time

import torch


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--engine", choices=["static", "dynamic"], default="dynamic")
    ap.add_argument("--num-layers", type=int, default=4)
    ap.add_argument("--hidden-size", type=int, default=1024)
    ap.add_argument("--num-attention-heads", type=int, default=8)
    ap.add_argument("--num-query-groups", type=int, default=None)
    ap.add_argument("--ffn-hidden-size", type=int, default=None)
    ap.add_argument("--vocab-size", type=int, default=32000)
    ap.add_argument("--num-requests", type=int, default=16)
    ap.add_argument("--prompt-length", type=int, default=128)
    ap.add_argument("--num-tokens-to-generate", type=int, default=64)
    ap.add_argument("--max-sequence-length", type=int, default=2048)
    ap.add_argument("--chunk-size", type=int, default=256)
    ap.add_argument("--load", default=None, help="directory of a core checkpoint")
    a = ap.parse_args(argv)
    from ..config import TransformerConfig
    from ..models.gpt import GPTModel
    from .engine import DynamicInferenceEngine, SamplingParams, StaticInferenceEngine
    cuda = torch.cuda.is_available()
    dt = torch.bfloat16 if cuda else torch.float32
    cfg = TransformerConfig(num_layers=a.num_layers, hidden_size=a.hidden_size, num_attention_heads=a.num_attention_heads,
                            num_query_groups=a.num_query_groups, ffn_hidden_size=a.ffn_hidden_size or 4 * a.hidden_size,
                            normalization="RMSNorm", gated_linear_unit=True, add_bias_linear=False, params_dtype=dt,
                            bf16=cuda, use_cpu_initialization=not cuda, hidden_dropout=0.0, attention_dropout=0.0)
    model = GPTModel(cfg, a.vocab_size, a.max_sequence_length, position_embedding_type="rope", parallel_output=False)
    if a.load:
        from ..checkpoint.convert import load_core
        model.load_state_dict(load_core(a.load), strict=False)
    if cuda:
        model = model.cuda()
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(1, a.vocab_size, (a.prompt_length,), generator=g).tolist() for _ in range(a.num_requests)]
    sp = SamplingParams(top_k=1, num_tokens_to_generate=a.num_tokens_to_generate)
    if a.engine == "static":
        eng = StaticInferenceEngine(model, max_batch_size=a.num_requests, max_sequence_length=a.max_sequence_length)
    else:
        eng = DynamicInferenceEngine(model, max_requests=a.num_requests, max_sequence_length=a.max_sequence_length,
                                     chunk_size=a.chunk_size)
    sync = torch.cuda.synchronize if cuda else (lambda: None)
    eng.generate(prompts[:2], SamplingParams(top_k=1, num_tokens_to_generate=4))       # warm-up
    sync()
    t0 = time.perf_counter()
    ttft = None
    if a.engine == "dynamic":
        ids = [eng.add_request(p, sp) for p in prompts]
        while eng.has_unfinished_requests():
            eng.step()
            if ttft is None:
                sync()
                ttft = time.perf_counter() - t0
        outs = [eng.scheduler.completed[i] for i in ids]
    else:
        outs = eng.generate(prompts, sp)
    sync()
    dt_s = time.perf_counter() - t0
    n = sum(len(o.generated_tokens) for o in outs)
    print(json.dumps({"engine": a.engine, "requests": len(outs), "generated_tokens": n, "seconds": dt_s,
                      "requests_per_s": len(outs) / dt_s, "tokens_per_s": n / dt_s,
                      "time_to_first_token_s": ttft}))


if __name__ == "__main__":
    main()
