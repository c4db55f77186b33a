"""Generation engines against a plain full-sequence forward (greedy), sampling filters, chunk allocator."""
import pytest
import torch

from megatron_lm_b200.config import TransformerConfig
from megatron_lm_b200.inference import (ChunkAllocator, DynamicInferenceEngine, SamplingParams, StaticInferenceEngine,
                                        sample_from_logits)
from megatron_lm_b200.models.gpt import GPTModel


def _model(device="cpu", dtype=torch.float32, hn=16, pos="rope"):
    torch.manual_seed(7)
    cfg = TransformerConfig(num_layers=2, hidden_size=4 * hn, num_attention_heads=4, num_query_groups=2,
                            ffn_hidden_size=8 * hn, normalization="RMSNorm", gated_linear_unit=True,
                            add_bias_linear=False, params_dtype=dtype,
                            bf16=dtype == torch.bfloat16, hidden_dropout=0.0, attention_dropout=0.0)
    m = GPTModel(cfg, vocab_size=128, max_sequence_length=64, parallel_output=False,
                 share_embeddings_and_output_weights=False, position_embedding_type=pos).to(device)
    return m.eval()


def _greedy_reference(model, prompt, n):
    toks = list(prompt)
    dev = next(model.parameters()).device
    with torch.no_grad():
        for _ in range(n):
            logits = model(torch.tensor([toks], device=dev))
            toks.append(int(logits[0, -1].float().argmax()))
    return toks[len(prompt):]


@pytest.mark.parametrize("pos", ["rope", "learned_absolute"])
def test_static_engine_matches_full_forward(pos):
    model = _model(pos=pos)
    prompts = [[5, 9, 2, 33, 7], [11, 4, 6]]
    eng = StaticInferenceEngine(model, max_batch_size=4, max_sequence_length=32)
    out = eng.generate(prompts, SamplingParams(top_k=1, num_tokens_to_generate=6, return_log_probs=True))
    for req, p in zip(out, prompts):
        ref = _greedy_reference(model, p, 6 + (5 - len(p)))
        assert req.generated_tokens[:len(ref)] == ref[:len(req.generated_tokens)]
        assert len(req.generated_log_probs) == len(req.generated_tokens)


def test_dynamic_engine_matches_full_forward_and_recycles_chunks():
    model = _model()
    prompts = [[5, 9, 2, 33, 7], [11, 4, 6], [1, 2, 3, 4, 5, 6, 7, 8, 9]]
    eng = DynamicInferenceEngine(model, max_requests=2, max_sequence_length=32, chunk_size=4, num_chunks=16)
    out = eng.generate(prompts, SamplingParams(top_k=1, num_tokens_to_generate=5))
    for req, p in zip(out, prompts):
        assert req.generated_tokens == _greedy_reference(model, p, 5)
    assert eng.context.alloc.available == 16 and len(eng.context.free_slots) == 2


def test_sampling_filters():
    g = torch.Generator().manual_seed(0)
    logits = torch.tensor([[0.0, 5.0, 4.0, -2.0, 1.0]]).repeat(200, 1)
    tk = sample_from_logits(logits, SamplingParams(top_k=2), generator=g)
    assert set(tk.tolist()) <= {1, 2}
    tp = sample_from_logits(logits, SamplingParams(top_p=0.7), generator=g)
    assert set(tp.tolist()) <= {1, 2}
    assert sample_from_logits(logits, SamplingParams(top_k=1)).tolist() == [1] * 200
    with pytest.raises(ValueError):
        sample_from_logits(logits, SamplingParams(top_k=9))


def test_chunk_allocator():
    a = ChunkAllocator(4)
    x = a.allocate(3)
    assert len(set(x)) == 3 and a.available == 1
    assert a.allocate(2) is None
    a.release(x)
    assert a.available == 4


@pytest.mark.gpu
def test_engines_gpu_decode_kernel():
    model = _model("cuda", torch.bfloat16, hn=64)
    prompts = [[5, 9, 2, 33, 7, 8, 1], [11, 4, 6]]
    # logits of the incremental path (prefill + decode kernel over the cache) against a full forward
    from megatron_lm_b200.inference import StaticInferenceContext
    ids = torch.tensor([prompts[0] + [3, 4, 5]], device="cuda")
    with torch.no_grad():
        full = model(ids).float()
        ctx = StaticInferenceContext(1, 32)
        a = model(ids[:, :7], inference_context=ctx).float(); ctx.advance()
        outs = [a]
        for i in range(7, 10):
            outs.append(model(ids[:, i:i + 1], inference_context=ctx).float()); ctx.advance()
    inc = torch.cat(outs, dim=1)
    assert torch.allclose(inc, full, atol=5e-2, rtol=5e-2), (inc - full).abs().max()
    st = StaticInferenceEngine(model, max_batch_size=4, max_sequence_length=48)
    dy = DynamicInferenceEngine(model, max_requests=4, max_sequence_length=48, chunk_size=16)
    sp = SamplingParams(top_k=1, num_tokens_to_generate=8)
    o_dy = dy.generate(prompts, sp)
    for req, p in zip(o_dy, prompts):
        # paged decode against full-forward logits, token by token (teacher-forced on the engine's tokens)
        seq = torch.tensor([p + req.generated_tokens], device="cuda")
        with torch.no_grad():
            lg = model(seq).float()[0]
        for i, t in enumerate(req.generated_tokens):
            row = lg[len(p) + i - 1]
            assert row[t] >= row.max() - 0.15
    assert len(st.generate(prompts, sp)) == 2


def test_dynamic_engine_streams_tokens_as_they_are_produced():
    model = _model()
    prompts = [[5, 9, 2, 33, 7], [11, 4, 6]]
    eng = DynamicInferenceEngine(model, max_requests=2, max_sequence_length=32, chunk_size=4, num_chunks=16)
    got = {0: [], 1: []}
    order, finished = [], set()
    for rid, tok, delta, fin in eng.stream(prompts, SamplingParams(top_k=1, num_tokens_to_generate=4)):
        got[rid].append(tok)
        order.append(rid)
        assert delta is None                      # no tokenizer attached
        if fin:
            finished.add(rid)
    for rid, p in enumerate(prompts):
        assert got[rid] == _greedy_reference(model, p, 4)
    assert finished == {0, 1}
    assert order[:4].count(0) == 2 and order[:4].count(1) == 2      # interleaved: both requests advance every step


def test_encoder_decoder_engine_matches_a_manual_greedy_loop():
    from megatron_lm_b200.inference import EncoderDecoderInferenceEngine
    from megatron_lm_b200.models.t5 import T5Model
    torch.manual_seed(3)
    cfg = TransformerConfig(num_layers=2, hidden_size=32, num_attention_heads=4, ffn_hidden_size=64, hidden_dropout=0.0,
                            attention_dropout=0.0)
    m = T5Model(cfg, vocab_size=64, max_sequence_length=16).eval()
    enc = [[3, 4, 5, 6, 7, 8]]
    out = EncoderDecoderInferenceEngine(m, bos_id=1, max_target_length=8).generate(
        enc, SamplingParams(top_k=1, num_tokens_to_generate=5))
    dec = [1]
    with torch.no_grad():
        for _ in range(5):
            logits = m(torch.tensor(enc), torch.tensor([dec]))
            dec.append(int(logits[0, -1].float().argmax()))
    assert out[0].generated_tokens == dec[1:]


def test_vlm_engine_generates_from_an_image_and_a_prompt():
    from megatron_lm_b200.inference import VLMInferenceEngine
    from megatron_lm_b200.models.multimodal import LLaVAModel
    torch.manual_seed(0)

    def cfg(h=32):
        return TransformerConfig(num_layers=1, hidden_size=h, num_attention_heads=4, ffn_hidden_size=2 * h,
                                 hidden_dropout=0.0, attention_dropout=0.0)
    m = LLaVAModel(cfg(), 64, 64, cfg(16), cfg(), img_h=8, img_w=8, patch_dim=4, drop_vision_class_token=True,
                   image_token_index=-200).eval()
    images = torch.randn(1, 3, 8, 8)
    eng = VLMInferenceEngine(m, max_batch_size=1, max_sequence_length=32)
    out = eng.generate_with_images([[5, -200, 7]], images, SamplingParams(top_k=1, num_tokens_to_generate=3))
    ids = [5, -200, 7]
    with torch.no_grad():
        for _ in range(3):
            logits = m(images, torch.tensor([ids]))
            ids.append(int(logits[0, -1].float().argmax()))
    assert out[0].generated_tokens == ids[3:]


def test_dynamic_engine_preempts_when_the_cache_runs_out_and_recomputes():
    """Three requests that together need twice the cache: the youngest is put back in the queue, recomputed later,
    and every request still produces the tokens of an unconstrained run."""
    model = _model()
    prompts = [[5, 9, 2, 33, 7, 1], [11, 4, 6, 8, 3, 2], [7, 7, 9, 1, 2, 3]]
    sp = SamplingParams(top_k=1, num_tokens_to_generate=10)
    roomy = DynamicInferenceEngine(model, max_requests=4, max_sequence_length=32, chunk_size=4)
    want = [r.generated_tokens for r in roomy.generate(prompts, sp)]
    assert roomy.preemptions == 0
    tight = DynamicInferenceEngine(model, max_requests=4, max_sequence_length=32, chunk_size=4, num_chunks=6)
    got = tight.generate(prompts, sp)
    assert tight.preemptions > 0
    assert [r.generated_tokens for r in got] == want
    assert tight.context.alloc.available == 6 and len(tight.context.free_slots) == 4


def test_dynamic_engine_admission_limits():
    model = _model()
    prompts = [[5, 9, 2, 33, 7, 1], [11, 4, 6, 8, 3, 2], [7, 7, 9, 1, 2, 3]]
    sp = SamplingParams(top_k=1, num_tokens_to_generate=3)
    # a token cap per step: the second prompt (6 tokens) does not fit beside the first within 8 tokens
    eng = DynamicInferenceEngine(model, max_requests=4, max_sequence_length=32, chunk_size=4, max_tokens_override=8)
    for p in prompts:
        eng.add_request(p, sp)
    eng.step()
    assert len(eng.scheduler.active) == 1 and len(eng.scheduler.waiting) == 2
    eng.step()                                          # 1 decode token + 6 prompt tokens = 7 <= 8
    assert len(eng.scheduler.active) == 2
    while eng.has_unfinished_requests():
        eng.step()
    ref = DynamicInferenceEngine(model, max_requests=4, max_sequence_length=32, chunk_size=4).generate(prompts, sp)
    assert [eng.scheduler.completed[i].generated_tokens for i in range(3)] == [r.generated_tokens for r in ref]
    # guaranteed fraction: with half of 8 chunks kept for running requests, a second request (2 chunks + reserve)
    # is admitted only while 4 chunks stay free
    eng = DynamicInferenceEngine(model, max_requests=4, max_sequence_length=32, chunk_size=4, num_chunks=8,
                                 buffer_guaranteed_fraction=0.5)
    for p in prompts:
        eng.add_request(p, sp)
    eng.step()
    assert len(eng.scheduler.active) == 2 and len(eng.scheduler.waiting) == 1      # 2 + 2 chunks used, 4 kept
    # slot count from the overflow factor: 16 chunks, 8 per request of maximal length, factor 2 -> 4 slots
    eng = DynamicInferenceEngine(model, max_requests=1, max_sequence_length=32, chunk_size=4, num_chunks=16,
                                 buffer_overflow_factor=2.0)
    assert eng.context.max_requests == 4 and eng.scheduler.max_batch_size == 4
    eng = DynamicInferenceEngine(model, max_requests=1, max_sequence_length=32, chunk_size=4, max_requests_override=3)
    assert eng.context.max_requests == 3


def test_top_n_log_probabilities_and_segments():
    model = _model()

    class Tok:
        eod = None
        def tokenize(self, s): return [int(x) for x in s.split()]
        def detokenize(self, ids): return " ".join(f"<{i}>" for i in ids)
    prompts = [[5, 9, 2, 33], [11, 4, 6, 8]]
    sp = SamplingParams(top_k=1, num_tokens_to_generate=3, return_log_probs=True, top_n_logprobs=4,
                        return_prompt_top_n_logprobs=True, return_segments=True)
    sp.add_attributes({"min_length": 2})
    assert sp.min_length == 2
    dyn = DynamicInferenceEngine(model, max_requests=4, max_sequence_length=32, chunk_size=4, tokenizer=Tok())
    for req, p in zip(dyn.generate(prompts, sp), prompts):
        assert len(req.generated_top_n_logprobs) == 3 and all(len(d) == 4 for d in req.generated_top_n_logprobs)
        # greedy decoding: the chosen token is the most likely one and its log probability matches
        for tok, lp, alts in zip(req.generated_tokens, req.generated_log_probs, req.generated_top_n_logprobs):
            best = max(alts, key=alts.get)
            assert best == tok and abs(alts[tok] - lp) < 1e-5
        assert len(req.prompt_top_n_logprobs) == len(p) - 1
        with torch.no_grad():
            full = torch.log_softmax(model(torch.tensor([p]))[0].float(), -1)
        for i, alts in enumerate(req.prompt_top_n_logprobs):
            want = full[i].topk(4)
            assert sorted(alts) == sorted(want.indices.tolist())
            assert abs(max(alts.values()) - float(want.values[0])) < 1e-4
        assert req.segments == [f"<{t}>" for t in p + req.generated_tokens]
    sp2 = SamplingParams(top_k=1, num_tokens_to_generate=3, top_n_logprobs=2, return_segments=True)
    st = StaticInferenceEngine(model, tokenizer=Tok(), max_batch_size=2, max_sequence_length=32).generate(prompts, sp2)
    assert all(len(r.generated_top_n_logprobs) == 3 and len(r.segments) == 7 for r in st)
    with pytest.raises(NotImplementedError):
        StaticInferenceEngine(model, max_batch_size=2, max_sequence_length=32).generate(prompts, sp)
