"""Text generation: KV-cache contexts, sampling, a static-batch engine and a dynamic
(continuous-batching) engine with a paged KV cache.

Counterparts in the reference (megatron/core/inference/): ``StaticInferenceContext`` and
``DynamicInferenceContext`` with its ``ChunkAllocator`` (contexts/dynamic_context.py:72,
dynamic_chunk_allocator.py:9), ``Scheduler`` (scheduler.py:17), ``TextGenerationController``
sampling (text_generation_controllers/text_generation_controller.py:168-310),
``StaticInferenceEngine`` (engines/static_engine.py:30) and ``DynamicInferenceEngine``
(engines/dynamic_engine.py:37: ``add_request`` :157, ``step`` :386).

The model's ``SelfAttention`` hands its fused, already rotated QKV activation to
``context.attend``; the context appends K/V to its cache and runs either the flash-attention
kernel (prefill, several query positions) or the single-query decode kernel over the cache.
"""
from __future__ import annotations

import math
from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional, Sequence, Tuple

import torch

from ..ops import _lib
from ..ops.attention import attention
from ..ops.sampling import sample as fused_sample

_lib.register_signatures({
    "mlb_attn_decode": "ippppppiiiiliifp",
    "mlb_kv_append": "ppppppplilii" "ip",
})


@dataclass
class SamplingParams:
    temperature: float = 1.0
    top_k: int = 0
    top_p: float = 0.0
    return_log_probs: bool = False
    return_segments: bool = False
    num_tokens_to_generate: int = 30
    top_n_logprobs: int = 0
    return_prompt_top_n_logprobs: bool = False

    def add_attributes(self, attribute_value_pair: dict) -> None:
        """Extra request-level attributes (e.g. ``{"min_length": 4}``) carried along with the standard ones."""
        for k, v in attribute_value_pair.items():
            setattr(self, k, v)


def top_n_log_probs(logits_row: torch.Tensor, n: int) -> Dict[int, float]:
    """{token id: log probability} of the ``n`` most likely next tokens."""
    lp = torch.log_softmax(logits_row.float(), dim=-1)
    vals, idx = lp.topk(min(n, lp.numel()))
    return {int(i): float(v) for i, v in zip(idx.tolist(), vals.tolist())}


def sample_from_logits(logits: torch.Tensor, params: SamplingParams, vocab_size: Optional[int] = None,
                       generator=None) -> torch.Tensor:
    """logits [b, v] -> token ids [b].  top_k == 1 is greedy; top-k and top-p (nucleus) filter before
    the temperature-scaled multinomial draw."""
    if params.top_k > logits.size(-1):
        raise ValueError("top-k is larger than the vocabulary")
    if params.top_p > 1.0:
        raise ValueError("top-p must be at most 1")
    if logits.is_cuda and logits.dtype in (torch.float32, torch.bfloat16, torch.float16):
        # one kernel: filter + inverse-CDF draw from uniforms of the caller's generator
        u = torch.rand(logits.shape[0], device=logits.device, generator=generator)
        out = fused_sample(logits, u, params.temperature, params.top_k, params.top_p)
    elif params.top_k == 1:
        out = torch.argmax(logits, dim=-1)
    else:
        x = logits.float().clone()
        if params.temperature != 1.0:
            x.div_(params.temperature)
        if params.top_k > 1:
            kth = torch.topk(x, params.top_k, dim=-1)[0][..., -1, None]
            x.masked_fill_(x < kth, float("-inf"))
        elif params.top_p > 0.0:
            srt, idx = torch.sort(x, descending=True, dim=-1)
            cum = srt.softmax(dim=-1).cumsum(dim=-1)
            remove = cum > params.top_p
            remove[..., 1:] = remove[..., :-1].clone()
            remove[..., 0] = False
            x.masked_fill_(remove.scatter(-1, idx, remove), float("-inf"))
        out = torch.multinomial(x.softmax(dim=-1), num_samples=1, generator=generator).view(-1)
    if vocab_size is not None:
        out = torch.clamp(out, min=0, max=vocab_size - 1)
    return out


# ----------------------------------------------------------------------------- contexts
class _ContextBase:
    def ssm_cache(self, layer_number, mixer, like):
        """Convolution window and state-space state of a Mamba mixer (pure and hybrid Mamba models decode through
        the same engines as attention models; reference: tools/run_mamba_text_generation_server.py)."""
        if not getattr(self, "supports_ssm", False):
            raise NotImplementedError("state-space layers decode with the static engine (one state per batch row); "
                                      "the paged dynamic context holds attention keys and values only")
        if not hasattr(self, "_ssm"):
            from ..models.mamba import MambaInferenceCache
            self._ssm = MambaInferenceCache()
        return self._ssm.ssm_cache(layer_number, mixer, like)

    def rope_span(self, input_ids) -> Tuple[int, int]:
        """(number of positions the rotary table must cover from ``offset``, offset) for this step."""
        raise NotImplementedError


class StaticInferenceContext(_ContextBase):
    """Contiguous KV cache [max_batch, max_len, ng, hn] per layer; all sequences advance together."""

    supports_ssm = True

    def __init__(self, max_batch_size: int, max_sequence_length: int):
        self.max_batch, self.max_len = max_batch_size, max_sequence_length
        self.k: Dict[int, torch.Tensor] = {}
        self.v: Dict[int, torch.Tensor] = {}
        self.offset = 0                 # tokens already cached
        self.step_len = 0

    def reset(self):
        self.offset = 0

    def rope_span(self, input_ids):
        self.step_len = input_ids.shape[1]
        return self.step_len, self.offset

    def advance(self):
        self.offset += self.step_len

    def attend(self, layer_number: int, qkv5: torch.Tensor, scale: float) -> torch.Tensor:
        s, b, ng, tot, d = qkv5.shape
        qpg = tot - 2
        if layer_number not in self.k:
            shape = (self.max_batch, self.max_len, ng, d)
            self.k[layer_number] = torch.zeros(shape, dtype=qkv5.dtype, device=qkv5.device)
            self.v[layer_number] = torch.zeros(shape, dtype=qkv5.dtype, device=qkv5.device)
        kc, vc = self.k[layer_number], self.v[layer_number]
        o0, o1 = self.offset, self.offset + s
        if o1 > self.max_len:
            raise RuntimeError("sequence exceeds the KV cache")
        kc[:b, o0:o1] = qkv5[:, :, :, qpg].transpose(0, 1)
        vc[:b, o0:o1] = qkv5[:, :, :, qpg + 1].transpose(0, 1)
        q = qkv5[:, :, :, :qpg]
        if s == 1 and qkv5.is_cuda:
            qd = q[0].contiguous()                                         # [b, ng, qpg, d]
            out = torch.empty_like(qd)
            lens = torch.full((b,), o1, dtype=torch.int32, device=qkv5.device)
            _lib.check(_lib.lib().mlb_attn_decode(_lib.dt(qd), qd.data_ptr(), kc.data_ptr(), vc.data_ptr(),
                                                  lens.data_ptr(), None, out.data_ptr(), b, ng, qpg, d, self.max_len,
                                                  0, 0, float(scale), _lib.stream()), "attn_decode")
            return out.view(1, b, ng * qpg * d)
        kk = kc[:b, :o1].transpose(0, 1)                                    # [sk, b, ng, d] views of the cache
        vv = vc[:b, :o1].transpose(0, 1)
        o = attention(q.contiguous() if not q.is_cuda else q, kk, vv, causal=True, scale=scale)
        return o.reshape(s, b, ng * qpg * d)


class ChunkAllocator:
    """Free-list of fixed-size KV chunks."""

    def __init__(self, num_chunks: int):
        self.total = num_chunks
        self.free: List[int] = list(range(num_chunks - 1, -1, -1))

    def allocate(self, n: int) -> Optional[List[int]]:
        if n > len(self.free):
            return None
        return [self.free.pop() for _ in range(n)]

    def release(self, chunks: Sequence[int]) -> None:
        self.free.extend(chunks)

    @property
    def available(self) -> int:
        return len(self.free)


class DynamicInferenceContext(_ContextBase):
    """Paged KV cache shared by requests of different lengths.  A step carries a flat list of tokens
    (``seq_of[i]``, ``pos_of[i]``): whole prompts of newly admitted requests and one token of each
    request that is decoding."""

    def __init__(self, max_requests: int, max_sequence_length: int, chunk_size: int = 256,
                 buffer_size_gb: Optional[float] = None, num_chunks: Optional[int] = None, num_layers: int = 1,
                 buffer_guaranteed_fraction: float = 0.0, max_tokens: Optional[int] = None):
        """``buffer_size_gb`` is the whole cache (keys and values of all ``num_layers`` layers).
        ``buffer_guaranteed_fraction`` of the chunks is kept out of reach of admissions, so that requests already
        running can keep growing; ``max_tokens`` caps the tokens of one step (prompts of new requests + one token per
        running request).  Reference: megatron/core/inference/contexts/dynamic_context.py:60-220."""
        self.max_requests, self.max_len, self.chunk = max_requests, max_sequence_length, chunk_size
        self.max_chunks = (max_sequence_length + chunk_size - 1) // chunk_size
        self.num_chunks = num_chunks
        self.buffer_gb = buffer_size_gb
        self.num_layers = max(int(num_layers), 1)
        self.guaranteed_fraction = float(buffer_guaranteed_fraction)
        self.max_tokens = max_tokens
        self.k: Dict[int, torch.Tensor] = {}
        self.v: Dict[int, torch.Tensor] = {}
        self.alloc: Optional[ChunkAllocator] = None
        self.block_table = None
        self.lens = [0] * max_requests                      # cached tokens per slot
        self.slot_chunks: Dict[int, List[int]] = {}
        self.free_slots = list(range(max_requests - 1, -1, -1))
        self.step_tokens: List[Tuple[int, int]] = []        # (slot, position) of each token of the step
        self.step_groups: List[Tuple[int, int, int]] = []   # (slot, first token index, count)
        self._step_no = 0
        self._reserved_step = -1

    def _ensure(self, layer, ng, d, dtype, device):
        if self.alloc is None:
            if self.num_chunks is None:
                if self.buffer_gb is not None:
                    per_chunk = 2 * self.chunk * ng * d * torch.empty((), dtype=dtype).element_size() * self.num_layers
                    self.num_chunks = max(int(self.buffer_gb * 2 ** 30 // max(per_chunk, 1)), self.max_chunks)
                else:
                    self.num_chunks = self.max_requests * self.max_chunks
            self.alloc = ChunkAllocator(self.num_chunks)
            self.block_table = torch.zeros(self.max_requests, self.max_chunks, dtype=torch.int32, device=device)
        if layer not in self.k:
            shape = (self.num_chunks, self.chunk, ng, d)
            self.k[layer] = torch.zeros(shape, dtype=dtype, device=device)
            self.v[layer] = torch.zeros(shape, dtype=dtype, device=device)

    # -- request bookkeeping (host) ------------------------------------------------
    def chunks_needed(self, slot_len: int, extra: int) -> int:
        have = (slot_len + self.chunk - 1) // self.chunk
        need = (slot_len + extra + self.chunk - 1) // self.chunk
        return need - have

    def total_chunks(self) -> int:
        return self.num_chunks or self.max_requests * self.max_chunks

    def free_chunks(self) -> int:
        return self.alloc.available if self.alloc is not None else self.total_chunks()

    def can_admit(self, prompt_len: int, reserve: int = 0, others_active: bool = False, committed: int = 0) -> bool:
        """Room for a new request?  ``committed`` chunks are already promised to other requests of the same step.
        While other requests run, an admission must leave the guaranteed part of the buffer free for their growth;
        a lone request may use everything."""
        if not self.free_slots:
            return False
        keep = int(self.guaranteed_fraction * self.total_chunks()) if others_active else 0
        return self.chunks_needed(0, prompt_len + reserve) + keep + committed <= self.free_chunks()

    def admit(self) -> int:
        slot = self.free_slots.pop()
        self.lens[slot] = 0
        self.slot_chunks[slot] = []
        return slot

    def release(self, slot: int) -> None:
        if self.alloc is not None:
            self.alloc.release(self.slot_chunks.get(slot, []))
        self.slot_chunks.pop(slot, None)
        self.lens[slot] = 0
        self.free_slots.append(slot)

    def begin_step(self, groups: List[Tuple[int, int]]):
        """groups: (slot, number of new tokens).  Returns position ids of the step's flat token list."""
        self.step_tokens, self.step_groups = [], []
        self._step_no += 1
        for slot, n in groups:
            self.step_groups.append((slot, len(self.step_tokens), n))
            for i in range(n):
                self.step_tokens.append((slot, self.lens[slot] + i))
        return [p for _, p in self.step_tokens]

    def _reserve_chunks(self):
        for slot, _, n in self.step_groups:
            need = self.chunks_needed(self.lens[slot], n)
            if need:
                got = self.alloc.allocate(need)
                if got is None:
                    raise RuntimeError("KV cache exhausted")
                base = len(self.slot_chunks[slot])
                self.slot_chunks[slot].extend(got)
                self.block_table[slot, base:base + need] = torch.tensor(got, dtype=torch.int32,
                                                                        device=self.block_table.device)

    def end_step(self):
        for slot, _, n in self.step_groups:
            self.lens[slot] += n

    def rope_span(self, input_ids):
        return self.max_len, 0          # positions differ per token: select_rope picks each token's row

    def select_rope(self, rotary, position_ids):
        cos, sin = rotary
        pos = position_ids.reshape(-1)
        return cos[pos].contiguous(), sin[pos].contiguous()

    # -- device side ------------------------------------------------------------------
    def attend(self, layer_number: int, qkv5: torch.Tensor, scale: float) -> torch.Tensor:
        n_tok, one, ng, tot, d = qkv5.shape                   # tokens along dim 0, "batch" of 1
        qpg = tot - 2
        dev = qkv5.device
        self._ensure(layer_number, ng, d, qkv5.dtype, dev)
        if self._reserved_step != self._step_no:            # first layer of this step: chunks and index vectors
            self._reserve_chunks()
            self._reserved_step = self._step_no
            self._seq_of = torch.tensor([s for s, _ in self.step_tokens], dtype=torch.int32, device=dev)
            self._pos_of = torch.tensor([p for _, p in self.step_tokens], dtype=torch.int32, device=dev)
        kc, vc = self.k[layer_number], self.v[layer_number]
        k_new = qkv5[:, 0, :, qpg]                             # [n_tok, ng, d] strided
        v_new = qkv5[:, 0, :, qpg + 1]
        if qkv5.is_cuda and qkv5.element_size() == 2 and qpg + 2 == tot and k_new.stride(1) == (qpg + 2) * d:
            kk, vv = k_new.contiguous(), v_new.contiguous()
            _lib.check(_lib.lib().mlb_kv_append(kk.data_ptr(), vv.data_ptr(), kc.data_ptr(), vc.data_ptr(),
                                                self._seq_of.data_ptr(), self._pos_of.data_ptr(),
                                                self.block_table.data_ptr(), ng * d, ng * d, 0, self.chunk,
                                                self.max_chunks, n_tok, _lib.stream()), "kv_append")
        else:
            for i, (slot, pos) in enumerate(self.step_tokens):
                c = self.slot_chunks[slot][pos // self.chunk]
                kc[c, pos % self.chunk] = k_new[i]
                vc[c, pos % self.chunk] = v_new[i]
        out = torch.empty(n_tok, ng, qpg, d, dtype=qkv5.dtype, device=dev)
        decode_rows, decode_slots = [], []
        for slot, start, n in self.step_groups:
            total = self.lens[slot] + n
            if n == 1 and qkv5.is_cuda:
                decode_rows.append(start)
                decode_slots.append(slot)
                continue
            # prefill (or CPU): gather this request's cache and run causal attention with sq <= sk
            chunks = self.slot_chunks[slot]
            kk = kc[chunks].reshape(-1, ng, d)[:total].unsqueeze(1)
            vv = vc[chunks].reshape(-1, ng, d)[:total].unsqueeze(1)
            q = qkv5[start:start + n, :, :, :qpg]
            o = attention(q.contiguous(), kk.contiguous(), vv.contiguous(), causal=True, scale=scale)
            out[start:start + n] = o.reshape(n, ng, qpg, d)
        if decode_rows:
            rows = torch.tensor(decode_rows, device=dev)
            qd = qkv5[rows, 0, :, :qpg].contiguous()
            od = torch.empty_like(qd)
            # the decode kernel indexes the block table by sequence number: give it the rows of these slots
            bt = self.block_table[torch.tensor(decode_slots, device=dev)].contiguous()
            lens = torch.tensor([self.lens[s] + 1 for s in decode_slots], dtype=torch.int32, device=dev)
            _lib.check(_lib.lib().mlb_attn_decode(_lib.dt(qd), qd.data_ptr(), kc.data_ptr(), vc.data_ptr(),
                                                  lens.data_ptr(), bt.data_ptr(), od.data_ptr(), len(decode_rows), ng,
                                                  qpg, d, 0, self.chunk, self.max_chunks, float(scale), _lib.stream()),
                       "attn_decode")
            out[rows] = od
        return out.view(n_tok, 1, ng * qpg * d)


# ----------------------------------------------------------------------------- requests / scheduler
@dataclass
class InferenceRequest:
    request_id: int
    prompt_tokens: List[int]
    sampling_params: SamplingParams
    generated_tokens: List[int] = field(default_factory=list)
    generated_log_probs: List[float] = field(default_factory=list)
    status: str = "waiting"            # waiting -> active -> completed
    slot: int = -1
    prompt: Optional[str] = None
    generated_text: Optional[str] = None
    segments: Optional[List[str]] = None                       # every token detokenised on its own (return_segments)
    generated_top_n_logprobs: List[Dict[int, float]] = field(default_factory=list)
    prompt_top_n_logprobs: List[Dict[int, float]] = field(default_factory=list)


class Scheduler:
    """Waiting / active / completed pools with a cap on concurrently active requests."""

    def __init__(self, max_batch_size: int):
        self.max_batch_size = max_batch_size
        self.waiting: Deque[InferenceRequest] = deque()
        self.active: Dict[int, InferenceRequest] = {}
        self.completed: Dict[int, InferenceRequest] = {}
        self._next_id = 0

    def add_request(self, prompt_tokens: List[int], params: SamplingParams, prompt: Optional[str] = None) -> int:
        rid = self._next_id
        self._next_id += 1
        self.waiting.append(InferenceRequest(rid, list(prompt_tokens), params, prompt=prompt))
        return rid

    def have_requests_pending(self) -> bool:
        return bool(self.waiting or self.active)

    def activate(self, req: InferenceRequest):
        req.status = "active"
        self.active[req.request_id] = req

    def complete(self, req: InferenceRequest):
        req.status = "completed"
        self.active.pop(req.request_id, None)
        self.completed[req.request_id] = req


# ----------------------------------------------------------------------------- engines
class StaticInferenceEngine:
    """Generates for a fixed batch: prompts are right-padded, decoding starts at the shortest prompt
    length, and positions still inside a longer prompt are forced to the prompt's token."""

    def __init__(self, model, tokenizer=None, max_batch_size: int = 8, max_sequence_length: int = 2048,
                 eod_id: Optional[int] = None, pad_id: int = 0):
        self.model, self.tokenizer = model, tokenizer
        self.max_batch, self.max_len = max_batch_size, max_sequence_length
        self.eod = eod_id if eod_id is not None else (tokenizer.eod if tokenizer is not None else None)
        self.pad = pad_id

    @torch.no_grad()
    def generate(self, prompts: Sequence, sampling_params: Optional[SamplingParams] = None, generator=None):
        sp = sampling_params or SamplingParams()
        toks = [self.tokenizer.tokenize(p) if isinstance(p, str) else list(p) for p in prompts]
        if len(toks) > self.max_batch:
            raise ValueError("more prompts than max_batch_size")
        dev = next(self.model.parameters()).device
        lens = [len(t) for t in toks]
        min_len, max_prompt = min(lens), max(lens)
        total = min(max_prompt + sp.num_tokens_to_generate, self.max_len)
        b = len(toks)
        ids = torch.full((b, total), self.pad, dtype=torch.long, device=dev)
        for i, t in enumerate(toks):
            ids[i, :len(t)] = torch.tensor(t, device=dev)
        lens_t = torch.tensor(lens, device=dev)
        ctx = StaticInferenceContext(b, total)
        was_training = self.model.training
        self.model.eval()
        done = torch.zeros(b, dtype=torch.bool, device=dev)
        log_probs = [[] for _ in range(b)]
        top_n = [[] for _ in range(b)]
        if sp.return_prompt_top_n_logprobs:
            raise NotImplementedError("top-n log probabilities of the prompt come from the dynamic engine "
                                      "(the static engine steps through ragged prompts token by token)")
        prev = 0
        for pos in range(min_len, total):
            logits = self.model(ids[:, prev:pos], inference_context=ctx)            # [b, pos-prev, v]
            ctx.advance()
            last = logits[:, -1].float()
            new = sample_from_logits(last, sp, None, generator)
            in_prompt = lens_t > pos
            new = torch.where(in_prompt, ids[:, pos], new)
            if self.eod is not None:
                new = torch.where(done, torch.full_like(new, self.eod), new)
            if sp.return_log_probs:
                lp = torch.log_softmax(last, dim=-1).gather(1, new[:, None]).squeeze(1)
                for i in range(b):
                    if not bool(in_prompt[i]) and not bool(done[i]):
                        log_probs[i].append(float(lp[i]))
            if sp.top_n_logprobs > 0:
                for i in range(b):
                    if not bool(in_prompt[i]) and not bool(done[i]):
                        top_n[i].append(top_n_log_probs(last[i], sp.top_n_logprobs))
            ids[:, pos] = new
            if self.eod is not None:
                done |= (new == self.eod) & ~in_prompt
                if bool(done.all()):
                    total = pos + 1
                    break
            prev = pos
        self.model.train(was_training)
        out = []
        for i in range(b):
            seq = ids[i, :total].tolist()
            gen = seq[lens[i]:]
            if self.eod is not None and self.eod in gen:
                gen = gen[:gen.index(self.eod) + 1]
            req = InferenceRequest(i, toks[i], sp, gen, log_probs[i], "completed")
            req.generated_top_n_logprobs = top_n[i][:len(gen)]
            if self.tokenizer is not None:
                req.generated_text = self.tokenizer.detokenize(gen)
                if sp.return_segments:
                    req.segments = [self.tokenizer.detokenize([t]) for t in toks[i] + gen]
            out.append(req)
        return out


class DynamicInferenceEngine:
    """Continuous batching: each ``step`` admits waiting requests while the paged cache has room,
    runs one forward over the new prompts' tokens plus one token per decoding request, samples, and
    retires finished requests (their chunks return to the allocator)."""

    def __init__(self, model, max_requests: int = 16, max_sequence_length: int = 2048, chunk_size: int = 256,
                 buffer_size_gb: Optional[float] = None, tokenizer=None, eod_id: Optional[int] = None,
                 num_chunks: Optional[int] = None, buffer_guaranteed_fraction: float = 0.0,
                 buffer_overflow_factor: Optional[float] = None, max_requests_override: Optional[int] = None,
                 max_tokens_override: Optional[int] = None):
        """``buffer_overflow_factor`` f sizes the request slots at f x (requests of maximal length that fit the
        buffer): more short requests than the worst case allows; ``max_requests_override`` / ``max_tokens_override``
        set the slot count and the per-step token cap outright.  When the cache runs out under running requests the
        youngest one is put back in the queue (its chunks are freed, its tokens so far become its prompt)."""
        self.model, self.tokenizer = model, tokenizer
        cfg = getattr(model, "config", None)
        layers = getattr(cfg, "num_layers", 1) or 1
        if buffer_overflow_factor is not None and (num_chunks is not None or buffer_size_gb is not None) and cfg is not None:
            chunks = num_chunks
            if chunks is None:
                ng = (cfg.num_query_groups or cfg.num_attention_heads) // max(getattr(cfg, "tensor_model_parallel_size", 1), 1)
                d = cfg.kv_channels or cfg.hidden_size // cfg.num_attention_heads
                elem = torch.empty((), dtype=cfg.params_dtype).element_size()
                chunks = int(buffer_size_gb * 2 ** 30 // max(2 * chunk_size * ng * d * elem * layers, 1))
            per_request = (max_sequence_length + chunk_size - 1) // chunk_size
            max_requests = max(1, int(buffer_overflow_factor * chunks / per_request))
        if max_requests_override is not None:
            max_requests = int(max_requests_override)
        self.context = DynamicInferenceContext(max_requests, max_sequence_length, chunk_size, buffer_size_gb, num_chunks,
                                               num_layers=layers, buffer_guaranteed_fraction=buffer_guaranteed_fraction,
                                               max_tokens=max_tokens_override)
        self.scheduler = Scheduler(max_requests)
        self.preemptions = 0
        self.eod = eod_id if eod_id is not None else (tokenizer.eod if tokenizer is not None else None)
        self.max_len = max_sequence_length

    def add_request(self, prompt, sampling_params: Optional[SamplingParams] = None) -> int:
        toks = self.tokenizer.tokenize(prompt) if isinstance(prompt, str) else list(prompt)
        if len(toks) >= self.max_len:
            raise ValueError("prompt longer than max_sequence_length")
        return self.scheduler.add_request(toks, sampling_params or SamplingParams(), prompt if isinstance(prompt, str) else None)

    def has_unfinished_requests(self) -> bool:
        return self.scheduler.have_requests_pending()

    @torch.no_grad()
    def step(self, generator=None) -> List[InferenceRequest]:
        sch, ctx = self.scheduler, self.context
        groups, feed, owners = [], [], []
        # running requests take one token each; when the cache cannot hold their growth, the youngest goes back
        # to the head of the queue and is recomputed later
        while len(sch.active) > 1 and \
                sum(ctx.chunks_needed(ctx.lens[r.slot], 1) for r in sch.active.values()) > ctx.free_chunks():
            self._preempt(max(sch.active.values(), key=lambda r: r.request_id))
        for req in sch.active.values():
            groups.append((req.slot, 1))
            feed.append([req.generated_tokens[-1]])
            owners.append(req)
        n_tokens = len(groups)
        committed = sum(ctx.chunks_needed(ctx.lens[r.slot], 1) for r in sch.active.values())
        while sch.waiting and len(sch.active) < sch.max_batch_size:
            nxt = sch.waiting[0]
            n_new = len(nxt.prompt_tokens) + len(nxt.generated_tokens)
            if ctx.max_tokens is not None and groups and n_tokens + n_new > ctx.max_tokens:
                break
            if not ctx.can_admit(n_new, 1, others_active=bool(sch.active), committed=committed):
                break
            committed += ctx.chunks_needed(0, n_new)
            req = sch.waiting.popleft()
            req.slot = ctx.admit()
            sch.activate(req)
            # a request that was put back carries tokens it already produced: they are part of what is recomputed
            toks = req.prompt_tokens + req.generated_tokens
            groups.append((req.slot, len(toks)))
            feed.append(toks)
            owners.append(req)
            n_tokens += len(toks)
        if not groups:
            return []
        dev = next(self.model.parameters()).device
        positions = ctx.begin_step(groups)
        ids = torch.tensor([t for f in feed for t in f], dtype=torch.long, device=dev).unsqueeze(0)     # [1, n_tok]
        pos = torch.tensor(positions, dtype=torch.long, device=dev).unsqueeze(0)
        was_training = self.model.training
        self.model.eval()
        logits = self.model(ids, position_ids=pos, inference_context=ctx)[0]                       # [n_tok, v]
        self.model.train(was_training)
        ctx.end_step()
        finished = []
        for (slot, start, n), req in zip(ctx.step_groups, owners):
            last = logits[start + n - 1].float().unsqueeze(0)
            tok = int(sample_from_logits(last, req.sampling_params, None, generator)[0])
            req.generated_tokens.append(tok)
            sp = req.sampling_params
            if sp.return_log_probs:
                req.generated_log_probs.append(float(torch.log_softmax(last, -1)[0, tok]))
            if sp.top_n_logprobs > 0:
                req.generated_top_n_logprobs.append(top_n_log_probs(last[0], sp.top_n_logprobs))
                if sp.return_prompt_top_n_logprobs and n > 1 and not req.prompt_top_n_logprobs:
                    # the prefill step: position i of the prompt predicts token i + 1
                    npr = len(req.prompt_tokens)
                    req.prompt_top_n_logprobs = [top_n_log_probs(logits[start + i], sp.top_n_logprobs)
                                                 for i in range(min(n, npr) - 1)]
            total = len(req.prompt_tokens) + len(req.generated_tokens)
            if (self.eod is not None and tok == self.eod) or total >= self.max_len or \
                    len(req.generated_tokens) >= req.sampling_params.num_tokens_to_generate:
                ctx.release(req.slot)
                sch.complete(req)
                if self.tokenizer is not None:
                    req.generated_text = self.tokenizer.detokenize(req.generated_tokens)
                    if req.sampling_params.return_segments:
                        req.segments = [self.tokenizer.detokenize([t]) for t in req.prompt_tokens + req.generated_tokens]
                finished.append(req)
        return finished

    def _preempt(self, req: InferenceRequest) -> None:
        self.context.release(req.slot)
        self.scheduler.active.pop(req.request_id, None)
        req.slot, req.status = -1, "waiting"
        self.scheduler.waiting.appendleft(req)
        self.preemptions += 1

    def generate(self, prompts: Sequence, sampling_params: Optional[SamplingParams] = None, generator=None):
        ids = [self.add_request(p, sampling_params) for p in prompts]
        while self.has_unfinished_requests():
            self.step(generator)
        return [self.scheduler.completed[i] for i in ids]

    def stream(self, prompts: Sequence, sampling_params: Optional[SamplingParams] = None, generator=None):
        """Generator form of :meth:`generate`: after every engine step yields, for each request that produced a
        token in that step, ``(request_id, token, text_delta, finished)`` - ``text_delta`` is the newly decoded
        text when the engine has a tokenizer (detokenised incrementally, so multi-token characters come out whole),
        else None (reference: text_generation_controller.py:1032 ``stream_tokens``)."""
        ids = [self.add_request(p, sampling_params) for p in prompts]
        mine = set(ids)
        seen = {i: 0 for i in ids}
        text = {i: "" for i in ids}
        while any(i in self.scheduler.active or any(r.request_id == i for r in self.scheduler.waiting) for i in mine):
            finished = {r.request_id for r in self.step(generator)}
            for i in ids:
                req = self.scheduler.active.get(i) or self.scheduler.completed.get(i)
                if req is None:
                    continue
                while seen[i] < len(req.generated_tokens):
                    tok = req.generated_tokens[seen[i]]
                    seen[i] += 1
                    delta = None
                    if self.tokenizer is not None:
                        full = self.tokenizer.detokenize(req.generated_tokens[:seen[i]])
                        delta, text[i] = full[len(text[i]):], full
                    yield i, tok, delta, (i in finished and seen[i] == len(req.generated_tokens))


class EncoderDecoderInferenceEngine:
    """Greedy / sampled decoding for encoder-decoder models (T5): the encoder runs once per batch, the decoder is
    re-run on the growing target prefix (no KV cache: targets are short next to the encoder input).
    ``model(encoder_ids, decoder_ids, ...)`` must return logits [b, t, v]
    (reference: inference/model_inference_wrappers/t5/t5_inference_wrapper.py)."""

    def __init__(self, model, bos_id: int, eod_id: Optional[int] = None, pad_id: int = 0, max_target_length: int = 128):
        self.model, self.bos, self.eod, self.pad, self.max_t = model, bos_id, eod_id, pad_id, max_target_length

    @torch.no_grad()
    def generate(self, encoder_inputs: Sequence[Sequence[int]], sampling_params: Optional[SamplingParams] = None,
                 generator=None):
        sp = sampling_params or SamplingParams()
        dev = next(self.model.parameters()).device
        b = len(encoder_inputs)
        L = max(len(x) for x in encoder_inputs)
        enc = torch.full((b, L), self.pad, dtype=torch.long, device=dev)
        for i, x in enumerate(encoder_inputs):
            enc[i, :len(x)] = torch.tensor(list(x), device=dev)
        enc_mask = enc != self.pad
        dec = torch.full((b, 1), self.bos, dtype=torch.long, device=dev)
        done = torch.zeros(b, dtype=torch.bool, device=dev)
        was_training = self.model.training
        self.model.eval()
        steps = min(sp.num_tokens_to_generate, self.max_t)
        for _ in range(steps):
            if bool((~enc_mask).any()) and _accepts(self.model, "encoder_attn_mask"):
                logits = self.model(enc, dec, encoder_attn_mask=enc_mask)      # padded batch: mask the padding
            else:
                logits = self.model(enc, dec)
            new = sample_from_logits(logits[:, -1].float(), sp, None, generator)
            if self.eod is not None:
                new = torch.where(done, torch.full_like(new, self.eod), new)
                done |= new == self.eod
            dec = torch.cat((dec, new[:, None]), dim=1)
            if self.eod is not None and bool(done.all()):
                break
        self.model.train(was_training)
        out = []
        for i in range(b):
            gen = dec[i, 1:].tolist()
            if self.eod is not None and self.eod in gen:
                gen = gen[:gen.index(self.eod) + 1]
            out.append(InferenceRequest(i, list(encoder_inputs[i]), sp, gen, [], "completed"))
        return out


def _accepts(model, name: str) -> bool:
    import inspect
    try:
        return name in inspect.signature(model.forward).parameters
    except (TypeError, ValueError):
        return False


class VLMInferenceEngine(StaticInferenceEngine):
    """Text generation conditioned on images for LLaVA-style models: the first forward carries the image tensor
    (the model splices the projected image embeddings into the prompt and fills the KV cache), later steps are
    text-only (reference: inference/model_inference_wrappers/multimodal/vlm_inference_wrapper.py)."""

    @torch.no_grad()
    def generate_with_images(self, prompts: Sequence, images: torch.Tensor,
                             sampling_params: Optional[SamplingParams] = None, generator=None):
        sp = sampling_params or SamplingParams()
        toks = [self.tokenizer.tokenize(p) if isinstance(p, str) else list(p) for p in prompts]
        if len({len(t) for t in toks}) != 1:
            raise ValueError("image-conditioned generation takes prompts of one length (pad them first)")
        dev = next(self.model.parameters()).device
        ids = torch.tensor(toks, dtype=torch.long, device=dev)
        was_training = self.model.training
        self.model.eval()
        gen = []
        done = torch.zeros(len(toks), dtype=torch.bool, device=dev)
        for step in range(sp.num_tokens_to_generate):
            # no cache across the image splice: the sequence is short and the model decides where the image goes
            logits = self.model(images, ids)
            new = sample_from_logits(logits[:, -1].float(), sp, None, generator)
            if self.eod is not None:
                new = torch.where(done, torch.full_like(new, self.eod), new)
                done |= new == self.eod
            gen.append(new)
            ids = torch.cat((ids, new[:, None]), dim=1)
            if self.eod is not None and bool(done.all()):
                break
        self.model.train(was_training)
        g = torch.stack(gen, dim=1).tolist() if gen else [[] for _ in toks]
        out = []
        for i, t in enumerate(toks):
            seq = g[i]
            if self.eod is not None and self.eod in seq:
                seq = seq[:seq.index(self.eod) + 1]
            req = InferenceRequest(i, t, sp, seq, [], "completed")
            if self.tokenizer is not None:
                req.generated_text = self.tokenizer.detokenize(seq)
            out.append(req)
        return out
