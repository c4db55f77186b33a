"""HTTP text-generation server and its request handling.

``python -m megatron_lm_b200.inference.server --port 5000 ...`` after building a model, or embed
``MegatronServer(engine).run(host, port)``.

Reference: megatron/inference/text_generation_server.py (``MegatronGenerate.put`` :35, request validation
:40-200, ``MegatronServer`` :208) and text_generation/api.py:90 (``generate_and_post_process``), beam search
text_generation/generation.py:334.  The wire format is kept: ``PUT /api`` with JSON
{"prompts": [...], "tokens_to_generate": n, "temperature", "top_k", "top_p", "logprobs", "add_BOS",
 "random_seed", "beam_width", "length_penalty", "stop_token"} -> {"text": [...], "segments", "logprobs"}.
Implemented on the standard library's http.server (no web framework needed).
"""
from __future__ import annotations

import json
import threading
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from typing import List, Optional

import torch

from .engine import SamplingParams, StaticInferenceContext


def validate_request(req: dict, max_batch: int = 128):
    """Returns (error message or None, normalised request)."""
    if "prompts" not in req:
        return "prompts argument required", None
    prompts = req["prompts"]
    if not isinstance(prompts, list) or not prompts or not all(isinstance(p, str) for p in prompts):
        return "prompts is not a list of strings", None
    if len(prompts) > max_batch:
        return f"Maximum number of prompts is {max_batch}", None
    out = {"prompts": prompts}
    n = req.get("tokens_to_generate", 64)
    if not isinstance(n, int) or n < 0:
        return "tokens_to_generate must be an integer greater than or equal to 0", None
    out["tokens_to_generate"] = n
    lp = req.get("logprobs", False)
    if not isinstance(lp, bool):
        return "logprobs must be a boolean value", None
    if n == 0 and not lp:
        return "tokens_to_generate=0 implies logprobs should be True", None
    out["logprobs"] = lp
    t = req.get("temperature", 1.0)
    if not isinstance(t, (int, float)) or not 0.0 < t <= 100.0:
        return "temperature must be a positive number less than or equal to 100.0", None
    out["temperature"] = float(t)
    k = req.get("top_k", 0)
    if not isinstance(k, int) or not 0 <= k <= 1000:
        return "top_k must be an integer equal to or greater than 0 and less than or equal to 1000", None
    p = req.get("top_p", 0.0)
    if not isinstance(p, (int, float)) or not 0.0 <= p <= 1.0:
        return "top_p must be less than or equal to 1.0", None
    if k > 0 and p > 0.0:
        return "cannot set both top-k and top-p samplings.", None
    out["top_k"], out["top_p"] = k, float(p)
    for flag in ("add_BOS", "stop_on_double_eol", "stop_on_eol", "no_log"):
        v = req.get(flag, False)
        if not isinstance(v, bool):
            return f"{flag} must be a boolean value", None
        out[flag] = v
    seed = req.get("random_seed", -1)
    if not isinstance(seed, int) or seed < -1:
        return "random_seed must be a non-negative integer", None
    out["random_seed"] = seed
    bw = req.get("beam_width")
    if bw is not None:
        if not isinstance(bw, int) or bw < 1:
            return "beam_width must be an integer > 1", None
        if len(prompts) > 1:
            return "When doing beam_search, batch size must be 1", None
    out["beam_width"] = bw
    out["stop_token"] = req.get("stop_token", None)
    out["length_penalty"] = float(req.get("length_penalty", 1.0))
    return None, out


@torch.no_grad()
def beam_search(model, prompt: List[int], beam_width: int, tokens_to_generate: int, stop_token: int,
                length_penalty: float = 1.0, max_len: int = 2048):
    """Length-penalised beam search for one prompt; returns (token lists, scores) best first."""
    dev = next(model.parameters()).device
    beams = [(list(prompt), 0.0)]
    done = []
    for _ in range(tokens_to_generate):
        ids = torch.tensor([b[0] for b in beams], device=dev)
        logits = model(ids)[:, -1].float()
        lp = torch.log_softmax(logits, dim=-1)
        cand = []
        for bi, (toks, score) in enumerate(beams):
            top = torch.topk(lp[bi], beam_width)
            for v, t in zip(top.values.tolist(), top.indices.tolist()):
                cand.append((toks + [t], score + v))
        cand.sort(key=lambda c: c[1], reverse=True)
        beams = []
        for toks, score in cand:
            if toks[-1] == stop_token:
                done.append((toks, score / (len(toks) - len(prompt)) ** length_penalty))
            else:
                beams.append((toks, score))
            if len(beams) == beam_width:
                break
        if len(done) >= beam_width or not beams or len(beams[0][0]) >= max_len:
            break
    done.extend((t, s / max(len(t) - len(prompt), 1) ** length_penalty) for t, s in beams)
    done.sort(key=lambda c: c[1], reverse=True)
    done = done[:beam_width]
    return [d[0] for d in done], [d[1] for d in done]


def generate_and_post_process(engine, req: dict):
    """Run a validated request through a generation engine; returns the response dict."""
    tok = engine.tokenizer
    prompts = req["prompts"]
    if req.get("beam_width"):
        ids = tok.tokenize(prompts[0])
        stop = req["stop_token"] if req.get("stop_token") is not None else tok.eod
        seqs, scores = beam_search(engine.model, ids, req["beam_width"], req["tokens_to_generate"], stop,
                                   req["length_penalty"])
        return {"text": [tok.detokenize(s) for s in seqs], "segments": [[tok.detokenize([t]) for t in s] for s in seqs],
                "scores": scores}
    gen = None
    if req.get("random_seed", -1) >= 0:
        dev = next(engine.model.parameters()).device
        gen = torch.Generator(device=dev).manual_seed(req["random_seed"])
    sp = SamplingParams(temperature=req["temperature"], top_k=req["top_k"] or (0 if req["top_p"] > 0 else 1),
                        top_p=req["top_p"], return_log_probs=req["logprobs"],
                        num_tokens_to_generate=req["tokens_to_generate"])
    toks = []
    for p in prompts:
        t = tok.tokenize(p)
        if req.get("add_BOS") and getattr(tok, "bos", None) is not None:
            t = [tok.bos] + t
        toks.append(t)
    outs = engine.generate(toks, sp, generator=gen)
    text = [p + tok.detokenize(o.generated_tokens) for p, o in zip(prompts, outs)]
    resp = {"text": text, "segments": [[tok.detokenize([t]) for t in (tk + o.generated_tokens)] for tk, o in zip(toks, outs)]}
    if req["logprobs"]:
        resp["logprobs"] = [o.generated_log_probs for o in outs]
    return resp


class MegatronServer:
    def __init__(self, engine, max_batch: int = 128, max_tokens_to_oom: Optional[int] = None):
        """``max_tokens_to_oom``: a request whose batch x (longest prompt + tokens to generate) exceeds it is refused
        instead of being allowed to exhaust memory (reference: text_generation/generation.py --max-tokens-to-oom)."""
        self.engine, self.max_batch, self.max_tokens_to_oom = engine, max_batch, max_tokens_to_oom
        self.lock = threading.Lock()

    def handle(self, body: bytes):
        try:
            req = json.loads(body)
        except json.JSONDecodeError:
            return 400, {"message": "request body is not JSON"}
        err, norm = validate_request(req, self.max_batch)
        if err:
            return 400, {"message": err}
        if self.max_tokens_to_oom is not None:
            tok = getattr(self.engine, "tokenizer", None)
            longest = max(len(tok.tokenize(p)) if tok is not None else len(p.split()) for p in norm["prompts"])
            total = len(norm["prompts"]) * (longest + norm["tokens_to_generate"])
            if total > self.max_tokens_to_oom:
                return 400, {"message": f"Too many tokens.  {total} is greater than {self.max_tokens_to_oom}"}
        with self.lock:                       # one generation at a time, like the reference
            try:
                return 200, generate_and_post_process(self.engine, norm)
            except ValueError as e:
                return 400, {"message": str(e)}

    def handle_completions(self, body: bytes):
        """``POST /completions``: the completions request of OpenAI-style clients - ``prompt`` (text, list of texts,
        token ids or list of token-id lists), ``max_tokens``, ``temperature`` (0 = greedy), ``top_k``, ``top_p``,
        ``logprobs`` (number of alternatives per token, at most 10), ``echo``, ``seed``, ``stop``; one choice per
        prompt with text, token strings, their log probabilities, text offsets and the finish reason
        (reference: megatron/inference/endpoints/completions.py:39-230)."""
        try:
            req = json.loads(body)
        except json.JSONDecodeError:
            return 400, {"message": "request body is not JSON"}
        tok = self.engine.tokenizer
        if "prompt" not in req or "max_tokens" not in req:
            return 400, {"message": "prompt and max_tokens are required"}
        p = req["prompt"]
        if isinstance(p, str):
            prompts = [tok.tokenize(p)]
        elif isinstance(p, list) and p and all(isinstance(x, int) for x in p):
            prompts = [list(p)]
        elif isinstance(p, list) and p and all(isinstance(x, str) for x in p):
            prompts = [tok.tokenize(x) for x in p]
        elif isinstance(p, list) and p and all(isinstance(x, list) and all(isinstance(t, int) for t in x) for x in p):
            prompts = [list(x) for x in p]
        else:
            return 400, {"message": "prompt must be a string, a list of strings, token ids or lists of token ids"}
        n_gen, top_n = int(req["max_tokens"]), int(req.get("logprobs", 0) or 0)
        echo = bool(req.get("echo", False))
        if int(req.get("best_of", 1)) > 1:
            return 400, {"message": "best_of > 1 not supported"}
        if int(req.get("n", 1)) > 1:
            return 400, {"message": "num_completions > 1 not supported"}
        if not echo and n_gen == 0:
            return 400, {"message": "echo=False not supported when tokens_to_generate == 0"}
        if top_n > 10:
            return 400, {"message": "return_topk_logprobs > 10 not supported"}
        if len(prompts) > self.max_batch:
            return 400, {"message": f"Maximum number of prompts is {self.max_batch}"}
        temperature = float(req.get("temperature", 1.0))
        top_k, top_p = int(req.get("top_k", 0)), float(req.get("top_p", 1.0))
        if temperature == 0:
            temperature, top_k, top_p = 1.0, 1, 0.0
        if top_p >= 1.0:
            top_p = 0.0
        if top_k == 0 and top_p == 0.0 and float(req.get("temperature", 1.0)) == 0:
            top_k = 1
        stop = req.get("stop", None)
        stop = [stop] if isinstance(stop, str) else list(stop or [])
        sp = SamplingParams(temperature=temperature, top_k=top_k, top_p=top_p, return_log_probs=True,
                            num_tokens_to_generate=max(n_gen, 1), top_n_logprobs=top_n)
        gen = None
        if int(req.get("seed", -1)) >= 0:
            dev = next(self.engine.model.parameters()).device
            gen = torch.Generator(device=dev).manual_seed(int(req["seed"]))
        with self.lock:
            try:
                outs = self.engine.generate(prompts, sp, generator=gen)
            except ValueError as e:
                return 400, {"message": str(e)}
        choices = []
        for i, (ids, o) in enumerate(zip(prompts, outs)):
            new = o.generated_tokens[:n_gen]
            lps = list(o.generated_log_probs[:n_gen])
            alts = list(o.generated_top_n_logprobs[:n_gen]) if top_n else []
            reason = "length"
            if getattr(tok, "eod", None) is not None and tok.eod in new:
                cut = new.index(tok.eod)
                new, lps, alts, reason = new[:cut], lps[:cut], alts[:cut], "stop"
            pieces = [tok.detokenize([t]) for t in new]
            text = tok.detokenize(new) if new else ""
            for word in stop:
                at = text.find(word) if word else -1
                if at >= 0:
                    text, reason = text[:at], "stop"
                    keep, total = 0, 0
                    for piece in pieces:                      # tokens that lie wholly before the stop string
                        if total + len(piece) > at:
                            break
                        total += len(piece)
                        keep += 1
                    new, lps, alts, pieces = new[:keep], lps[:keep], alts[:keep], pieces[:keep]
            shown_tokens = ([tok.detokenize([t]) for t in ids] if echo else []) + pieces
            shown_lps = ([None] * len(ids) if echo else []) + lps
            offsets, pos = [], 0
            for piece in shown_tokens:
                offsets.append(pos)
                pos += len(piece)
            logprobs = {"token_logprobs": shown_lps, "tokens": shown_tokens, "text_offset": offsets,
                        "top_logprobs": ([None] * len(ids) if echo else []) +
                        [{tok.detokenize([k]): v for k, v in a.items()} for a in alts] if top_n else None}
            choices.append({"index": i, "text": (tok.detokenize(ids) if echo else "") + text, "logprobs": logprobs,
                            "finish_reason": reason})
        return 200, {"choices": choices}

    def run(self, host: str = "0.0.0.0", port: int = 5000):
        server = self

        class Handler(BaseHTTPRequestHandler):
            def do_PUT(self):
                route = self.path.rstrip("/")
                if route not in ("/api", "/completions", "/v1/completions"):
                    self.send_error(404)
                    return
                n = int(self.headers.get("Content-Length", 0))
                body = self.rfile.read(n)
                code, payload = server.handle(body) if route == "/api" else server.handle_completions(body)
                data = json.dumps(payload).encode()
                self.send_response(code)
                self.send_header("Content-Type", "application/json")
                self.send_header("Content-Length", str(len(data)))
                self.end_headers()
                self.wfile.write(data)
            do_POST = do_PUT

            def log_message(self, *a):
                pass
        self.httpd = ThreadingHTTPServer((host, port), Handler)
        self.httpd.serve_forever()
