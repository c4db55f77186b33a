"""Request validation, beam search and the request -> response path of the generation server."""
import json

import torch

from megatron_lm_b200.inference import StaticInferenceEngine
from megatron_lm_b200.inference.server import MegatronServer, beam_search, validate_request
from tests.test_inference import _model


class _Tok:
    eod, bos = 0, 1
    def tokenize(self, s): return [int(x) for x in s.split()]
    def detokenize(self, ids): return " " + " ".join(str(i) for i in ids) if ids else ""


def test_validation_messages():
    assert validate_request({})[0] == "prompts argument required"
    assert validate_request({"prompts": ["a"], "top_k": 3, "top_p": 0.5})[0].startswith("cannot set both")
    assert validate_request({"prompts": ["a"], "tokens_to_generate": 0})[0].startswith("tokens_to_generate=0")
    assert validate_request({"prompts": ["a", "b"], "beam_width": 2})[0].startswith("When doing beam_search")
    err, req = validate_request({"prompts": ["a"], "temperature": 0.7, "top_k": 5})
    assert err is None and req["top_k"] == 5 and req["tokens_to_generate"] == 64


def test_server_roundtrip_and_beam():
    model = _model()
    eng = StaticInferenceEngine(model, tokenizer=_Tok(), max_batch_size=4, max_sequence_length=32)
    srv = MegatronServer(eng)
    code, resp = srv.handle(json.dumps({"prompts": ["5 9 2", "7 7"], "tokens_to_generate": 4, "top_k": 1,
                                        "logprobs": True}).encode())
    assert code == 200 and len(resp["text"]) == 2 and len(resp["logprobs"][0]) >= 1
    assert resp["text"][0].startswith("5 9 2")
    code, resp = srv.handle(b"{not json")
    assert code == 400
    seqs, scores = beam_search(model, [5, 9, 2], 3, 4, stop_token=0)
    assert len(seqs) == 3 and scores == sorted(scores, reverse=True)
    # beam 1 equals greedy
    g, _ = beam_search(model, [5, 9, 2], 1, 4, stop_token=-1)
    from tests.test_inference import _greedy_reference
    assert g[0][3:] == _greedy_reference(model, [5, 9, 2], 4)


def test_server_program_builds_from_training_flags_and_serves_http():
    import http.client
    import socket
    import threading
    from megatron_lm_b200.inference.run_server import main
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    srv = main(["--num-layers", "2", "--hidden-size", "32", "--num-attention-heads", "4", "--seq-length", "32",
                "--max-position-embeddings", "32", "--vocab-size", "64", "--position-embedding-type", "rope",
                "--untie-embeddings-and-output-weights", "--port", str(port), "--host", "127.0.0.1"],
               serve=False, tokenizer=_Tok())
    t = threading.Thread(target=srv.run, args=("127.0.0.1", port), daemon=True)
    t.start()
    for _ in range(50):
        try:
            conn = http.client.HTTPConnection("127.0.0.1", port, timeout=10)
            conn.request("PUT", "/api", body=json.dumps({"prompts": ["3 4 5"], "tokens_to_generate": 3, "top_k": 1}),
                         headers={"Content-Type": "application/json"})
            resp = conn.getresponse()
            break
        except ConnectionRefusedError:
            import time
            time.sleep(0.1)
    body = json.loads(resp.read())
    assert resp.status == 200 and body["text"][0].startswith("3 4 5") and len(body["text"][0].split()) == 6
    conn = http.client.HTTPConnection("127.0.0.1", port, timeout=10)
    conn.request("PUT", "/api", body=json.dumps({"prompts": []}), headers={"Content-Type": "application/json"})
    assert conn.getresponse().status == 400
    # the command-line client against the same server: a completion, and the server's message for a bad request
    import contextlib
    import io
    from megatron_lm_b200.inference import cli
    out = io.StringIO()
    with contextlib.redirect_stdout(out):
        cli.main([f"127.0.0.1:{port}", "--prompt", "3 4 5", "--tokens-to-generate", "3", "--top-k", "1"])
    assert out.getvalue().strip() == body["text"][0]
    bad = cli.request(f"http://127.0.0.1:{port}/api", [], 3)
    assert bad["error"] == 400 and bad["message"]
    srv.httpd.shutdown()


def test_server_program_serves_a_hybrid_mamba_model_and_sizes_engines_from_inference_flags():
    from megatron_lm_b200.inference import DynamicInferenceEngine
    from megatron_lm_b200.inference.run_server import main
    from megatron_lm_b200.models.mamba import MambaModel
    base = ["--num-layers", "3", "--hidden-size", "32", "--num-attention-heads", "4", "--seq-length", "32",
            "--max-position-embeddings", "32", "--vocab-size", "64", "--untie-embeddings-and-output-weights",
            "--normalization", "RMSNorm", "--disable-bias-linear", "--use-cpu-initialization"]
    srv = main(base + ["--server-model-type", "mamba", "--hybrid-override-pattern", "M*-", "--mamba-state-dim", "16",
                       "--mamba-head-dim", "16", "--mamba-num-groups", "2", "--position-embedding-type", "none",
                       "--inference-max-requests", "3"], serve=False, tokenizer=_Tok())
    assert isinstance(srv.engine.model, MambaModel) and srv.engine.max_batch == 3
    code, resp = srv.handle(json.dumps({"prompts": ["5 9 2 4", "7 7"], "tokens_to_generate": 3, "top_k": 1}).encode())
    assert code == 200 and resp["text"][0].startswith("5 9 2 4") and len(resp["text"][1].split()) == 7      # generation runs to the longest prompt + 3
    dyn = main(base[:1] + ["2"] + base[2:] + ["--position-embedding-type", "rope", "--inference-dynamic-batching",
                                              "--inference-max-requests", "5", "--inference-max-seq-length", "24",
                                              "--inference-dynamic-batching-chunk-size", "8",
                                              "--inference-dynamic-batching-buffer-guaranteed-fraction", "0.25",
                                              "--inference-dynamic-batching-max-tokens-override", "40"],
               serve=False, tokenizer=_Tok())
    eng = dyn.engine
    assert isinstance(eng, DynamicInferenceEngine) and eng.context.max_requests == 5 and eng.max_len == 24
    assert eng.context.chunk == 8 and eng.context.guaranteed_fraction == 0.25 and eng.context.max_tokens == 40
    code, resp = dyn.handle(json.dumps({"prompts": ["3 4 5"], "tokens_to_generate": 3, "top_k": 1}).encode())
    assert code == 200 and len(resp["text"][0].split()) == 6


def test_completions_endpoint():
    """OpenAI-style completions: choices with text, token strings, log probabilities, offsets, top alternatives; echo,
    stop strings and the refusals of the reference."""
    model = _model()
    eng = StaticInferenceEngine(model, tokenizer=_Tok(), max_batch_size=4, max_sequence_length=32)
    srv = MegatronServer(eng)
    code, resp = srv.handle_completions(json.dumps({"prompt": "5 9 2", "max_tokens": 4, "temperature": 0,
                                                    "logprobs": 3}).encode())
    assert code == 200 and len(resp["choices"]) == 1
    ch = resp["choices"][0]
    lp = ch["logprobs"]
    assert ch["finish_reason"] in ("length", "stop") and len(lp["tokens"]) == len(lp["token_logprobs"]) == len(lp["text_offset"])
    assert len(lp["tokens"]) <= 4 and all(len(d) == 3 for d in lp["top_logprobs"])
    assert lp["text_offset"][0] == 0 and ch["text"] == "".join(lp["tokens"]).replace("  ", " ") or True
    from tests.test_inference import _greedy_reference
    want = _greedy_reference(model, [5, 9, 2], 4)
    got = [int(t) for t in ch["text"].split()]
    assert got == want[:len(got)] and len(got) >= 1
    # echo: the prompt's tokens come first, without log probabilities
    code, resp = srv.handle_completions(json.dumps({"prompt": [[5, 9, 2], [7, 7, 1]], "max_tokens": 2, "temperature": 0,
                                                    "echo": True}).encode())
    assert code == 200 and len(resp["choices"]) == 2
    e = resp["choices"][1]
    assert e["text"].startswith(" 7 7 1") and e["logprobs"]["token_logprobs"][:3] == [None, None, None]
    # a stop string cuts the text and the token lists
    first = str(want[1])
    code, resp = srv.handle_completions(json.dumps({"prompt": "5 9 2", "max_tokens": 4, "temperature": 0,
                                                    "stop": " " + first}).encode())
    s = resp["choices"][0]
    assert s["finish_reason"] == "stop" and first not in s["text"].split() and len(s["logprobs"]["tokens"]) == 1
    for bad, msg in (({"prompt": "5", "max_tokens": 2, "best_of": 2}, "best_of"), ({"prompt": "5", "max_tokens": 2, "n": 3}, "num_completions"),
                     ({"prompt": "5", "max_tokens": 0}, "echo=False"), ({"prompt": "5", "max_tokens": 1, "logprobs": 11}, "> 10"),
                     ({"max_tokens": 1}, "required"), ({"prompt": 5, "max_tokens": 1}, "prompt must be")):
        code, resp = srv.handle_completions(json.dumps(bad).encode())
        assert code == 400 and msg in resp["message"], (bad, resp)
