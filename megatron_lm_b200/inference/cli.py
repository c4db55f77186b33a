"""Command-line client of the text generation server: sends ``PUT /api`` requests and prints the completions
(reference: tools/text_generation_cli.py).

    python -m megatron_lm_b200.inference.cli localhost:5000                    # interactive
    python -m megatron_lm_b200.inference.cli localhost:5000 --prompt "Hello" --tokens-to-generate 32
"""
from __future__ import annotations

import argparse
import json
import urllib.error
import urllib.request


def request(url: str, prompts, tokens_to_generate: int, timeout: float = 300.0, **extra) -> dict:
    """One request; returns the decoded JSON body, or ``{"error": status, "message": ...}``."""
    body = json.dumps({"prompts": list(prompts), "tokens_to_generate": int(tokens_to_generate), **extra}).encode()
    req = urllib.request.Request(url, data=body, method="PUT", headers={"Content-Type": "application/json"})
    try:
        with urllib.request.urlopen(req, timeout=timeout) as r:
            return json.loads(r.read().decode())
    except urllib.error.HTTPError as e:
        try:
            msg = json.loads(e.read().decode()).get("message", "")
        except Exception:
            msg = str(e)
        return {"error": e.code, "message": msg}


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("address", help="host:port of the server")
    ap.add_argument("--prompt", action="append", default=None, help="send these prompts once instead of asking")
    ap.add_argument("--tokens-to-generate", type=int, default=64)
    ap.add_argument("--temperature", type=float, default=None)
    ap.add_argument("--top-k", type=int, default=None)
    ap.add_argument("--top-p", type=float, default=None)
    a = ap.parse_args(argv)
    url = a.address if a.address.startswith("http") else "http://" + a.address
    url = url.rstrip("/") + "/api"
    extra = {k: v for k, v in (("temperature", a.temperature), ("top_k", a.top_k), ("top_p", a.top_p)) if v is not None}

    def show(res):
        if "error" in res:
            print(f"Error {res['error']}: {res['message']}")
        else:
            for t in res.get("text", []):
                print(t)

    if a.prompt:
        show(request(url, a.prompt, a.tokens_to_generate, **extra))
        return
    while True:
        try:
            sentence = input("Enter prompt: ")
            n = int(input("Enter number of tokens to generate: ") or a.tokens_to_generate)
        except (EOFError, KeyboardInterrupt):
            print()
            return
        show(request(url, [sentence], n, **extra))


if __name__ == "__main__":
    main()
