"""Chat with a running server through its OpenAI-compatible route, with nothing but ``requests``.

    mstar serve qwen3_omni --port 8000        # or tiny / higgs_audio / bagel ...
    python examples/openai_chat.py "What is in this picture?" --image cat.png
"""
import argparse
import base64
import json
import mimetypes

import requests


def data_url(path: str) -> str:
    mime = mimetypes.guess_type(path)[0] or "application/octet-stream"
    with open(path, "rb") as f:
        return f"data:{mime};base64,{base64.b64encode(f.read()).decode()}"


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("prompt")
    ap.add_argument("--base-url", default="http://127.0.0.1:8000")
    ap.add_argument("--image")
    ap.add_argument("--max-tokens", type=int, default=128)
    a = ap.parse_args()
    content = [{"type": "text", "text": a.prompt}]
    if a.image:
        content.append({"type": "image_url", "image_url": {"url": data_url(a.image)}})
    body = {"model": "default", "stream": True, "max_tokens": a.max_tokens,
            "messages": [{"role": "user", "content": content}]}
    with requests.post(f"{a.base_url}/v1/chat/completions", json=body, stream=True, timeout=600) as r:
        r.raise_for_status()
        for line in r.iter_lines():
            if not line.startswith(b"data: ") or line == b"data: [DONE]":
                continue
            delta = json.loads(line[6:])["choices"][0]["delta"]
            if delta.get("content"):
                print(delta["content"], end="", flush=True)
    print()


if __name__ == "__main__":
    main()
