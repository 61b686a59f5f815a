"""Text to speech through the OpenAI-compatible route: the WAV is written while it streams in.

    mstar serve orpheus --port 8000
    python examples/openai_tts.py "Streaming speech from a B200." -o out.wav
"""
import argparse

import requests


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("text")
    ap.add_argument("-o", "--out", default="speech.wav")
    ap.add_argument("--base-url", default="http://127.0.0.1:8000")
    ap.add_argument("--voice", default="tara")
    a = ap.parse_args()
    body = {"model": "default", "input": a.text, "voice": a.voice, "response_format": "wav", "stream": True}
    n = 0
    with requests.post(f"{a.base_url}/v1/audio/speech", json=body, stream=True, timeout=600) as r, open(a.out, "wb") as f:
        r.raise_for_status()
        for chunk in r.iter_content(chunk_size=None):
            f.write(chunk)
            n += len(chunk)
    print(f"wrote {a.out} ({n} bytes)")


if __name__ == "__main__":
    main()
