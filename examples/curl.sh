#!/usr/bin/env bash
# Talk to a running server with curl.   mstar serve orpheus --port 8000   (or any other model)
set -euo pipefail
BASE=${BASE:-http://127.0.0.1:8000}

curl -s "$BASE/health"; echo
curl -s "$BASE/v1/models"; echo

# native endpoint: multipart form, NDJSON stream of {"modality", "data" (base64), "metadata"}
curl -sN "$BASE/generate" -F text="hello there" -F output_modalities=text -F streaming=true \
     -F model_kwargs='{"max_tokens": 32, "temperature": 0.7}'; echo

# OpenAI-compatible chat (server-sent events)
curl -sN "$BASE/v1/chat/completions" -H 'Content-Type: application/json' \
     -d '{"model": "default", "stream": true, "max_tokens": 32, "messages": [{"role": "user", "content": "hi"}]}'; echo

# OpenAI-compatible speech: streamed WAV to a file (TTS models)
curl -s "$BASE/v1/audio/speech" -H 'Content-Type: application/json' \
     -d '{"model": "default", "input": "hello from the command line", "voice": "tara", "response_format": "wav"}' \
     -o speech.wav && echo "wrote speech.wav"
