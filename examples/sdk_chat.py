"""Python SDK: blocking and streaming text generation.

    mstar serve tiny --port 8000
    python examples/sdk_chat.py "1 2 3 4"
"""
import sys

from mstar_b200.client import MStarClient


def main():
    prompt = sys.argv[1] if len(sys.argv) > 1 else "hello"
    client = MStarClient("http://127.0.0.1:8000")
    print("health:", client.health())
    res = client.generate(prompt, max_tokens=32, temperature=0.7)
    print("blocking :", res.text)
    print("streaming: ", end="")
    for chunk in client.stream(prompt, max_tokens=32, temperature=0.7):
        print(getattr(chunk, "text", ""), end="", flush=True)
    print()


if __name__ == "__main__":
    main()
