"""Python SDK: text to speech, saved as WAV.

    mstar serve orpheus --port 8000
    python examples/sdk_tts.py "Hello from the SDK." -o hello.wav
"""
import argparse

from mstar_b200.client import MStarClient


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("text")
    ap.add_argument("-o", "--out", default="speech.wav")
    ap.add_argument("--voice", default="tara")
    a = ap.parse_args()
    audio = MStarClient("http://127.0.0.1:8000").tts(a.text, voice=a.voice)
    audio.to_wav(a.out)
    print(f"wrote {a.out}: {len(audio.to_numpy())} samples at {audio.sample_rate} Hz")


if __name__ == "__main__":
    main()
