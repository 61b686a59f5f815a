"""Python SDK: text-to-image (BAGEL, Cosmos3).

    mstar serve bagel --port 8000
    python examples/sdk_image.py "a lighthouse at dusk" -o lighthouse.png
"""
import argparse

from mstar_b200.client import MStarClient


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("prompt")
    ap.add_argument("-o", "--out", default="image.png")
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--size", default="1024x1024")
    a = ap.parse_args()
    w, h = (int(x) for x in a.size.lower().split("x"))
    png = MStarClient("http://127.0.0.1:8000").generate_image(a.prompt, num_steps=a.steps, width=w, height=h)
    with open(a.out, "wb") as f:
        f.write(png)
    print(f"wrote {a.out} ({len(png)} bytes)")


if __name__ == "__main__":
    main()
