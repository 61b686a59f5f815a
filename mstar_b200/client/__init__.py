from .client import MStarClient
from .types import AudioBuffer, AudioChunk, GenerateResult, ImageChunk, TextChunk, VideoChunk

__all__ = ["MStarClient", "AudioBuffer", "AudioChunk", "GenerateResult", "ImageChunk", "TextChunk", "VideoChunk"]
