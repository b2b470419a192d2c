"""Typed multimodal request values (eredu-core/src/media.rs:62-370): an ordered list of text / image / audio / video
parts, and the segments a processor turns them into (token ids, or a placeholder run that a tower's embeddings
replace). Text-only models refuse non-text parts with a preparation error instead of ignoring them
(eredu/src/api/media.rs)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Union

from .audio import AudioWaveform
from .image import MediaError, RgbImage


@dataclass
class Video:
    frames: list            # list[RgbImage]
    fps: float

    def __post_init__(self):
        from .video import validate_rgb_frames

        validate_rgb_frames(self.frames)
        if not (self.fps > 0):
            raise MediaError(f"video FPS must be positive, got {self.fps}")


Part = Union[str, RgbImage, AudioWaveform, Video]


@dataclass
class MultimodalRequest:
    parts: list = field(default_factory=list)

    def text(self, s: str) -> "MultimodalRequest":
        self.parts.append(str(s))
        return self

    def image(self, im: RgbImage) -> "MultimodalRequest":
        self.parts.append(im)
        return self

    def audio(self, a: AudioWaveform) -> "MultimodalRequest":
        self.parts.append(a)
        return self

    def video(self, v: Video) -> "MultimodalRequest":
        self.parts.append(v)
        return self

    def modalities(self) -> set:
        kinds = {str: "text", RgbImage: "image", AudioWaveform: "audio", Video: "video"}
        return {kinds[type(p)] for p in self.parts}


@dataclass
class TokenizedSegment:
    kind: str                               # text | image | audio | video
    token_ids: list                         # text: the tokens; media: the placeholder ids that reserve the positions
    features: Optional[object] = None       # media: the processor output the tower consumes


class MultimodalPreparationError(MediaError):
    pass


def prepare_for_text_model(request: MultimodalRequest, encode) -> list[TokenizedSegment]:
    """Segments of a request for a model without media towers: any non-text part is an error."""
    extra = request.modalities() - {"text"}
    if extra:
        raise MultimodalPreparationError(f"this model accepts text only; the request carries {sorted(extra)}")
    return [TokenizedSegment("text", list(encode(p))) for p in request.parts]
