"""Video frame selection helpers (eredu/src/backend/mlx/runtime/media/video.rs:6-140): frame validation, uniform
sampling with round-half-even positions, rate-derived frame counts, timestamps, temporal padding and grouping."""
from __future__ import annotations

import math

from .image import MediaError, RgbImage


def validate_rgb_frames(frames: list[RgbImage]) -> tuple[int, int]:
    if not frames:
        raise MediaError("video must contain at least one frame")
    w, h = frames[0].width, frames[0].height
    for i, f in enumerate(frames):
        if (f.width, f.height) != (w, h):
            raise MediaError(f"video frame {i} is {f.width}x{f.height}, expected {w}x{h}")
    return w, h


def uniform_sample_indices(total_frames: int, sample_count: int) -> list[int]:
    if total_frames <= 0 or sample_count <= 0:
        raise MediaError(f"video sampling requires positive frame counts, got {total_frames} source and {sample_count} requested")
    n = min(sample_count, total_frames)
    if n == 1:
        return [0]
    last = total_frames - 1
    return [int(round(i * last / (n - 1))) for i in range(n)]     # Python's round() is round-half-even


def sampled_frame_count(total_frames: int, source_fps: float, target_fps: float, min_frames: int, max_frames: int) -> int:
    for name, v in (("source", source_fps), ("target", target_fps)):
        if not math.isfinite(v) or v <= 0:
            raise MediaError(f"video {name} FPS must be finite and positive, got {v}")
    if min_frames <= 0 or max_frames < min_frames:
        raise MediaError(f"video frame limits must be positive and ordered, got {min_frames}..{max_frames}")
    requested = int(total_frames / source_fps * target_fps)
    return max(min(max(requested, min_frames), max_frames, total_frames), 1)


def frame_timestamps(indices: list[int], source_fps: float) -> list[float]:
    if not math.isfinite(source_fps) or source_fps <= 0:
        raise MediaError(f"video source FPS must be finite and positive, got {source_fps}")
    return [i / source_fps for i in indices]


def format_mm_ss(timestamp: float) -> str:
    if not math.isfinite(timestamp) or timestamp < 0:
        raise MediaError(f"video timestamp must be finite and non-negative, got {timestamp}")
    s = int(math.floor(timestamp))
    return f"{s // 60:02d}:{s % 60:02d}"


def pad_frame_indices(indices: list[int], temporal_factor: int) -> list[int]:
    """Repeat the last frame until the count is a multiple of ``temporal_factor``."""
    if not indices or temporal_factor <= 0:
        raise MediaError("temporal frame padding requires frames and a positive factor")
    rem = len(indices) % temporal_factor
    return list(indices) + [indices[-1]] * ((temporal_factor - rem) % temporal_factor)


def temporal_group_timestamps(indices: list[int], source_fps: float, temporal_factor: int) -> list[float]:
    """One timestamp per group of ``temporal_factor`` frames: the mean of the group's first and last frame times."""
    if not math.isfinite(source_fps) or source_fps <= 0:
        raise MediaError(f"video source FPS must be finite and positive, got {source_fps}")
    if temporal_factor <= 0 or not indices or len(indices) % temporal_factor != 0:
        raise MediaError(f"{len(indices)} frame indices cannot be grouped by temporal factor {temporal_factor}")
    out = []
    for g in range(0, len(indices), temporal_factor):
        first, last = indices[g] / source_fps, indices[g + temporal_factor - 1] / source_fps
        out.append((first + last) / 2.0)
    return out
