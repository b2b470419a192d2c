"""RGB8 images: validated views (row stride), separable resampling with Catmull-Rom and Lanczos-3 kernels (the filter
support widens with the down-scaling ratio, so shrinking is anti-aliased), rescale + per-channel normalisation to
channel-first float32 (eredu/src/backend/mlx/runtime/media/image.rs:9-250)."""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np


class MediaError(ValueError):
    pass


@dataclass
class RgbImage:
    pixels: np.ndarray   # uint8 [height, width, 3], tightly packed
    @property
    def width(self) -> int:
        return int(self.pixels.shape[1])

    @property
    def height(self) -> int:
        return int(self.pixels.shape[0])

    @classmethod
    def packed(cls, data, width: int, height: int) -> "RgbImage":
        return cls.with_row_stride(data, width, height, width * 3)

    @classmethod
    def with_row_stride(cls, data, width: int, height: int, row_stride: int) -> "RgbImage":
        """View over a byte buffer whose rows are ``row_stride`` bytes apart (padding after each row is dropped)."""
        if width <= 0 or height <= 0:
            raise MediaError(f"image dimensions must be positive, got {width}x{height}")
        if row_stride < width * 3:
            raise MediaError(f"row stride {row_stride} is shorter than a row of {width} RGB pixels")
        buf = np.frombuffer(bytes(data), dtype=np.uint8) if not isinstance(data, np.ndarray) else data.reshape(-1).astype(np.uint8)
        need = (height - 1) * row_stride + width * 3
        if buf.size < need:
            raise MediaError(f"pixel buffer holds {buf.size} bytes, {need} needed")
        rows = [buf[y * row_stride:y * row_stride + width * 3] for y in range(height)]
        return cls(np.stack(rows).reshape(height, width, 3).copy())


@dataclass
class NormalizedImage:
    data: np.ndarray     # float32 [3, height, width]

    @property
    def channels(self) -> int:
        return int(self.data.shape[0])

    @property
    def height(self) -> int:
        return int(self.data.shape[1])

    @property
    def width(self) -> int:
        return int(self.data.shape[2])

    def get(self, channel: int, y: int, x: int) -> float:
        return float(self.data[channel, y, x])


def _catmull_rom(x):
    x = np.abs(x)
    a = -0.5
    return np.where(x < 1, (a + 2) * x ** 3 - (a + 3) * x ** 2 + 1,
                    np.where(x < 2, a * x ** 3 - 5 * a * x ** 2 + 8 * a * x - 4 * a, 0.0))


def _lanczos3(x):
    x = np.abs(x)
    return np.where(x < 3, np.sinc(x) * np.sinc(x / 3), 0.0)


def _weights(src: int, dst: int, kernel, support: float) -> np.ndarray:
    """Row-stochastic resampling matrix [dst, src]: output sample i is centred at (i + 0.5) * src / dst and the
    kernel is stretched by the ratio when shrinking."""
    ratio = src / dst
    scale = max(ratio, 1.0)
    centres = (np.arange(dst) + 0.5) * ratio
    pos = np.arange(src) + 0.5
    w = kernel((pos[None, :] - centres[:, None]) / scale)
    w[np.abs(pos[None, :] - centres[:, None]) > support * scale] = 0.0
    s = w.sum(1, keepdims=True)
    return (w / np.where(s == 0, 1.0, s)).astype(np.float64)


def _resize(image: RgbImage, width: int, height: int, kernel, support: float) -> RgbImage:
    if width <= 0 or height <= 0:
        raise MediaError(f"resize dimensions must be positive, got {width}x{height}")
    if width == image.width and height == image.height:
        return RgbImage(image.pixels.copy())
    x = image.pixels.astype(np.float64)
    # rows first (vertical pass), clamped and rounded between the passes like an 8-bit intermediate image
    wy = _weights(image.height, height, kernel, support)
    x = np.clip(np.rint(np.einsum("oh,hwc->owc", wy, x)), 0, 255)
    wx = _weights(image.width, width, kernel, support)
    x = np.clip(np.rint(np.einsum("ow,hwc->hoc", wx, x)), 0, 255)
    return RgbImage(x.astype(np.uint8))


def resize_rgb8_bicubic(image: RgbImage, width: int, height: int) -> RgbImage:
    return _resize(image, width, height, _catmull_rom, 2.0)


def resize_rgb8_lanczos3(image: RgbImage, width: int, height: int) -> RgbImage:
    return _resize(image, width, height, _lanczos3, 3.0)


def rescale_and_normalize_rgb8(image: RgbImage, rescale_factor: float, mean, std) -> NormalizedImage:
    """(pixel * rescale_factor - mean[c]) / std[c], channel-first."""
    if not np.isfinite(rescale_factor):
        raise MediaError(f"image rescale factor must be finite, got {rescale_factor}")
    std = np.asarray(std, dtype=np.float32)
    mean = np.asarray(mean, dtype=np.float32)
    if std.shape != (3,) or mean.shape != (3,) or np.any(std == 0) or not np.all(np.isfinite(std)):
        raise MediaError(f"image normalisation needs three finite non-zero standard deviations, got {std.tolist()}")
    x = image.pixels.astype(np.float32) * np.float32(rescale_factor)
    return NormalizedImage(np.ascontiguousarray(((x - mean) / std).transpose(2, 0, 1)))


def load_image(path) -> RgbImage:
    """Decode an image file to RGB8 (needs Pillow; formats are whatever it reads)."""
    try:
        from PIL import Image
    except ImportError as e:  # pragma: no cover
        raise MediaError("decoding image files needs the Pillow package") from e
    with Image.open(path) as im:
        return RgbImage(np.asarray(im.convert("RGB"), dtype=np.uint8).copy())
