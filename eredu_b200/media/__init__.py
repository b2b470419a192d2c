"""Model-independent media preprocessing: RGB image resize / normalisation, log-mel audio features, video frame
sampling (counterparts of eredu/src/backend/mlx/runtime/media/{image,audio,video}.rs and the value types of
eredu-core/src/media.rs). Everything here is host-side numpy: the outputs are the typed tensors a multimodal model's
input pipeline uploads."""
from .audio import AudioWaveform, LogMelConfig, LogMelFeatures, extract_log_mel
from .image import NormalizedImage, RgbImage, load_image, rescale_and_normalize_rgb8, resize_rgb8_bicubic, resize_rgb8_lanczos3
from .request import (MultimodalPreparationError, MultimodalRequest, TokenizedSegment, Video, prepare_for_text_model)
from .video import (format_mm_ss, frame_timestamps, pad_frame_indices, sampled_frame_count, temporal_group_timestamps,
                    uniform_sample_indices, validate_rgb_frames)

__all__ = ["load_image", "AudioWaveform", "LogMelConfig", "LogMelFeatures", "extract_log_mel", "NormalizedImage", "RgbImage",
           "rescale_and_normalize_rgb8", "resize_rgb8_bicubic", "resize_rgb8_lanczos3", "format_mm_ss", "frame_timestamps",
           "pad_frame_indices", "sampled_frame_count", "temporal_group_timestamps", "uniform_sample_indices",
           "validate_rgb_frames", "MultimodalPreparationError", "MultimodalRequest", "TokenizedSegment", "Video",
           "prepare_for_text_model"]
