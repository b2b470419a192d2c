"""Public facade: load a model, generate tokens, chat."""
from .loaded import LoadedModel, ModelLoadOptions, QuantizationOptions  # noqa: F401
