"""Public facade: load a model, generate tokens, chat."""
from .loaded import LoadedModel, ModelLoadOptions, QuantizationOptions  # noqa: F401
from .inspection import inspect_text_model  # noqa: F401,E402
