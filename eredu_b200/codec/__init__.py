"""Neural audio codecs (the speech side of realtime models)."""
from .mimi import Mimi, MimiConfig

__all__ = ["Mimi", "MimiConfig"]
