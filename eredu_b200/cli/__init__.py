"""Command-line front end (``python -m eredu_b200.cli``)."""
from .main import build_parser, main  # noqa: F401
