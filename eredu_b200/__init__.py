"""eredu_b200: a Blackwell-native LLM inference runtime (PyTorch + hand-written sm_100a kernels)."""
__version__ = "0.1.0"
