"""kungfu_b200: a one-GPU inference engine for Gemma 2 on B200 (sm_100a), built from parts."""
__version__ = "0.1.0"

from .api import Engine, load_model  # noqa: E402,F401
