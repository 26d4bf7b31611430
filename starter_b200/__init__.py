"""starter_b200: a small Qwen3 model library with generation of its own, for one B200."""

from . import models  # noqa: F401  (registers the architectures)

__version__ = "0.1.0"
