"""leone_b200: a single-GPU inference engine for NVIDIA B200 (sm_100a)."""
from . import models as _models  # noqa: F401  (registers built-in architectures)
from . import parts as _parts    # noqa: F401  (registers built-in parts)

__version__ = "0.1.0"


def generate(*args, **kwargs):
    from .engine.generate import generate as _generate
    return _generate(*args, **kwargs)


__all__ = ["generate", "__version__"]
