"""pulsar_b200: a small, whole inference engine for one B200 (sm_100a)."""
from . import models as _models  # noqa: F401  (registers the built-in architectures and parts)

__version__ = "0.1.0"
