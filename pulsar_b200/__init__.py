"""pulsar_b200: a small, whole inference engine for one B200 (sm_100a)."""
from . import models as _models  # noqa: F401  (registers the built-in architectures and parts)

__version__ = "0.1.0"


def __getattr__(name):
    # Lazy: the engine pulls in the CUDA library's loader only when it is used.
    if name in ("Pulsar", "Session", "generate"):
        from . import api
        return getattr(api, name)
    if name in ("AsyncPulsar", "AsyncSession"):
        from . import aio
        return getattr(aio, name)
    if name in ("Engine",):
        from .engine.engine import Engine
        return Engine
    raise AttributeError(name)
