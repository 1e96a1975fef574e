"""delta_b200: a single-GPU inference engine for the Yi architecture with DELTA's
selective cache, written for B200 (sm_100a)."""
from . import models  # noqa: F401  (registers the architectures)
from .config import EngineConfig, SelectiveCacheConfig, YiConfig

__all__ = ["EngineConfig", "SelectiveCacheConfig", "YiConfig"]


def __getattr__(name):
    # the engine pulls in the CUDA library; import it on first use
    if name in ("LMBackend", "ModelRunner", "RowInput"):
        from . import engine
        return getattr(engine, name)
    raise AttributeError(name)
