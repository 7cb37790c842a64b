"""Drop-in name of the reference's zbal wheel: ``import zbal``."""
from memfabric_hybrid_b200.zbal import *  # noqa: F401,F403
from memfabric_hybrid_b200.zbal import __version__, heap_stats, snapshot, empty_cache  # noqa: F401


def __getattr__(name):
    import memfabric_hybrid_b200.zbal as _z
    return getattr(_z, name)
