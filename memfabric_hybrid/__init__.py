"""Drop-in name of the reference's Python wheel: ``import memfabric_hybrid as mf``."""
from memfabric_hybrid_b200.api import *  # noqa: F401,F403
from memfabric_hybrid_b200.api import bm, shm, TransferEngine  # noqa: F401
