"""Drop-in name of the reference's tensorRTL wheel: ``import tensor_rtl``."""
from memfabric_hybrid_b200.tensor_rtl import *  # noqa: F401,F403
