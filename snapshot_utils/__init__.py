"""Drop-in name of the reference's allocator snapshot tools: ``from snapshot_utils.gva_layout_analyzer import ...``."""
import sys as _sys

import memfabric_hybrid_b200.zbal.snapshot_utils as _p
from memfabric_hybrid_b200.zbal.snapshot_utils import *  # noqa: F401,F403

for _n in ("gva_layout_analyzer", "gva_snapshot_replay", "gva_layout_viz"):
    _sys.modules[__name__ + "." + _n] = getattr(_p, _n)
