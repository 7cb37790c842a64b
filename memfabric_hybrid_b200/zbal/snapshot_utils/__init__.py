"""Offline tools for allocator snapshots in the PyTorch memory-visualiser layout (``segments`` + ``device_traces``, what
``zbal.dump_snapshot()`` returns and what ``torch.cuda.memory._snapshot()`` pickles): an address-ordered model of the
trace, a replay through the symmetric-heap allocator, drawings (SVG, no plotting library needed) and a Chrome-trace export.
Parity of role and of names: app/zbal/simulator/python/snapshot_utils of the reference."""
from . import gva_layout_analyzer, gva_layout_viz, gva_snapshot_replay  # noqa: F401
from .gva_layout_analyzer import Block, MemoryAllocatorSimulator  # noqa: F401
from .gva_layout_viz import (parse_mem_to_profile, parser_file_ops, visualize_file_memory, visualize_file_snapshot,  # noqa: F401
                             visualize_sim_memory)
from .gva_snapshot_replay import replay_snapshot  # noqa: F401
