"""Tensor resharding between parallel layouts (training TP/EP layout -> serving layout, expert migration):
plans in ``plan``, executors in ``executor``. Parity: app/tensorRTL/src/tensor_rtl/__init__.py of the reference."""
from .executor import (All2AllVExcutor, All2AllVExecutor, BatchP2PExecutor, Executor, MemoryFabricExecutor, MfBmConfig,  # noqa: F401
                       Planner)
from .pack import pack_tensors, unpack_tensors  # noqa: F401
from .plan import MFCommTask, P2PCommTask, PTensor, PTensorSet, overlaps, shard_bounds  # noqa: F401
from .eplb import ExpertMigrator, balanced_placement, pair_slots, remap_topk, replica_table  # noqa: F401
from .rl_reshard import InferLayout, ParamSpec, TrainLayout, TrainToInferResharder, decoder_specs  # noqa: F401
