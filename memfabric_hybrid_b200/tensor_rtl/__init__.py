"""Tensor resharding between parallel layouts (training TP/EP layout -> serving layout, expert migration):
plans in ``plan``, executors in ``executor``. Parity: app/tensorRTL/src/tensor_rtl/__init__.py of the reference."""
from .abc import BaseCommTask, Executor, Planner  # noqa: F401
from .buffer_pool import BufferPool  # noqa: F401
from .executor import All2AllVExcutor, All2AllVExecutor, BatchP2PExecutor, MemoryFabricExecutor, MfBmConfig  # noqa: F401
from .utils import get_dtype_size  # noqa: F401
from .pack import pack_tensors, unpack_tensors  # noqa: F401
from .plan import MFCommTask, P2PCommTask, PTensor, PTensorSet, overlaps, shard_bounds  # noqa: F401
from .eplb import ExpertMigrator, balanced_placement, pair_slots, remap_topk, replica_table  # noqa: F401
from .rl_reshard import InferLayout, ParamSpec, TrainLayout, TrainToInferResharder, decoder_specs  # noqa: F401
