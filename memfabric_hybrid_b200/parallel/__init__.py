"""Parallelism helpers on top of the zbal backend: mesh and bring-up (``mesh``), data-parallel gradient
reduction (``dp``), pipeline stage links (``pp``); tensor and expert parallelism are the fused kernels of
``ops.tp.TensorParallel`` and ``ops.moe.MoEComm`` (re-exported here)."""
from .dp import GradReducer  # noqa: F401
from .mesh import Context, Mesh, init, shutdown  # noqa: F401
from .pp import StageLink  # noqa: F401


def __getattr__(name):
    if name == "TensorParallel":
        from ..ops.tp import TensorParallel
        return TensorParallel
    if name == "MoEComm":
        from ..ops.moe import MoEComm
        return MoEComm
    raise AttributeError(name)
