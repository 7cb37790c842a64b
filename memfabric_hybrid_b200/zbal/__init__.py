"""zbal: symmetric-heap allocator, ``torch.distributed`` backend "zbal", and the DeepEP-style MoE ``Buffer``.

Importing this package registers the process-group backend. Public names follow the reference's Python
package (app/zbal/src/python/zbal/__init__.py:34-61).
"""
from .module import (ZBALBootstrapType, __version__, dump_snapshot, empty_cache, expand_heap, get_heap_stats, heap_stats, in_symmetric_heap,  # noqa: F401
                     is_initialized, is_mix_alloc, mem_get_info, memviz_snapshot, record_memory_history, simulate_init, snapshot, switch_to_allocator,
                     symmetric_tensors, zbal_get_symm_base_addr, zbal_init, zbal_set_logger_level, zbal_uninit)
from .process_group import ProcessGroupZBAL, WorkZBAL, register  # noqa: F401
from .utils import Config, EventOverlap  # noqa: F401

register()


def __getattr__(name):
    if name == "Buffer":
        from .buffer import Buffer
        return Buffer
    raise AttributeError(name)


__all__ = ["switch_to_allocator", "zbal_get_symm_base_addr", "record_memory_history", "dump_snapshot", "get_heap_stats", "zbal_init",
           "zbal_uninit", "ZBALBootstrapType", "zbal_set_logger_level", "simulate_init", "is_mix_alloc", "mem_get_info", "Buffer",
           "Config", "EventOverlap", "ProcessGroupZBAL", "__version__"]
