"""memfabric_hybrid_b200: a Blackwell-native memory fabric.

Pools the HBM of every GPU of an NVSwitch domain plus pinned host DRAM into one global virtual
address space identical in every process, and moves / reduces data on it with sm_100a kernels.

    api        the reference-compatible Python surface (also importable as ``memfabric_hybrid``)
    ops        kernels: xcopy, collectives, MoE dispatch/combine, grouped GEMM, fused TP GEMMs
    parallel   torch.distributed backend, expert / tensor / pipeline parallel helpers
    models     DeepSeek-V3-shaped MoE layer, Llama-3-70B-shaped TP MLP
    zbal       allocator + collectives + DeepEP-style Buffer on the symmetric heap
    tensor_rtl tensor resharding planner and executors
"""
__version__ = "0.1.0"
