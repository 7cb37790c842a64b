"""Llama-style tensor-parallel MLP: y = down( silu(gate(x)) * up(x) ), sequence-sharded in and out.

Fused path (this framework): all-gather of the sequence shards is fused into the gate/up GEMM (with the
SwiGLU in its epilogue), and the down projection GEMM is fused with the reduce-scatter.
Baseline path: NCCL all_gather + cuBLAS matmuls + NCCL reduce_scatter (what a stock PyTorch TP layer does).
Weights are random-init N(0, 0.02): rank r holds rows [r*F/W, (r+1)*F/W) of gate/up and the matching
columns of down."""
from __future__ import annotations

import torch

from ..ops import gemm
from ..ops.tp import TensorParallel


class TensorParallelMLP:
    def __init__(self, heap, hidden: int, ffn: int, max_tokens: int, seed: int = 0, dtype=torch.bfloat16, fp8: bool = False):
        self.world, self.rank = heap.world, heap.rank
        assert ffn % self.world == 0 and (ffn // self.world) % 128 == 0
        self.hidden, self.ffn, self.f_local = hidden, ffn, ffn // self.world
        g = torch.Generator("cuda").manual_seed(seed * 1000 + self.rank)
        dev = torch.device("cuda", torch.cuda.current_device())
        self.w_gate = (torch.randn(self.f_local, hidden, device=dev, generator=g) * 0.02).to(dtype)
        self.w_up = (torch.randn(self.f_local, hidden, device=dev, generator=g) * 0.02).to(dtype)
        self.w_down = (torch.randn(hidden, self.f_local, device=dev, generator=g) * 0.02).to(dtype)
        self.w_gate_up = gemm.interleave_gate_up(self.w_gate, self.w_up)
        self.tp = TensorParallel(heap, max_tokens, hidden, max_out=hidden, fp8=fp8)
        self.fp8 = fp8
        if fp8:
            # e4m3 weights with 128 x 128 power-of-two block scales; gate / up rows interleaved per 128 for the SwiGLU epilogue
            from ..ops import moe as M
            gu = torch.cat([self.w_gate, self.w_up])                      # [2 F/W, H], gate rows then up rows
            q, self.ws_gate_up = M.quantize_weight_fp8(gu)
            self.wq_gate_up = M.interleave_gate_up_fp8(q[None], 128)[0]
            self.wq_down, self.ws_down = M.quantize_weight_fp8(self.w_down)

    def forward_fp8(self, x_shard: torch.Tensor) -> torch.Tensor:
        """The same layer with fp8 tensor-core math: the shard is quantised on its way into the gather buffers, SwiGLU and
        the re-quantisation are the first GEMM's epilogue, the second GEMM's partial tiles are reduce-scattered in bf16."""
        hq, hs = self.tp.ag_gemm_fp8(x_shard, self.wq_gate_up, self.ws_gate_up)
        return self.tp.gemm_rs_fp8(hq, hs, self.wq_down, self.ws_down)

    def forward(self, x_shard: torch.Tensor) -> torch.Tensor:
        """x_shard [T/W, hidden] -> y_shard [T/W, hidden]."""
        h = self.tp.ag_gemm(x_shard, self.w_gate_up, swiglu=True)
        return self.tp.gemm_rs(h, self.w_down)

    def forward_baseline(self, x_shard: torch.Tensor) -> torch.Tensor:
        import torch.distributed as dist
        if self.world > 1:
            x = torch.empty((x_shard.shape[0] * self.world, self.hidden), dtype=x_shard.dtype, device=x_shard.device)
            dist.all_gather_into_tensor(x, x_shard.contiguous())
        else:
            x = x_shard
        h = torch.nn.functional.silu(x @ self.w_gate.t()) * (x @ self.w_up.t())
        y = h @ self.w_down.t()
        if self.world == 1:
            return y
        out = torch.empty((x_shard.shape[0], self.hidden), dtype=y.dtype, device=y.device)
        dist.reduce_scatter_tensor(out, y)
        return out
