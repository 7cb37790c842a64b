"""DeepSeek-V3-shaped MoE layer with expert parallelism over the symmetric heap.

Router: softmax over `experts` logits, top-k (k = 8), weights renormalised over the chosen experts.
Experts: SwiGLU FFN (hidden -> 2 x intermediate -> hidden) in fp8 e4m3, activations scaled per 1 x 128,
weights per 128 x 128 block, random-init N(0, 0.02). Rank r owns experts [r * E/W, (r + 1) * E/W)."""
from __future__ import annotations

import torch

from ..ops import moe as M


class ExpertParallelMoE:
    def __init__(self, heap, hidden: int = 7168, intermediate: int = 2048, experts: int = 256, topk: int = 8,
                 max_tokens: int = 4096, max_recv: int | None = None, seed: int = 0):
        self.world, self.rank = heap.world, heap.rank
        self.hidden, self.inter, self.experts, self.topk = hidden, intermediate, experts, topk
        self.el = experts // self.world
        dev = torch.device("cuda", torch.cuda.current_device())
        self.w1, self.w2 = self.make_weights(self.rank, seed, dev)
        w1q, self.w1s = M.quantize_weight_fp8(self.w1)
        self.w1q = M.interleave_gate_up_fp8(w1q)
        self.w2q, self.w2s = M.quantize_weight_fp8(self.w2)
        self.comm = M.MoEComm(heap, max_tokens, hidden, experts, topk, max_recv, intermediate)

    def make_weights(self, rank: int, seed: int, dev):
        """bf16 master weights of the experts a rank owns (any rank can regenerate any other rank's)."""
        g = torch.Generator(device=dev).manual_seed(seed * 7919 + rank)
        w1 = (torch.randn(self.el, 2 * self.inter, self.hidden, device=dev, generator=g) * 0.02).to(torch.bfloat16)
        w2 = (torch.randn(self.el, self.hidden, self.inter, device=dev, generator=g) * 0.02).to(torch.bfloat16)
        return w1, w2

    @staticmethod
    def route(logits: torch.Tensor, topk: int):
        p = torch.softmax(logits.float(), dim=-1)
        w, idx = torch.topk(p, topk, dim=-1)
        return idx.to(torch.int32), (w / w.sum(-1, keepdim=True)).float()

    def forward(self, x: torch.Tensor, logits: torch.Tensor) -> torch.Tensor:
        idx, w = self.route(logits, self.topk)
        st = self.comm.dispatch(x, idx, w)
        self.comm.expert_ffn(st, self.w1q, self.w1s, self.w2q, self.w2s)
        return self.comm.combine(st)
