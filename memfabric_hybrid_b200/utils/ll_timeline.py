"""Device timeline of the low-latency MoE pair (one cooperative launch per direction) on N GPUs.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29531 \
        -m memfabric_hybrid_b200.utils.ll_timeline --out-dir out

Every rank writes ``ll_trace_<rank>.json`` (Chrome trace) and rank 0 prints, per phase, the number of events, the
median and the longest duration, and the (start, duration) pairs of CTA 0 in microseconds.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--out-dir", default=".")
    ap.add_argument("--tokens", type=int, default=128)
    ap.add_argument("--pairs", type=int, default=3)
    a = ap.parse_args()
    from ..models.deepseek_moe import ExpertParallelMoE
    from ..ops.heap import SymmetricHeap
    from . import devtrace
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl")
    heap = SymmetricHeap(f"127.0.0.1:{int(os.environ['MASTER_PORT']) + 41}", world, rank, local, 3 << 30)
    H, I, K, E, T = 7168, 2048, 8, 32 * world, a.tokens
    layer = ExpertParallelMoE(heap, H, I, E, K, max_tokens=T, max_recv=T * K * world, seed=1)
    g = torch.Generator("cuda").manual_seed(rank)
    x = torch.randn(T, H, device="cuda", generator=g).to(torch.bfloat16)
    idx, w = layer.route(torch.randn(T, E, device="cuda", generator=g), K)
    idx32, w32 = idx.to(torch.int32).contiguous(), w.float().contiguous()
    y = torch.zeros((layer.comm.max_recv, H), dtype=torch.bfloat16, device="cuda")   # stands in for the expert outputs
    out = torch.empty((T, H), dtype=torch.bfloat16, device="cuda")
    for _ in range(3):
        st = layer.comm.ll_dispatch(x, idx32, w32)
        layer.comm.ll_combine(y, st, out=out)
    torch.cuda.synchronize()
    dist.barrier()
    devtrace.enable(lanes=256, per_lane=64)
    for _ in range(a.pairs):
        dist.barrier()
        torch.cuda.synchronize()
        st = layer.comm.ll_dispatch(x, idx32, w32)
        layer.comm.ll_combine(y, st, out=out)
    torch.cuda.synchronize()
    path = os.path.join(a.out_dir, f"ll_trace_{rank}.json")
    devtrace.dump(path, rank=rank)
    if rank == 0:
        by = {}
        for e in json.load(open(path))["traceEvents"]:
            by.setdefault(e["name"], []).append((e["tid"], round(e["ts"], 1), round(e["dur"], 1)))
        for name, v in by.items():
            durs = sorted(d for _, _, d in v)
            print(name, "n", len(v), "median_us", durs[len(durs) // 2], "max_us", durs[-1], "cta0", [(ts, d) for tid, ts, d in v if tid == 0][:6],
                  flush=True)
    devtrace.disable()
    torch.cuda.synchronize()
    heap.close()
    SymmetricHeap.shutdown()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
